from .engine import Engine, StepError
from .generate import GenerationError, Request, plan_batches, run_batch, run_generation
from .load import load_model, parse_dtype, random_model
from .model import Model, describe_config, expected_tensors
from .step import StepContext, Workspace

__all__ = ["Engine", "StepError", "GenerationError", "Request", "plan_batches", "run_batch", "run_generation",
           "load_model", "parse_dtype", "random_model", "Model", "describe_config", "expected_tensors",
           "StepContext", "Workspace"]
