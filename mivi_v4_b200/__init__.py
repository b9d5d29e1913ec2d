"""mivi_v4_b200: a small, whole model library for the LFM2 / LFM2.5 hybrid
decoder on one B200: from a model folder (config.json, model.safetensors) or
random weights to generated tokens, with hand-written sm_100a kernels, a true
32-bit path, and a trace replay program.

    from mivi_v4_b200 import Engine, SamplingParams, load_model
    engine = Engine(load_model("model_dir", dtype="bfloat16"), max_tokens=8192)
    new_tokens = engine.generate([[1, 2, 3], [4, 5]], max_new_tokens=32, sampling=SamplingParams.greedy())
"""
from .config import ConfigError, Lfm2Config, known_architectures, register_architecture
from .engine import Engine, GenerationError, Model, StepError, load_model, random_model
from .ops.kernels import KernelError
from .sampling import SamplingParams
from .weights import WeightsError, write_random_model

__all__ = ["ConfigError", "Lfm2Config", "known_architectures", "register_architecture", "Engine", "Model",
           "StepError", "GenerationError", "KernelError", "load_model", "random_model", "SamplingParams", "WeightsError", "write_random_model"]
__version__ = "0.1.0"
