"""From a model folder (config.json, model.safetensors) to a model with its
weights on the device.  The model class is chosen by config.json's
``architectures`` through the registry, as everywhere in the library."""
from __future__ import annotations

import tempfile
from typing import Optional, Union

import torch

from ..config import read_config_json
from ..weights import load_tensors, write_random_model
from .model import Model, describe_config

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           "f32": torch.float32}


def parse_dtype(dtype: Union[str, torch.dtype]) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype {dtype}: the library runs in bfloat16 or float32")
        return dtype
    if dtype not in _DTYPES:
        raise ValueError(f"dtype {dtype!r}; known: {', '.join(sorted(_DTYPES))}")
    return _DTYPES[dtype]


def load_model(model_dir: str, dtype: Union[str, torch.dtype] = "bfloat16", device: str = "cuda:0") -> Model:
    dtype = parse_dtype(dtype)
    config, spec = describe_config(read_config_json(model_dir))
    model = Model(spec, config)
    named = load_tensors(model_dir, model.named_param_specs(), dtype, device, spec.ignorable)
    model.load_params(named, dtype, device)
    return model


def random_model(config_dict: dict, seed: int = 0, dtype: Union[str, torch.dtype] = "bfloat16",
                 device: str = "cuda:0", model_dir: Optional[str] = None) -> Model:
    """A model with random weights: written as a model folder (a temporary one
    unless ``model_dir`` is given) and loaded back, so it takes the same path
    as a checkpoint."""
    dtype = parse_dtype(dtype)
    store = "bfloat16" if dtype == torch.bfloat16 else "float32"
    if model_dir is not None:
        return load_model(write_random_model(model_dir, config_dict, seed, store), dtype, device)
    with tempfile.TemporaryDirectory(prefix="mivi_model_") as tmp:
        return load_model(write_random_model(tmp, config_dict, seed, store), dtype, device)
