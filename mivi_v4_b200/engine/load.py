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
                 device: str = "cuda:0", model_dir: Optional[str] = None, on_device: bool = False,
                 init: str = "baseline") -> Model:
    """A model with random weights: written as a model folder (a temporary one
    unless ``model_dir`` is given) and loaded back, so it takes the same path
    as a checkpoint.  ``on_device`` draws the same distributions directly on
    the device instead (other values for the same seed, no file): the quick
    way to a large model for measurements."""
    dtype = parse_dtype(dtype)
    if on_device:
        from ..weights.loader import run_dtype
        from ..weights.random_init import init_std
        config, spec = describe_config(config_dict)
        model = Model(spec, config)
        gen = torch.Generator(device=device)
        gen.manual_seed(int(seed))
        named = {}
        stored = "BF16" if dtype == torch.bfloat16 else "F32"
        for name, ps in model.named_param_specs().items():
            rd = run_dtype(stored, ps.role, dtype)
            if ps.role == "table" or ps.init == "zeros":
                named[name] = torch.zeros(ps.shape, dtype=rd, device=device)
                continue
            mean, std = init_std(ps, init)
            t = torch.empty(ps.shape, dtype=torch.float32, device=device).normal_(mean, std, generator=gen)
            named[name] = t.to(torch.bfloat16).to(rd) if dtype == torch.bfloat16 else t
        model.load_params(named, dtype, device)
        return model
    store = "bfloat16" if dtype == torch.bfloat16 else "float32"
    if model_dir is not None:
        return load_model(write_random_model(model_dir, config_dict, seed, store, init), dtype, device)
    with tempfile.TemporaryDirectory(prefix="mivi_model_") as tmp:
        return load_model(write_random_model(tmp, config_dict, seed, store, init), dtype, device)
