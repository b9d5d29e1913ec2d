"""Random weights from a configuration and a seed, written as a model folder
(config.json, model.safetensors) that the loader reads like any other.

Distributions: matrices and embeddings N(0, 0.02), convolution taps N(0, 0.2),
norm weights 1 + N(0, 0.1), biases N(0, 0.02).  Drawn in float32 on the CPU
from one generator, tensor by tensor in the order of the model's name table,
then stored in the requested dtype: the same seed gives the same folder on
every machine.  The reference has only closed-form fixture generators
(training/export/generate_fixture.py:20-38).
"""
from __future__ import annotations

import json
import os
from typing import Dict

import torch

from ..parts.spec import ParamSpec
from .safetensors_io import write_file

_STD = {"linear": (0.0, 0.02), "conv": (0.0, 0.2), "norm": (1.0, 0.1), "bias": (0.0, 0.02)}
_STORE = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
          "float16": torch.float16}


def random_tensors(expected: Dict[str, ParamSpec], seed: int, store_dtype: torch.dtype) -> Dict[str, torch.Tensor]:
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    out: Dict[str, torch.Tensor] = {}
    for name, spec in expected.items():
        if spec.role == "table":
            out[name] = torch.zeros(spec.shape, dtype=torch.int32)
        elif spec.init == "zeros":
            out[name] = torch.zeros(spec.shape, dtype=store_dtype)
        else:
            mean, std = _STD[spec.init]
            out[name] = (mean + std * torch.randn(spec.shape, generator=gen, dtype=torch.float32)).to(store_dtype)
    return out


def write_random_model(model_dir: str, config_dict: dict, seed: int = 0, store_dtype: str = "bfloat16") -> str:
    """Write config.json and model.safetensors for ``config_dict`` (which names
    its architecture under ``architectures``) with weights drawn from ``seed``."""
    from ..engine.model import expected_tensors        # late: engine imports weights
    if store_dtype not in _STORE:
        raise ValueError(f"store dtype {store_dtype!r}; known: {', '.join(sorted(_STORE))}")
    expected = expected_tensors(config_dict)
    os.makedirs(model_dir, exist_ok=True)
    cfg = dict(config_dict)
    cfg.setdefault("torch_dtype", "bfloat16" if _STORE[store_dtype] == torch.bfloat16 else store_dtype)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(cfg, f, indent=2)
    write_file(os.path.join(model_dir, "model.safetensors"), random_tensors(expected, seed, _STORE[store_dtype]),
               metadata={"format": "pt", "seed": str(seed)})
    return model_dir
