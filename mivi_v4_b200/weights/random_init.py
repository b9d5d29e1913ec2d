"""Random weights from a configuration and a seed, written as a model folder
(config.json, model.safetensors) that the loader reads like any other.

Distributions: matrices and embeddings N(0, 0.02), convolution taps N(0, 0.2),
norm weights 1 + N(0, 0.1), biases N(0, 0.02).  Drawn in float32 on the CPU
from one generator, tensor by tensor in the order of the model's name table,
then stored in the requested dtype: the same seed gives the same folder on
every machine.  The reference has only closed-form fixture generators
(training/export/generate_fixture.py:20-38).

``init="loud"`` draws matrices with standard deviation 1/sqrt(columns),
convolution taps with 1/sqrt(width) and biases with 0.1 instead: every part
of every layer then moves the residual stream by as much as it holds, at any
width, so that no part's fault can hide below the rounding of another.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional

import torch

from ..parts.spec import ParamSpec
from .safetensors_io import write_file

_STD = {"linear": (0.0, 0.02), "conv": (0.0, 0.2), "norm": (1.0, 0.1), "bias": (0.0, 0.02)}
_STORE = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
          "float16": torch.float16}


INITS = ("baseline", "loud")


def init_std(spec: ParamSpec, init: str = "baseline"):
    """(mean, standard deviation) that ``spec``'s tensor is drawn with."""
    mean, std = _STD[spec.init]
    if init == "loud":
        if spec.init in ("linear", "conv"):
            std = float(spec.shape[-1]) ** -0.5
        elif spec.init == "bias":
            std = 0.1
    return mean, std


def random_tensors(expected: Dict[str, ParamSpec], seed: int, store_dtype: torch.dtype, init: str = "baseline",
                   store_overrides: Optional[Dict[str, torch.dtype]] = None) -> Dict[str, torch.Tensor]:
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    out: Dict[str, torch.Tensor] = {}
    for name, spec in expected.items():
        store = (store_overrides or {}).get(name, store_dtype)
        if spec.role == "table":
            out[name] = torch.zeros(spec.shape, dtype=torch.int32)
        elif spec.init == "zeros":
            out[name] = torch.zeros(spec.shape, dtype=store)
        else:
            mean, std = init_std(spec, init)
            out[name] = (mean + std * torch.randn(spec.shape, generator=gen, dtype=torch.float32)).to(store)
    return out


def write_random_model(model_dir: str, config_dict: dict, seed: int = 0, store_dtype: str = "bfloat16",
                       init: str = "baseline", store_overrides: Optional[Dict[str, str]] = None) -> str:
    """Write config.json and model.safetensors for ``config_dict`` (which names
    its architecture under ``architectures``) with weights drawn from ``seed``.
    ``store_overrides``: tensor name -> store dtype for tensors that are kept in another dtype
    than the rest (a checkpoint with some matrices in 32-bit)."""
    from ..engine.model import expected_tensors        # late: engine imports weights
    if store_dtype not in _STORE:
        raise ValueError(f"store dtype {store_dtype!r}; known: {', '.join(sorted(_STORE))}")
    if init not in INITS:
        raise ValueError(f"init {init!r}; known: {', '.join(INITS)}")
    expected = expected_tensors(config_dict)
    overrides = {}
    for name, d in (store_overrides or {}).items():
        if name not in expected:
            raise ValueError(f"store_overrides names {name!r}, which the model does not have")
        if d not in _STORE:
            raise ValueError(f"store dtype {d!r} for {name}; known: {', '.join(sorted(_STORE))}")
        overrides[name] = _STORE[d]
    os.makedirs(model_dir, exist_ok=True)
    cfg = dict(config_dict)
    cfg.setdefault("torch_dtype", "bfloat16" if _STORE[store_dtype] == torch.bfloat16 else store_dtype)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(cfg, f, indent=2)
    write_file(os.path.join(model_dir, "model.safetensors"),
               random_tensors(expected, seed, _STORE[store_dtype], init, overrides),
               metadata={"format": "pt", "seed": str(seed), "init": init})
    return model_dir
