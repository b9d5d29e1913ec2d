"""Weights from a model folder by tensor name.

The reference resolves each tensor by exact name and fails with
MissingWeight / DimMismatch on the first fault
(crates/mivi-model/src/loader.rs:223-251, 359-415;
crates/mivi-model/src/model.rs:26-49).  Here every name and shape is checked
against what the model's parts declare before any tensor is read, and all
faults are reported in ONE error: missing tensors, unexpected tensors, wrong
shapes, unusable dtypes.

Dtypes: in a bfloat16 run, matrices stored as BF16 stay bfloat16 and F16 is
converted to bfloat16; a matrix stored in 32-bit stays in 32-bit (its products
then run on the 32-bit kernel).  In a float32 run everything is widened to
float32, which is exact.  Vectors (norm weights, biases, convolution taps) are
widened to float32 in both, because the kernels read them in 32-bit; integer
tables become int32.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from ..parts.spec import ParamSpec
from .safetensors_io import SafetensorsError, TensorEntry, read_model_headers, read_tensor

_FLOAT = ("F32", "BF16", "F16", "F64")
_INT = ("I64", "I32", "I16", "I8", "U8")


class WeightsError(ValueError):
    """The checkpoint does not fit the model.  ``missing``, ``unexpected``,
    ``wrong_shape`` [(name, got, want)] and ``wrong_dtype`` [(name, got)] hold
    the particulars that the message lists."""

    def __init__(self, where: str, missing: List[str], unexpected: List[str],
                 wrong_shape: List[Tuple[str, tuple, tuple]], wrong_dtype: List[Tuple[str, str]]):
        self.missing, self.unexpected = missing, unexpected
        self.wrong_shape, self.wrong_dtype = wrong_shape, wrong_dtype
        lines = [f"the tensors of {where} do not fit the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shape ({len(wrong_shape)}): " + ", ".join(
                f"{n} is {list(g)}, expected {list(w)}" for n, g, w in wrong_shape))
        if wrong_dtype:
            lines.append(f"  unusable dtype ({len(wrong_dtype)}): " + ", ".join(f"{n} is {d}" for n, d in wrong_dtype))
        super().__init__("\n".join(lines))


def check_entries(where: str, expected: Dict[str, ParamSpec], entries: Dict[str, TensorEntry],
                  ignorable: Tuple[str, ...] = ()) -> None:
    missing = [n for n in expected if n not in entries]
    unexpected = [n for n in entries if n not in expected and n not in ignorable]
    wrong_shape, wrong_dtype = [], []
    for n, spec in expected.items():
        e = entries.get(n)
        if e is None:
            continue
        if tuple(e.shape) != tuple(spec.shape):
            wrong_shape.append((n, tuple(e.shape), tuple(spec.shape)))
        ok = _INT if spec.role == "table" else _FLOAT
        if e.dtype not in ok:
            wrong_dtype.append((n, e.dtype))
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightsError(where, missing, unexpected, wrong_shape, wrong_dtype)


def run_dtype(stored: str, role: str, dtype: torch.dtype) -> torch.dtype:
    """The dtype a tensor runs in, from how it is stored, what it is, and the
    dtype of the run."""
    if role == "table":
        return torch.int32
    if role == "vector" or dtype == torch.float32:
        return torch.float32
    return torch.float32 if stored in ("F32", "F64") else torch.bfloat16


def load_tensors(model_dir: str, expected: Dict[str, ParamSpec], dtype: torch.dtype, device,
                 ignorable: Tuple[str, ...] = ()) -> Dict[str, torch.Tensor]:
    try:
        entries = read_model_headers(model_dir)
    except SafetensorsError as e:
        raise WeightsError(f"{model_dir} ({e})", sorted(expected), [], [], []) from None
    check_entries(model_dir, expected, entries, ignorable)
    out: Dict[str, torch.Tensor] = {}
    for name, spec in expected.items():
        t = read_tensor(entries[name])
        out[name] = t.to(run_dtype(entries[name].dtype, spec.role, dtype)).to(device)
    return out
