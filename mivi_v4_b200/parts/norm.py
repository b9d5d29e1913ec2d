"""Norms."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..ops import kernels as K
from .base import Part
from .registry import register
from .spec import ParamSpec


@register("norm", "rmsnorm")
class RMSNorm(Part):
    """y = x * (mean(x^2) + eps)^-1/2 * weight over the last dimension, in
    float32 (crates/mivi-core/src/simd/norm.rs:38-72; math.rs:14-29)."""

    def __init__(self, dim: int, eps: float):
        self.dim, self.eps = int(dim), float(eps)
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.dim,), "vector", "norm")}

    def forward(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        return K.rmsnorm(x, self.weight, self.eps, out, rows)

    def link(self, step, name: str) -> K.NormLink:
        """This norm as something the products around it carry (steps of few tokens): buffers for
        the rows bf16(x * weight) and the tile sums of squares, from the step's workspace."""
        n = step.n_tokens
        return K.NormLink(self, self.weight, self.eps, self.dim,
                          step.ws.get("link_rows_" + name, (n, self.dim), torch.bfloat16),
                          step.ws.get("link_sums_" + name, (n, -(-self.dim // 64) * 4), torch.float32))
