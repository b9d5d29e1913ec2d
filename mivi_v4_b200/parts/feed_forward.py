"""Feed-forwards: the parts of a layer that work on each token alone."""
from __future__ import annotations

from typing import Dict

import torch

from ..ops import kernels as K
from ..ops.linear import linear
from .base import Part
from .registry import register
from .spec import ParamSpec


@register("feed_forward", "swiglu")
class SwiGLU(Part):
    """x + (silu(g W1^T) * (g W3^T)) W2^T without biases
    (crates/mivi-model/src/ffn.rs:56-108).  W1 and W3 are laid end to end at
    load time so that one product yields gate and up."""

    def __init__(self, hidden: int, ff: int):
        self.hidden, self.ff = int(hidden), int(ff)

    def param_specs(self) -> Dict[str, ParamSpec]:
        H, F = self.hidden, self.ff
        return {"w1.weight": ParamSpec((F, H)), "w3.weight": ParamSpec((F, H)), "w2.weight": ParamSpec((H, F))}

    def load(self, t) -> None:
        w1, w3 = t["w1.weight"], t["w3.weight"]
        if w1.dtype != w3.dtype:
            w1, w3 = w1.float(), w3.float()
        self.w13 = torch.cat([w1, w3], dim=0).contiguous()
        self.w2 = t["w2.weight"]

    def forward(self, g, resid, step) -> None:
        N = g.shape[0]
        gu = step.ws.get("proj", (N, 2 * self.ff), torch.float32)
        linear(g, self.w13, gu)
        h = step.ws.get("ffh", (N, self.ff), step.dtype)
        K.swiglu(gu, h)
        linear(h, self.w2, resid, accumulate=True)
