"""Feed-forwards: the parts of a layer that work on each token alone."""
from __future__ import annotations

from typing import Dict

import torch

from ..ops import kernels as K
from ..ops.linear import linear, linear_swiglu, norm_link_ok, tensor_core_ok
from .base import Part
from .registry import register
from .spec import ParamSpec


@register("feed_forward", "swiglu")
class SwiGLU(Part):
    """x + (silu(g W1^T) * (g W3^T)) W2^T without biases
    (crates/mivi-model/src/ffn.rs:56-108).  W1 and W3 are merged at load time
    so that one product yields gate and up: in alternating groups of 16 rows
    (16 of W1, then the 16 of W3 for the same features) when the width allows,
    which lets the tensor-core kernels apply the activation in their
    epilogue; else end to end."""

    def __init__(self, hidden: int, ff: int):
        self.hidden, self.ff = int(hidden), int(ff)

    def param_specs(self) -> Dict[str, ParamSpec]:
        H, F = self.hidden, self.ff
        return {"w1.weight": ParamSpec((F, H)), "w3.weight": ParamSpec((F, H)), "w2.weight": ParamSpec((H, F))}

    def load(self, t) -> None:
        w1, w3 = t["w1.weight"], t["w3.weight"]
        if w1.dtype != w3.dtype:
            w1, w3 = w1.float(), w3.float()
        G = K.SWIGLU_GROUP
        self.group = G if self.ff % G == 0 else 0
        if self.group:
            F, H = w1.shape
            self.w13 = torch.stack([w1.view(F // G, G, H), w3.view(F // G, G, H)], dim=1).reshape(2 * F, H).contiguous()
        else:
            self.w13 = torch.cat([w1, w3], dim=0).contiguous()
        self.w2 = t["w2.weight"]

    def carries_norm(self, step):
        n = step.n_tokens
        return (bool(self.group) and norm_link_ok(n, self.w13, step.dtype)), norm_link_ok(n, self.w2, step.dtype, emits=True)

    def forward(self, g, resid, step, scale=None, emit=None) -> None:
        N = g.shape[0]
        h = self.scratch(step, "ffh", (N, self.ff), step.dtype)
        if self.group and tensor_core_ok(g, self.w13):
            linear_swiglu(g, self.w13, h, scale=scale)
        else:
            gu = self.scratch(step, "proj", (N, 2 * self.ff), torch.float32)
            linear(g, self.w13, gu, scale=scale)
            K.swiglu(gu, h, self.group)
        linear(h, self.w2, resid, accumulate=True, emit=emit)
