"""Position encodings.  A mixer that rotates its queries and keys asks its
position part for ``rotary()``; a part that encodes nothing returns None.  A part may
also define ``score_scale()``: a constant factor on the attention scores (an encoding
that stretches its frequencies and makes up for it by sharpening the softmax); the
mixer multiplies its 1/sqrt(head_dim) by it."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .base import Part
from .registry import register

ROPE_STYLES = ("interleaved", "half_split")


@register("position", "rope")
class Rope(Part):
    """Rotary encoding: pair i of a head turns by pos * theta^(-2i/head_dim)
    (crates/mivi-core/src/rope.rs:59-61, 116-121).  ``interleaved`` pairs the
    elements (2i, 2i+1) as the reference does (rope.rs:219-229);
    ``half_split`` pairs (i, i + head_dim/2).  The frequencies are worked out
    in float64 and rounded once to float32; the angle is a float32 product."""

    def __init__(self, head_dim: int, theta: float, style: str = "interleaved"):
        if head_dim % 2:
            raise ValueError(f"rotary encoding needs an even head size, got {head_dim}")
        if style not in ROPE_STYLES:
            raise ValueError(f"rope style {style!r}; known: {', '.join(ROPE_STYLES)}")
        self.head_dim, self.theta, self.style = int(head_dim), float(theta), style
        self._inv_freq: Optional[torch.Tensor] = None

    def rotary(self, device) -> Optional[Tuple[torch.Tensor, bool]]:
        if self._inv_freq is None or self._inv_freq.device != torch.device(device):
            i = torch.arange(self.head_dim // 2, dtype=torch.float64)
            inv = 1.0 / (torch.tensor(self.theta, dtype=torch.float64) ** (2.0 * i / self.head_dim))
            self._inv_freq = inv.to(torch.float32).to(device)
        return self._inv_freq, self.style == "half_split"

    def score_scale(self) -> float:
        return 1.0


@register("position", "none")
class NoPosition(Part):
    """No position encoding inside the mixer."""

    def rotary(self, device):
        return None
