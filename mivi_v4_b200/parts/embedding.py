"""Token embedding and output head."""
from __future__ import annotations

from typing import Dict

import torch

from ..ops import kernels as K
from ..ops.linear import linear, norm_link_ok
from .base import Part
from .registry import register
from .spec import ParamSpec


@register("embedding", "table")
class Embedding(Part):
    """x_t = E[token_t], no scaling (crates/mivi-model/src/model.rs:355-366)."""

    emits_norm = True            # forward(step, emit=link) can write the norm that follows it

    def __init__(self, vocab: int, hidden: int):
        self.vocab, self.hidden = int(vocab), int(hidden)

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.vocab, self.hidden))}

    def forward(self, step, emit=None) -> torch.Tensor:
        """``emit``: the first layer's first norm as a link (steps of few tokens); its rows and sums
        are then written here and that norm is no kernel of its own."""
        x = step.ws.get("resid", (step.n_tokens, self.hidden), torch.float32)
        return K.embed(self.weight, step.tokens, x, emit)


@register("head", "linear")
class LMHead(Part):
    """logits = f W^T in float32; W is the embedding table when ``tied``
    (crates/mivi-model/src/model.rs:455-473)."""

    def __init__(self, vocab: int, hidden: int, tied: bool):
        self.vocab, self.hidden, self.tied = int(vocab), int(hidden), bool(tied)

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {} if self.tied else {"weight": ParamSpec((self.vocab, self.hidden))}

    def carries_norm(self, step, embedding) -> bool:
        """Whether the product can apply the final norm's scale itself (steps of few rows)."""
        w = embedding.weight if self.tied else self.weight
        return norm_link_ok(step.n_out, w, step.dtype)

    def forward(self, f, step, embedding, scale=None) -> torch.Tensor:
        w = embedding.weight if self.tied else self.weight
        logits = step.ws.get("logits", (f.shape[0], self.vocab), torch.float32)
        return linear(f, w, logits, scale=scale)
