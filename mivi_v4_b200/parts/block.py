"""Arrangements of a layer's parts."""
from __future__ import annotations

from .base import Part
from .registry import register


@register("block", "prenorm")
class PreNormBlock(Part):
    """x += mixer(norm(x)); x += feed_forward(norm(x)): the arrangement of both
    layer kinds of the reference (crates/mivi-model/src/ssm.rs:65,155-166;
    transformer.rs:317,338; ffn.rs:64,106).  The residual stream stays in
    float32; the normed activations are in the model's dtype."""

    nested_roles = {"mixer_norm": "norm", "mixer": "mixer", "ffn_norm": "norm", "ffn": "feed_forward"}

    def __init__(self, mixer_norm, mixer, ffn_norm, ffn):
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn

    def nested(self):
        return {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "ffn_norm": self.ffn_norm, "ffn": self.ffn}

    def cache_need(self):
        return self.mixer.cache_need()

    def forward(self, resid, step, view) -> None:
        N, H = resid.shape
        u = step.ws.get("normed", (N, H), step.dtype)
        self.mixer_norm.forward(resid, u)
        self.mixer.forward(u, resid, step, view)
        g = step.ws.get("normed", (N, H), step.dtype)
        self.ffn_norm.forward(resid, g)
        self.ffn.forward(g, resid, step)
