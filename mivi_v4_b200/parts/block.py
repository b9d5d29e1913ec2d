"""Arrangements of a layer's parts."""
from __future__ import annotations

from ..ops.kernels import profile_stage
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
        """The mixer's needs, followed by the feed-forward's if it keeps something too (the block's need is
        then a list, and ``forward`` deals the views out again)."""
        need = self.mixer.cache_need()
        extra = self.ffn.cache_need() if hasattr(self.ffn, "cache_need") else None
        if extra is None:
            self._views = None
            return need
        mixer_list = isinstance(need, (list, tuple))
        mine = list(need) if mixer_list else ([] if need is None else [need])
        ffn_list = isinstance(extra, (list, tuple))
        self._views = (len(mine), mixer_list, ffn_list)
        return mine + (list(extra) if ffn_list else [extra])

    def entry_link(self, step):
        """The first norm of this block as a link that the block before may fill, or None."""
        if step.carry_norms and hasattr(self.mixer_norm, "link") and self.mixer.carries_norm(step)[0]:
            return self.mixer_norm.link(step, "entry")
        return None

    def forward(self, resid, step, view, after=None) -> None:
        """``after``: the block that runs next in this step, if any.  In a step of few tokens the two
        norms are not kernels of their own where the parts allow it: the product that completes the
        residual stream writes the next norm's rows, the product that reads them applies its scale."""
        N, H = resid.shape
        ffn_kw = {}
        if getattr(self, "_views", None) is not None:
            n_mixer, mixer_list, ffn_list = self._views
            views = list(view)
            view = views[:n_mixer] if mixer_list else (views[0] if n_mixer else None)
            ffn_kw["view"] = views[n_mixer:] if ffn_list else views[n_mixer]
        carry = step.carry_norms
        _, mixer_emits = self.mixer.carries_norm(step) if carry else (False, False)
        ffn_accepts, ffn_emits = self.ffn.carries_norm(step) if carry else (False, False)
        entry = step.take_link(self.mixer_norm)
        mid = self.ffn_norm.link(step, "mid") if mixer_emits and ffn_accepts and hasattr(self.ffn_norm, "link") else None
        leave = after.entry_link(step) if ffn_emits and after is not None and hasattr(after, "entry_link") else None
        kw = {}
        if entry is not None:
            u, kw["scale"] = entry.xg, entry
        else:
            u = self.scratch(step, "normed", (N, H), step.dtype)
            with profile_stage("norm"):
                self.mixer_norm.forward(resid, u)
        if mid is not None:
            kw["emit"] = mid
        with profile_stage("mixer " + getattr(self.mixer, "kind", "?")):
            self.mixer.forward(u, resid, step, view, **kw)
        kw = dict(ffn_kw)
        if mid is not None:
            g, kw["scale"] = mid.xg, mid
        else:
            g = self.scratch(step, "normed", (N, H), step.dtype)
            with profile_stage("norm"):
                self.ffn_norm.forward(resid, g)
        if leave is not None:
            kw["emit"] = leave
        with profile_stage("feed_forward " + getattr(self.ffn, "kind", "?")):
            self.ffn.forward(g, resid, step, **kw)
        step.leave_link(leave)
