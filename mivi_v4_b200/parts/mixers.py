"""Mixers: the parts of a layer that move information between tokens."""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..cache.needs import KVNeed, StateNeed
from ..ops import kernels as K
from ..ops.linear import (conv_rows_grouped, heads_fused_ok, linear, linear_heads, linear_shortconv_decode, norm_link_ok,
                          shortconv_decode_fused_ok)
from .base import Part
from .registry import register
from .spec import ParamSpec


@register("mixer", "short_conv")
class ShortConv(Part):
    """Gated short convolution: in_proj to (B, C, x), B*x, causal depthwise
    convolution of width ``kernel``, C*, out_proj
    (crates/mivi-model/src/ssm.rs:51-155).  Its state per sequence is the last
    kernel-1 values of B*x.  With ``bias`` the three linear maps carry one
    (the checkpoint format's conv_bias; the reference has none)."""

    def __init__(self, hidden: int, kernel: int, bias: bool = False):
        if not 1 <= kernel <= K.MAX_CONV_K:
            raise ValueError(f"convolution width {kernel} is outside 1..{K.MAX_CONV_K}")
        self.hidden, self.kernel, self.bias = int(hidden), int(kernel), bool(bias)

    def param_specs(self) -> Dict[str, ParamSpec]:
        H, k = self.hidden, self.kernel
        specs = {"in_proj.weight": ParamSpec((3 * H, H)),
                 "conv.weight": ParamSpec((H, 1, k), "vector", "conv"),
                 "out_proj.weight": ParamSpec((H, H))}
        if self.bias:
            specs.update({"in_proj.bias": ParamSpec((3 * H,), "vector", "bias"),
                          "conv.bias": ParamSpec((H,), "vector", "bias"),
                          "out_proj.bias": ParamSpec((H,), "vector", "bias")})
        return specs

    def load(self, t) -> None:
        self.w_in, self.w_out = t["in_proj.weight"], t["out_proj.weight"]
        self.w_in_grouped = None
        self.taps = t["conv.weight"].reshape(self.hidden, self.kernel).contiguous()
        self.b_in, self.b_conv, self.b_out = t.get("in_proj.bias"), t.get("conv.bias"), t.get("out_proj.bias")

    def cache_need(self):
        return StateNeed((self.kernel - 1, self.hidden))

    def carries_norm(self, step):
        n = step.n_tokens
        return norm_link_ok(n, self.w_in, step.dtype), norm_link_ok(n, self.w_out, step.dtype, emits=True)

    def forward(self, u, resid, step, view, scale=None, emit=None) -> None:
        N, H = u.shape
        z = self.scratch(step, "mix", (N, H), step.dtype)
        if step.is_decode and N == step.n_seqs and shortconv_decode_fused_ok(N, u, self.w_in):
            # a few sequences, one token each: the convolution is the projection's epilogue (from 9 sequences
            # on over a copy of the projection whose rows are regrouped, made when first wanted)
            w_in, grouped = self.w_in, conv_rows_grouped(N, self.w_in)
            if grouped:
                if self.w_in_grouped is None:
                    self.w_in_grouped = K.group_conv_rows(self.w_in)
                w_in = self.w_in_grouped
            linear_shortconv_decode(u, w_in, self.b_in, self.taps, self.b_conv, view.state, step.slots, z,
                                    scale=scale, grouped=grouped)
            linear(z, self.w_out, resid, bias=self.b_out, accumulate=True, emit=emit)
            return
        p = self.scratch(step, "proj", (N, 3 * H), torch.float32)
        linear(u, self.w_in, p, bias=self.b_in, scale=scale)
        K.shortconv(p, self.taps, self.b_conv, view.state, step.positions, step.seq_of, step.cu,
                    step.slots, step.starts, step.lens, z, step.n_seqs, decode=step.is_decode)
        linear(z, self.w_out, resid, bias=self.b_out, accumulate=True, emit=emit)


@register("mixer", "gqa")
class GroupedQueryAttention(Part):
    """Grouped-query attention over the cache: q, k, v projections, per-head
    RMSNorm of q and k (``qk_norm_eps`` None: none), the position part's
    rotation, append to the cache, causal softmax attention with scale
    1/sqrt(head_dim) and an optional window, out projection
    (crates/mivi-model/src/transformer.rs:55-110, 114-167, 304-350).
    ``shared_kv``: the layer has no k and v of its own and reads the cache of
    another layer (its schedule entry says which)."""

    nested_roles = {"position": "position"}

    def __init__(self, hidden: int, n_heads: int, n_kv_heads: int, head_dim: int, position,
                 qk_norm_eps: Optional[float] = None, window: int = 0, shared_kv: bool = False):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads are not a multiple of {n_kv_heads} kv heads")
        if head_dim % 8 or head_dim > K.MAX_HEAD_DIM:
            raise ValueError(f"head size {head_dim} must be a multiple of 8 and at most {K.MAX_HEAD_DIM}")
        self.hidden, self.nh, self.nkv, self.hd = int(hidden), int(n_heads), int(n_kv_heads), int(head_dim)
        self.position = position
        self.qk_norm_eps = None if qk_norm_eps is None else float(qk_norm_eps)
        self.window, self.shared_kv = int(window), bool(shared_kv)
        # a position part may put a constant factor on the scores
        self.scale = 1.0 / math.sqrt(self.hd) * float(getattr(position, "score_scale", lambda: 1.0)())

    def nested(self):
        return {"position": self.position}

    def param_specs(self) -> Dict[str, ParamSpec]:
        H, nh, nkv, hd = self.hidden, self.nh, self.nkv, self.hd
        specs = {"q_proj.weight": ParamSpec((nh * hd, H))}
        if not self.shared_kv:
            specs["k_proj.weight"] = ParamSpec((nkv * hd, H))
            specs["v_proj.weight"] = ParamSpec((nkv * hd, H))
        specs["out_proj.weight"] = ParamSpec((H, nh * hd))
        if self.qk_norm_eps is not None:
            specs["q_layernorm.weight"] = ParamSpec((hd,), "vector", "norm")
            if not self.shared_kv:
                specs["k_layernorm.weight"] = ParamSpec((hd,), "vector", "norm")
        return specs

    def load(self, t) -> None:
        if self.shared_kv:
            # the fused projection has the rows of k and v left out; the kernel skips them
            self.w_qkv = t["q_proj.weight"]
        else:
            ws = [t["q_proj.weight"], t["k_proj.weight"], t["v_proj.weight"]]
            if len({w.dtype for w in ws}) != 1:
                ws = [w.float() for w in ws]
            self.w_qkv = torch.cat(ws, dim=0).contiguous()
        self.w_o = t["out_proj.weight"]
        self.q_norm, self.k_norm = t.get("q_layernorm.weight"), t.get("k_layernorm.weight")

    def cache_need(self):
        return KVNeed(self.nkv, self.hd, self.window)

    def carries_norm(self, step):
        n = step.n_tokens
        return norm_link_ok(n, self.w_qkv, step.dtype), norm_link_ok(n, self.w_o, step.dtype, emits=True)

    def forward(self, u, resid, step, view, scale=None, emit=None) -> None:
        N = u.shape[0]
        nh, nkv, hd = self.nh, self.nkv, self.hd
        if view.writable == self.shared_kv:
            raise RuntimeError("a shared_kv attention layer must read another layer's cache, and only it may")
        width = (nh + (0 if self.shared_kv else 2 * nkv)) * hd
        q = self.scratch(step, "q", (N, nh * hd), step.dtype)
        rot = self.position.rotary(u.device)
        inv_freq, half_split = rot if rot is not None else (None, False)
        eps = self.qk_norm_eps if self.qk_norm_eps is not None else 0.0
        if not self.shared_kv and heads_fused_ok(N, u, self.w_qkv, hd, view.pool, half_split):
            # a few tokens: norm, rotation and the append to the cache are the projection's epilogue
            linear_heads(u, self.w_qkv, self.q_norm, self.k_norm, eps, inv_freq, half_split, step.positions,
                         step.seq_of, view.page_table, view.pool, q, nh, nkv, scale=scale)
        else:
            qkv = self.scratch(step, "proj", (N, width), torch.float32)
            linear(u, self.w_qkv, qkv, scale=scale)
            if self.shared_kv:
                K.qk_prepare_q_only(qkv, self.q_norm, eps, inv_freq, half_split, step.positions, q, nh, hd)
            else:
                K.qk_prepare(qkv, self.q_norm, self.k_norm, eps, inv_freq, half_split, step.positions,
                             step.seq_of, view.page_table, view.pool, q, nh, nkv, hd)
        o = self.scratch(step, "mix", (N, nh * hd), step.dtype)
        # few query tokens, or many sequences with a token or two each: every query token on its own
        few = N <= K.DECODE_ATTENTION_MAX_TOKENS or step.max_len <= K.DECODE_ATTENTION_MAX_QUERIES
        if few and K.attention_decode_tc_supported(step.dtype, hd, view.pool, self.window, nh, nkv):
            # few query tokens, head size 64: flash decoding with both products on tcgen05
            K.attention_decode_tc(q, view.pool, view.page_table, step.positions, step.seq_of, o, nh, nkv, hd,
                                  self.scale, step.ws)
        elif few:
            K.attention_decode(q, view.pool, view.page_table, step.positions, step.seq_of, o, nh, nkv, hd,
                               self.scale, self.window, step.ws)
        elif (N >= 128 * step.n_seqs and K.attention_prefill_tc_supported(step.dtype, hd, view.pool, self.window)):
            # long chunks: 256 query rows a block, both products on tcgen05
            K.attention_prefill_tc(q, view.pool, view.page_table, step.cu, step.starts, o, step.n_seqs, nh, nkv,
                                   hd, self.scale)
        elif K.attention_prefill_supported(step.dtype, hd):
            K.attention_prefill(q, view.pool, view.page_table, step.cu, step.starts, o, step.n_seqs, nh, nkv, hd,
                                self.scale, self.window)
        else:
            K.attention_generic(q, view.pool, view.page_table, step.positions, step.seq_of, o, nh, nkv, hd,
                                self.scale, self.window)
        if K.profiling_on():
            # keys that the step's queries read (each query its own context), for the attention launch
            pairs = sum(n * s + n * (n + 1) // 2 for s, n in zip(step.host_starts, step.host_lens))
            rows = pairs if few else sum(s + n for s, n in zip(step.host_starts, step.host_lens))
            K.account(2 * nkv * hd * view.pool.element_size() * rows + 2 * N * nh * hd * q.element_size(),
                      4 * nh * hd * pairs)
        linear(o, self.w_o, resid, accumulate=True, emit=emit)
