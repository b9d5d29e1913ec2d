"""Plain, slow implementation of the LFM2 / LFM2.5 hybrid decoder.

Whole sequences, no cache, one function for each part, float64 (or float32)
torch tensors on the CPU.  It shares no code with the package under test: it
reads ``config.json`` as a dict, takes the weights as a dict keyed by the
checkpoint's tensor names, and restates every formula from the reference
engine (aswin402/mivi-v4).  Each function cites the reference lines that it
restates; where the reference has nothing (``conv_bias``, the feed-forward
width rule, half-split rotary pairing) the docstring says so.

``tests/golden/make_golden.py`` compares this file once with the reference's
own Python oracle (``reference/reference_engine.py``) on a tiny random model
and commits the outputs, so this file rests on more than the formulas.
"""
from __future__ import annotations

import math

import torch


# --------------------------------------------------------------------------
# configuration (restated; the package has its own typed reader)
# --------------------------------------------------------------------------
def plain_ff_dim(cfg: dict) -> int:
    """Feed-forward width from the block_* keys.

    The reference reads the width directly from its model file
    (crates/mivi-model/src/loader.rs:59-65); the rule for the block_* keys is
    the checkpoint format's: no adjustment -> block_ff_dim; else
    int(2*block_ff_dim/3), times block_ffn_dim_multiplier, rounded up to a
    multiple of block_multiple_of.
    """
    ff = int(cfg["block_ff_dim"])
    if cfg.get("block_auto_adjust_ff_dim", False):
        ff = int(2 * ff / 3)
        mult = cfg.get("block_ffn_dim_multiplier", None)
        if mult is not None:
            ff = int(mult * ff)
        m = int(cfg.get("block_multiple_of", 256))
        ff = m * ((ff + m - 1) // m)
    return ff


def plain_dims(cfg: dict) -> dict:
    """Sizes derived as crates/mivi-model/src/loader.rs:150-154 does
    (head_dim = dim / n_heads) plus the checkpoint's own keys."""
    H = int(cfg["hidden_size"])
    nh = int(cfg["num_attention_heads"])
    nkv = int(cfg["num_key_value_heads"])
    return dict(
        H=H, nh=nh, nkv=nkv, hd=H // nh, L=int(cfg["num_hidden_layers"]),
        V=int(cfg["vocab_size"]), F=plain_ff_dim(cfg),
        k=int(cfg.get("conv_L_cache", 3)),
        eps=float(cfg.get("norm_eps", 1e-5)),
        theta=float(cfg.get("rope_theta", 1e6)),
        bias=bool(cfg.get("conv_bias", False)),
        tied=bool(cfg.get("tie_embedding", cfg.get("tie_word_embeddings", True))),
        rope_style=str(cfg.get("rope_style", "interleaved")),
        layer_types=list(cfg["layer_types"]),
    )


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------
def plain_rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x * (mean(x^2) + eps)^-1/2 * w over the last dim.

    crates/mivi-core/src/math.rs:14-29, crates/mivi-core/src/simd/norm.rs:7-72,
    reference/reference_engine.py:43-46.
    """
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(ms + eps) * w


def plain_rope(v: torch.Tensor, positions: torch.Tensor, theta: float,
               style: str = "interleaved") -> torch.Tensor:
    """Rotary position encoding of v [T, heads, hd] at absolute positions [T].

    inv_freq_i = theta^(-2i/hd); angle = pos * inv_freq_i; pairs (2i, 2i+1)
    rotate as (a c - b s, a s + b c): crates/mivi-core/src/rope.rs:59-61
    (frequencies), 116-121 (table), 219-229 (rotation);
    reference/reference_engine.py:66-81.  ``half_split`` pairs (i, i+hd/2)
    instead; the reference has no such mode, it is a parameter of the build.
    """
    T, nheads, hd = v.shape
    half = hd // 2
    i = torch.arange(half, dtype=torch.float64)
    inv_freq = 1.0 / (torch.tensor(theta, dtype=torch.float64) ** (2.0 * i / hd))
    ang = positions.to(torch.float64)[:, None] * inv_freq[None, :]      # [T, half]
    c = torch.cos(ang).to(v.dtype)[:, None, :]
    s = torch.sin(ang).to(v.dtype)[:, None, :]
    out = torch.empty_like(v)
    if style == "interleaved":
        a, b = v[..., 0::2], v[..., 1::2]
        out[..., 0::2] = a * c - b * s
        out[..., 1::2] = a * s + b * c
    elif style == "half_split":
        a, b = v[..., :half], v[..., half:]
        out[..., :half] = a * c - b * s
        out[..., half:] = a * s + b * c
    else:
        raise ValueError(style)
    return out


def _same(t: torch.Tensor) -> torch.Tensor:
    return t


def round_to(storage: torch.dtype):
    """A function that rounds a tensor to ``storage`` and widens it again.  Passed as ``rnd`` to the
    functions below, it is applied where a run in that storage dtype keeps an activation between two
    kernels: the inputs of the matrix products after the norms, the gated convolution's result, the
    queries, the cached keys and values, the softmax weights, the attention's result and the
    SwiGLU product.  Sums, norms, the softmax and the residual stream stay in the working dtype.
    The difference to a run without ``rnd`` is the rounding noise that such a run may show."""
    def rnd(t: torch.Tensor) -> torch.Tensor:
        return t.to(storage).to(t.dtype)
    return rnd


def plain_short_conv(u: torch.Tensor, w_in: torch.Tensor, w_conv: torch.Tensor,
                     w_out: torch.Tensor, b_in=None, b_conv=None, b_out=None, rnd=_same,
                     return_state: bool = False) -> torch.Tensor:
    """Gated short convolution over a whole sequence u [T, H] (already normed).

    p = u W_in^T; B, C, X = thirds of p in that order; bx = B*X;
    y_t[d] = sum_j w[d, j] * bx_{t-(k-1)+j}[d] with zeros before the sequence
    (tap k-1 is the current token); z = C*y; returns z W_out^T.
    crates/mivi-model/src/ssm.rs:68-85 (projection, split, first gate),
    87-140 (state shift and taps), 110 and 143-152 (second gate, out
    projection); reference/reference_engine.py:185-211.  The reference has no
    biases: b_in is added to p, b_conv to y, b_out to the result (the
    checkpoint format's ``conv_bias``).
    """
    T, H = u.shape
    k = w_conv.shape[-1]
    w_conv = w_conv.reshape(H, k)
    p = u @ w_in.T
    if b_in is not None:
        p = p + b_in
    Bg, Cg, X = p[:, :H], p[:, H:2 * H], p[:, 2 * H:]
    bx = Bg * X
    y = torch.zeros_like(bx)
    for t in range(T):
        for j in range(k):
            src = t - (k - 1) + j
            if src >= 0:
                y[t] += w_conv[:, j] * bx[src]
    if b_conv is not None:
        y = y + b_conv
    z = rnd(Cg * y)
    out = z @ w_out.T
    if b_out is not None:
        out = out + b_out
    if return_state:
        # what a cache keeps of this layer after the sequence: the last k-1 values of B*x, oldest first
        # (zeros where the sequence is shorter), crates/mivi-model/src/ssm.rs:87-108
        state = torch.zeros(k - 1, H, dtype=u.dtype)
        n = min(k - 1, T)
        if n:
            state[k - 1 - n:] = bx[T - n:]
        return out, state
    return out


def plain_attention(u: torch.Tensor, wq, wk, wv, wo, q_norm_w, k_norm_w, *, nh: int,
                    nkv: int, hd: int, eps: float, theta: float, style: str,
                    window: int = 0, kv=None, return_kv: bool = False, rnd=_same):
    """Grouped-query attention over a whole sequence u [T, H] (already normed).

    q, k, v projections without bias; per-head RMSNorm of q and k with one
    [hd] weight shared by all heads and the layer norms' eps, before the
    rotation (skipped if the weight is None, as the reference's Python oracle
    has none); rotation at absolute positions 0..T-1; head h reads kv head
    h // (nh / nkv); scores q.k / sqrt(hd) over t <= position (causal,
    including itself); softmax; sum of values; out projection.
    crates/mivi-model/src/transformer.rs:77-79, 81-96, 99-105, 114-167,
    293-298, 326-335; reference/reference_engine.py:130-169.
    ``window`` > 0 keeps only the last ``window`` keys (t > position - window);
    the reference has no window, this serves tests of the generic kernel.
    ``kv`` = (k, v) as another layer stored them (after norm and rotation)
    replaces this layer's own keys and values; ``return_kv`` also returns them.
    Both serve tests of a layer that reads another layer's cache.
    """
    T = u.shape[0]
    pos = torch.arange(T)
    q = (u @ wq.T).reshape(T, nh, hd)
    if q_norm_w is not None:
        q = plain_rms_norm(q, q_norm_w, eps)
    q = rnd(plain_rope(q, pos, theta, style))
    if kv is None:
        k = (u @ wk.T).reshape(T, nkv, hd)
        v = (u @ wv.T).reshape(T, nkv, hd)
        if k_norm_w is not None:
            k = plain_rms_norm(k, k_norm_w, eps)
        k, v = rnd(plain_rope(k, pos, theta, style)), rnd(v)
    else:
        k, v = kv
    group = nh // nkv
    scale = 1.0 / math.sqrt(hd)
    out = torch.zeros(T, nh, hd, dtype=u.dtype)
    for h in range(nh):
        g = h // group
        s = (q[:, h, :] @ k[:, g, :].T) * scale                 # [T, T]
        i = torch.arange(T)[:, None]
        j = torch.arange(T)[None, :]
        mask = j <= i
        if window > 0:
            mask = mask & (j > i - window)
        s = s.masked_fill(~mask, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = rnd(p) @ v[:, g, :]
    res = rnd(out.reshape(T, nh * hd)) @ wo.T
    return (res, (k, v)) if return_kv else res


def plain_swiglu(g: torch.Tensor, w1, w3, w2, rnd=_same) -> torch.Tensor:
    """(silu(g W1^T) * (g W3^T)) W2^T with silu(a) = a / (1 + e^-a).

    crates/mivi-model/src/ffn.rs:67-103, crates/mivi-core/src/math.rs:76-98,
    reference/reference_engine.py:49-54 and 175-178.
    """
    a = g @ w1.T
    b = g @ w3.T
    return rnd((a / (1.0 + torch.exp(-a))) * b) @ w2.T


# --------------------------------------------------------------------------
# the whole model
# --------------------------------------------------------------------------
def _w(weights: dict, name: str, dtype):
    return weights[name].to(dtype)


def _opt(weights: dict, name: str, dtype):
    """The per-head q/k norm is skipped when its weight is absent, as
    crates/mivi-model/src/transformer.rs:81-96 does (the Python oracle has
    none); a checkpoint of this architecture always has both."""
    return weights[name].to(dtype) if name in weights else None


def plain_forward(cfg: dict, weights: dict, tokens, dtype=torch.float64,
                  return_hidden: bool = False, rnd=_same, return_residuals: bool = False,
                  return_cache: bool = False) -> torch.Tensor:
    """Logits [T, V] of one whole sequence of token ids, no cache.

    Embedding row gather (crates/mivi-model/src/model.rs:355-366); per layer
    operator norm -> mixer -> residual, ffn norm -> SwiGLU -> residual
    (ssm.rs:65,155-166; transformer.rs:317,338; ffn.rs:64,106); final norm and
    the head, which is the embedding itself when tied (model.rs:437-473).
    ``rnd``: see :func:`round_to`.  ``return_residuals``: the residual stream after
    every layer, [layers, T, H], instead of the logits.  ``return_cache``: what a cache holds after
    the sequence, instead of the logits: {"kv": [attention layers, 2, T, kv heads, head_dim] (keys after
    norm and rotation, values), "state": [conv layers, k-1, H] (the last k-1 values of B*x)}.
    """
    d = plain_dims(cfg)
    H, eps = d["H"], d["eps"]
    tok = torch.as_tensor(tokens, dtype=torch.long)
    E = _w(weights, "model.embed_tokens.weight", dtype)
    x = E[tok]
    residuals, kept_kv, kept_state = [], [], []
    for i, kind in enumerate(d["layer_types"]):
        pre = f"model.layers.{i}."
        u = rnd(plain_rms_norm(x, _w(weights, pre + "operator_norm.weight", dtype), eps))
        if kind == "conv":
            b = d["bias"]
            y, state = plain_short_conv(
                u,
                _w(weights, pre + "conv.in_proj.weight", dtype),
                _w(weights, pre + "conv.conv.weight", dtype),
                _w(weights, pre + "conv.out_proj.weight", dtype),
                _w(weights, pre + "conv.in_proj.bias", dtype) if b else None,
                _w(weights, pre + "conv.conv.bias", dtype) if b else None,
                _w(weights, pre + "conv.out_proj.bias", dtype) if b else None,
                rnd=rnd, return_state=True,
            )
            x = x + y
            kept_state.append(state)
        elif kind == "full_attention":
            y, (k_, v_) = plain_attention(
                u,
                _w(weights, pre + "self_attn.q_proj.weight", dtype),
                _w(weights, pre + "self_attn.k_proj.weight", dtype),
                _w(weights, pre + "self_attn.v_proj.weight", dtype),
                _w(weights, pre + "self_attn.out_proj.weight", dtype),
                _opt(weights, pre + "self_attn.q_layernorm.weight", dtype),
                _opt(weights, pre + "self_attn.k_layernorm.weight", dtype),
                nh=d["nh"], nkv=d["nkv"], hd=d["hd"], eps=eps, theta=d["theta"],
                style=d["rope_style"], rnd=rnd, return_kv=True,
            )
            x = x + y
            kept_kv.append(torch.stack([k_, v_]))
        else:
            raise ValueError(kind)
        g = rnd(plain_rms_norm(x, _w(weights, pre + "ffn_norm.weight", dtype), eps))
        x = x + plain_swiglu(
            g,
            _w(weights, pre + "feed_forward.w1.weight", dtype),
            _w(weights, pre + "feed_forward.w3.weight", dtype),
            _w(weights, pre + "feed_forward.w2.weight", dtype),
            rnd=rnd,
        )
        residuals.append(x)
    if return_residuals:
        return torch.stack(residuals)
    if return_cache:
        return {"kv": torch.stack(kept_kv) if kept_kv else None,
                "state": torch.stack(kept_state) if kept_state else None}
    f = rnd(plain_rms_norm(x, _w(weights, "model.embedding_norm.weight", dtype), eps))
    if return_hidden:
        return f
    W = E if d["tied"] else _w(weights, "lm_head.weight", dtype)
    return f @ W.T


# --------------------------------------------------------------------------
# sampling (crates/mivi-model/src/sampler.rs)
# --------------------------------------------------------------------------
_MASK64 = (1 << 64) - 1


def plain_uniform(seed: int, stream: int, step: int) -> float:
    """The uniform number in [0, 1) that sequence ``stream`` draws at decoding
    step ``step``.

    The reference keeps one xorshift64* state for its single sequence and
    takes the top 24 bits of each output (sampler.rs:70-76).  A batch needs a
    draw that does not depend on what else is in the batch, so the build
    defines a counter-based stream: a splitmix64 finaliser over
    (seed, stream, step), top 24 bits / 2^24.  This function restates that
    definition; it is the specification that the kernel is tested against.
    """
    def mix(z: int) -> int:
        z = (z + 0x9E3779B97F4A7C15) & _MASK64
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
        return z ^ (z >> 31)
    z = mix(seed & _MASK64)
    z = mix(z ^ ((stream * 0xD1342543DE82EF95) & _MASK64))
    z = mix(z ^ ((step * 0xA24BAED4963EE407) & _MASK64))
    return (z >> 40) / 16777216.0


def plain_sample(logits: torch.Tensor, *, temperature: float = 0.0, top_k: int = 0,
                 top_p: float = 1.0, min_p: float = 0.0, repetition_penalty: float = 1.0,
                 presence_penalty: float = 0.0, frequency_penalty: float = 0.0,
                 recent=(), u: float = 0.0) -> int:
    """One token from a row of logits, in the reference's order
    (sampler.rs:92-136): penalties over the recent tokens (222-260), greedy if
    temperature <= 0 (first maximum wins, 305-315), temperature (282-287),
    min-p (263-279), top-k keeping ties at the k-th value (290-302), softmax,
    then the nucleus (150-218) or the plain categorical draw (138-148).
    All in float32 like the reference; ``u`` is the uniform draw.

    The nucleus is the shortest prefix, in descending order of probability
    (ties: lower index first), whose mass reaches top_p; the draw is
    u * mass walked over the kept tokens in index order, which gives every
    kept token the same probability as the reference's walk in sorted order.
    """
    x = logits.to(torch.float32).clone()
    V = x.numel()
    recent = [int(t) for t in recent if 0 <= int(t) < V]
    if recent and ((repetition_penalty > 0.0 and repetition_penalty != 1.0)
                   or presence_penalty != 0.0 or frequency_penalty != 0.0):
        seen = []
        for t in recent:
            if t in seen:
                continue
            seen.append(t)
            count = recent.count(t)
            if repetition_penalty > 0.0 and repetition_penalty != 1.0:
                rp = torch.tensor(repetition_penalty, dtype=torch.float32)
                x[t] = x[t] / rp if x[t] > 0 else x[t] * rp
            if presence_penalty != 0.0:
                x[t] = x[t] - torch.tensor(presence_penalty, dtype=torch.float32)
            if frequency_penalty != 0.0:
                x[t] = x[t] - torch.tensor(frequency_penalty, dtype=torch.float32) * float(count)
    if temperature <= 0.0:
        return int(torch.argmax(x))          # torch returns the first maximum
    x = x * (torch.tensor(1.0, dtype=torch.float32) / torch.tensor(temperature, dtype=torch.float32))
    if 0.0 < min_p < 1.0:
        thr = x.max() + torch.log(torch.tensor(min_p, dtype=torch.float32))
        x = torch.where(x < thr, torch.tensor(float("-inf")), x)
    if 0 < top_k < V:
        kth = torch.topk(x, top_k).values[-1]
        x = torch.where(x < kth, torch.tensor(float("-inf")), x)
    m = x.max()
    e = torch.exp(x - m)
    e = torch.where(torch.isfinite(x), e, torch.zeros_like(e))
    p = (e.double() / e.double().sum())      # float64 sums: the order of a float32 sum is not part of the spec
    keep = torch.ones(V, dtype=torch.bool)
    if top_p < 1.0:
        order = sorted(range(V), key=lambda i: (-float(p[i]), i))
        keep[:] = False
        mass = 0.0
        for i in order:
            if float(p[i]) <= 0.0:
                break
            keep[i] = True
            mass += float(p[i])
            if mass >= top_p:
                break
    pk = torch.where(keep, p, torch.zeros_like(p))
    total = float(pk.sum())
    r = u * total
    c = 0.0
    last = 0
    for i in range(V):
        if pk[i] > 0:
            c += float(pk[i])
            last = i
            if r < c:
                return i
    return last


def plain_generate(cfg: dict, weights: dict, prompt, max_new_tokens: int, *, stop_ids=(),
                   seed: int = 0, stream: int = 0, dtype=torch.float64, **sampling) -> list:
    """Generation of one sequence by whole-sequence recomputation.

    The loop of crates/mivi-model/src/model.rs:1131-1230 without its chat
    heuristics: sample from the last position's logits; a stop token ends the
    sequence and is not emitted (1166-1173); else append and go on, up to
    max_new_tokens.  The recent-token window for the penalties holds the last
    64 generated tokens (crates/mivi-model/src/config.rs:11).
    """
    toks = list(prompt)
    out = []
    for step in range(max_new_tokens):
        logits = plain_forward(cfg, weights, toks, dtype=dtype)[-1]
        nxt = plain_sample(logits, recent=out[-64:], u=plain_uniform(seed, stream, step), **sampling)
        if nxt in stop_ids:
            break
        out.append(nxt)
        toks.append(nxt)
    return out
