"""Launch wrappers: one Python function per kernel entry point.

Every wrapper checks what the kernel assumes (device, dtype, contiguity,
shapes, size limits) and raises ``KernelError`` with the offending value
instead of launching; the kernels themselves check nothing.  There is no CPU
implementation behind these functions: a tensor that is not on a CUDA device
is an error, and so is a library that cannot be built.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import Optional

import torch

from .build import DEBUG_CHECKS, load_library

F32, BF16 = 0, 1
MAX_HEAD_DIM = 256
MAX_CONV_K = 16
RECENT_MAX = 64
RECENT_RING = 128


class KernelError(RuntimeError):
    pass


_P, _I, _F, _Q, _UQ = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong, ctypes.c_ulonglong
_SIGNATURES = {
    "core": {
        "mv_embed": [_P, _I, _P, _P, _I, _I, _P],
        "mv_embed_link": [_P, _I, _P, _P, _I, _I, _P, _P, _P, _I, _P],
        "mv_embed_link_partials": [_I],
        "mv_rmsnorm": [_P, _P, _P, _I, _P, _I, _I, _F, _P],
        "mv_swiglu": [_P, _P, _I, _I, _I, _I, _P],
        "mv_copy_to_host": [_P, _P, _Q, _P],
        "mv_delay": [_Q, _P],
        "mv_gemm_simt": [_P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _P],
        "mv_shortconv": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P],
        "mv_shortconv_decode": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P],
        "mv_qk_prepare": [_P, _P, _P, _F, _P, _I, _P, _P, _P, _I, _I, _P, _Q, _I, _P, _I, _I, _I, _I, _I, _P],
        "mv_attention_generic": [_P, _P, _Q, _P, _I, _I, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _P],
        "mv_attention_decode": [_P, _P, _Q, _P, _I, _I, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _F, _I, _I,
                                _I, _I, _P],
        "mv_sample": [_P, _Q, _P, _I, _I, _F, _I, _F, _F, _F, _F, _F, _P, _P, _UQ, _P, _P, _P, _P, _P, _P, _P, _P],
    },
    "bf16": {
        "mv_gemm_small_m": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _I, _I, _I, _F, _P, _P, _P, _I, _P, _Q, _P],
        "mv_gemm_small_m_tile_rows": [_I, _I],
        "mv_gemm_small_m_shortconv": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _I, _I, _I, _F, _P, _Q, _P],
        "mv_gemm_small_m_heads": [_P, _P, _P, _P, _F, _P, _I, _P, _P, _P, _I, _I, _P, _Q, _P, _I, _I, _I, _I,
                                  _P, _I, _I, _I, _F, _P, _Q, _P],
        "mv_gemm_tc": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _I, _I, _I, _F, _P, _P],
        "mv_gemm_tc_pair": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _I, _I, _I, _F, _P, _P, _P, _I, _P, _P],
        "mv_gemm_tc_swap": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _I, _I, _I, _F, _P, _P, _P, _I, _P, _Q, _P, _P],
        "mv_gemm_tc_swap_shortconv": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _I, _I, _I, _F, _P, _Q,
                                      _P, _P],
        "mv_gemm_tc_swap_heads": [_P, _P, _P, _P, _F, _P, _P, _P, _P, _I, _I, _P, _Q, _P, _I, _I, _I, _I,
                                  _P, _I, _I, _I, _F, _P, _Q, _P, _P],
        "mv_attention_prefill": [_P, _P, _Q, _P, _I, _I, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _P],
        "mv_attention_decode_tc": [_P, _P, _Q, _P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _F, _I, _P, _P],
        "mv_attention_prefill_tc": [_P, _P, _Q, _P, _I, _P, _P, _P, _I, _I, _I, _I, _F, _P, _P],
    },
}
_fns = {}


class KernelProfile:
    """Device time of every launch made while it is active, by stage of the model and by entry point,
    with the bytes and floating-point operations that the launch's wrapper accounts for it.

    The reference times the stages of its forward pass behind a switch (embedding, attention and its
    stages, the convolution layers and their stages, logits: crates/mivi-model/src/model.rs:57-74,
    273-293) and prints them from its ``bench`` command.  Here every launch is bracketed by two CUDA
    events on the launching stream; that keeps consecutive kernels from overlapping, so the sum is a
    little more than what the same step takes when it is replayed from a recording."""

    def __init__(self):
        self.records = []            # [stage, entry point, start event, end event, bytes, flops]
        self.stage = "-"
        self.steps = 0

    def wrap(self, name: str, f):
        def timed(*args):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            code = f(*args)
            e1.record()
            self.records.append([self.stage, name, e0, e1, 0, 0])
            return code
        return timed

    def account(self, nbytes: int, flops: int) -> None:
        if self.records:
            self.records[-1][4] += int(nbytes)
            self.records[-1][5] += int(flops)

    def report(self, reset: bool = True) -> dict:
        """{"rows": [{stage, kernel, calls, us, share, gb_per_s, tflops}], "stages": {stage: us}, "total_us",
        "steps"}: rows sorted by time.  Waits for the device."""
        torch.cuda.synchronize()
        agg = {}
        for stage, name, e0, e1, nbytes, flops in self.records:
            row = agg.setdefault((stage, name), [0, 0.0, 0, 0])
            row[0] += 1
            row[1] += e0.elapsed_time(e1) * 1e3
            row[2] += nbytes
            row[3] += flops
        total = sum(r[1] for r in agg.values()) or 1.0
        rows = [dict(stage=k[0], kernel=k[1], calls=r[0], us=r[1], share=r[1] / total,
                     gb_per_s=(r[2] / r[1] / 1e3) if r[2] else None, tflops=(r[3] / r[1] / 1e6) if r[3] else None)
                for k, r in sorted(agg.items(), key=lambda kv: -kv[1][1])]
        stages = {}
        for row in rows:
            stages[row["stage"]] = stages.get(row["stage"], 0.0) + row["us"]
        out = dict(rows=rows, stages=stages, total_us=total, steps=self.steps)
        if reset:
            self.records, self.steps = [], 0
        return out


_profile: Optional[KernelProfile] = None


class _NoStage:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_STAGE = _NoStage()


class _Stage:
    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        self.prev, _profile.stage = _profile.stage, self.name

    def __exit__(self, *exc):
        if _profile is not None:
            _profile.stage = self.prev
        return False


def profile_stage(name: str):
    """``with profile_stage("mixer gqa"):`` names the stage of the launches inside, when a profile is active."""
    return _Stage(name) if _profile is not None else _NO_STAGE


class profiling:
    """``with profiling(p):`` every launch inside is timed into ``p`` (a KernelProfile, or None: nothing)."""

    def __init__(self, p: Optional[KernelProfile]):
        self.p = p

    def __enter__(self):
        global _profile
        self.prev, _profile = _profile, self.p
        return self.p

    def __exit__(self, *exc):
        global _profile
        _profile = self.prev
        return False


def delay(us: int) -> None:
    """Keep the current stream busy for ``us`` microseconds (at most 50,000)."""
    code = _fn("core", "mv_delay")(int(us), _stream())
    if code != 0:
        raise KernelError(f"mv_delay: launch failed with CUDA error {code}")


def profiling_on() -> bool:
    return _profile is not None


def account(nbytes: int = 0, flops: int = 0) -> None:
    """Bytes that the last launch has to move and operations it has to do, for the active profile."""
    if _profile is not None:
        _profile.account(nbytes, flops)


def _nbytes(*tensors) -> int:
    return sum(t.numel() * t.element_size() for t in tensors if t is not None)


def _fn(lib: str, name: str):
    key = (lib, name)
    f = _fns.get(key)
    if f is None:
        f = getattr(load_library(lib), name)
        f.argtypes = _SIGNATURES[lib][name]
        f.restype = ctypes.c_int
        _fns[key] = f
    if _profile is not None and not name.endswith(("_partials", "_tile_rows", "_to_host", "_delay")):
        return _profile.wrap(name, f)
    return f


def _guard(lib: str, file: str, device, n_pages: int = 0x7fffffff, n_slots: int = 0x7fffffff) -> None:
    """In a build with index checks: declare, for the kernels of one source file, how many pages and slots
    the tensors of the next launch really have.  Nothing in an ordinary build."""
    if not DEBUG_CHECKS:
        return
    name = "mv_set_guard_" + file
    f = _fns.get((lib, name))
    if f is None:
        f = getattr(load_library(lib), name)
        f.argtypes = [_I, _I, _P, _P]
        f.restype = ctypes.c_int
        _fns[(lib, name)] = f
    code = f(int(min(n_pages, 0x7fffffff)), int(min(n_slots, 0x7fffffff)), _error_flag(device).data_ptr(), _stream())
    if code != 0:
        raise KernelError(f"{name}: CUDA error {code}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    """The current CUDA stream's handle.  A step asks a hundred times: the two direct calls cost a
    tenth of building a ``torch.cuda.Stream`` object each time."""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported dtype {t.dtype}; the kernels take float32 and bfloat16")


def _need(t: Optional[torch.Tensor], name: str, dtype=None, shape=None, optional=False):
    if t is None:
        if optional:
            return None
        raise KernelError(f"{name}: missing tensor")
    if not t.is_cuda:
        raise KernelError(f"{name}: tensor is on {t.device}; this library runs on CUDA devices only")
    if not t.is_contiguous():
        raise KernelError(f"{name}: tensor is not contiguous (strides {t.stride()})")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: dtype {t.dtype}, expected {dtype}")
    if shape is not None:
        have = t.shape
        bad = len(shape) != len(have)
        if not bad:
            for s, d in zip(shape, have):         # a plain loop: this runs hundreds of times a step
                if s is not None and s != d:
                    bad = True
                    break
        if bad:
            raise KernelError(f"{name}: shape {tuple(have)}, expected {tuple(shape)}")
    return t.data_ptr()


_launches = 0
# kernels launched by one call of each entry point
_KERNELS_PER_CALL = {"mv_shortconv": 2}


def launch_count() -> int:
    """Kernels of this library launched so far in this process."""
    return _launches


def add_launches(n: int) -> None:
    """Kernels that ran without passing through a wrapper (a replayed CUDA graph)."""
    global _launches
    _launches += n


def _check(code: int, name: str) -> None:
    global _launches
    if code != 0:
        raise KernelError(f"{name}: launch failed with CUDA error {code}")
    _launches += _KERNELS_PER_CALL.get(name, 1)


# --------------------------------------------------------------------------
def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor,
          emit: Optional["NormLink"] = None) -> torch.Tensor:
    """out[n, :] = table[tokens[n], :] widened to float32.  ``emit``: a :class:`NormLink` whose rows
    bf16(out * weight) and partial sums of squares the kernel writes too, for the product after it."""
    N = tokens.numel()
    V, H = table.shape
    if emit is not None:
        n_part = int(_fn("core", "mv_embed_link_partials")(H))
        _need(emit.partials, "norm partials", torch.float32)
        if emit.dim != H or emit.partials.dim() != 2 or emit.partials.shape[0] < N or emit.partials.shape[1] < n_part:
            raise KernelError(f"embed: a norm link of width {emit.dim} with partials "
                              f"{tuple(emit.partials.shape)} cannot take {N} rows of {H}")
        _check(_fn("core", "mv_embed_link")(
            _need(table, "embedding table"), _dt(table), _need(tokens, "tokens", torch.int32),
            _need(out, "embedding out", torch.float32, (N, H)), N, H,
            _need(emit.weight, "norm weight", torch.float32, (H,)),
            _need(emit.xg, "normed rows", torch.bfloat16, (N, H)), emit.partials.data_ptr(), emit.partials.shape[1],
            _stream()), "mv_embed_link")
        emit.n_partials = n_part
        account(N * H * (table.element_size() + 4 + 2))
        return out
    _check(_fn("core", "mv_embed")(
        _need(table, "embedding table"), _dt(table), _need(tokens, "tokens", torch.int32),
        _need(out, "embedding out", torch.float32, (N, H)), N, H, _stream()), "mv_embed")
    account(N * H * (table.element_size() + 4))
    return out


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[i] = rmsnorm(x[rows[i]] or x[i]) * w, statistics in float32."""
    H = x.shape[-1]
    n = rows.numel() if rows is not None else x.shape[0]
    _check(_fn("core", "mv_rmsnorm")(
        _need(x, "rmsnorm x", torch.float32), _need(w, "rmsnorm weight", torch.float32, (H,)),
        _need(out, "rmsnorm out", None, (n, H)), _dt(out),
        _need(rows, "rmsnorm rows", torch.int32, optional=True), n, H, float(eps), _stream()), "mv_rmsnorm")
    account(n * H * (4 + out.element_size()))
    return out


SWIGLU_GROUP = 16


def swiglu(gu: torch.Tensor, out: torch.Tensor, group: int = 0) -> torch.Tensor:
    """out[n, f] = silu(gate) * up.  ``group`` 0: gate and up are the two halves
    of a row of ``gu``; 16: they alternate in groups of 16 columns."""
    N, F2 = gu.shape
    F = F2 // 2
    if group and F % group:
        raise KernelError(f"swiglu: width {F} is not a multiple of the group size {group}")
    _check(_fn("core", "mv_swiglu")(
        _need(gu, "swiglu in", torch.float32), _need(out, "swiglu out", None, (N, F)), _dt(out), N, F, int(group),
        _stream()), "mv_swiglu")
    account(_nbytes(gu, out))
    return out


STORE, ACCUMULATE = "store", "accumulate"


def _account_gemm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool) -> None:
    if _profile is not None:
        account(_nbytes(x, w) + (2 if accumulate else 1) * out.numel() * out.element_size(),
                2 * x.shape[0] * w.shape[0] * w.shape[1])


def gemm_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, bias: Optional[torch.Tensor] = None,
              accumulate: bool = False) -> torch.Tensor:
    """out = x @ w.T (+ bias), or out += ... when ``accumulate`` (out float32).
    CUDA-core kernel, float32 accumulation, any sizes."""
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelError(f"gemm: x is [{M}, {K}] but w is [{N}, {K2}]")
    if x.dtype != w.dtype:
        raise KernelError(f"gemm: x is {x.dtype} but w is {w.dtype}")
    if accumulate:
        mode = 2
        _need(out, "gemm out", torch.float32, (M, N))
    else:
        mode = 0 if out.dtype == torch.float32 else 1
        _need(out, "gemm out", None, (M, N))
        _dt(out)
    _check(_fn("core", "mv_gemm_simt")(
        _need(x, "gemm x"), _need(w, "gemm w"), _dt(x), _need(bias, "gemm bias", torch.float32, (N,), True),
        out.data_ptr(), mode, M, N, K, N, _stream()), "mv_gemm_simt")
    _account_gemm(x, w, out, accumulate)
    return out


SMALL_M_MAX = 64




@dataclass
class NormLink:
    """A norm carried by the two products around it, in a step of few tokens.  The product
    that completes the residual stream (``emit``) also writes ``xg`` = bf16(x_new * weight)
    and, per tile of its rows, the sum of x_new^2 into ``partials``; the product that reads
    the normed rows (``scale``) takes ``xg`` as its input and multiplies every token's
    results by rsqrt(sum(partials) / dim + eps).  Statistics and scale are float32."""
    norm: object                   # the norm part this stands for (identity only)
    weight: torch.Tensor           # float32 [dim]
    eps: float
    dim: int
    xg: torch.Tensor               # bfloat16 [tokens, dim]
    partials: torch.Tensor         # float32 [tokens, >= ceil(dim / 16)]: the tile sums of one token lie together
    n_partials: int = 0            # set by the emitting product


def gemm_small_m_tile_rows(N: int, mode: int) -> int:
    return int(_fn("bf16", "mv_gemm_small_m_tile_rows")(int(N), int(mode)))


def gemm_small_m(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, bias: Optional[torch.Tensor] = None,
                 accumulate: bool = False, swiglu: bool = False, scale: Optional[NormLink] = None,
                 emit: Optional[NormLink] = None, ahead: Optional[tuple] = None) -> torch.Tensor:
    """out = x @ w.T for at most 64 rows of x, bfloat16 operands: the
    weight-streaming tensor-core kernel of the decode step.  ``scale`` / ``emit``: the
    two ends of a :class:`NormLink`.  ``ahead``: (address, bytes) of what the step's next
    product will read; the kernel asks the L2 cache for it once it has its own weights."""
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelError(f"gemm: x is [{M}, {K}] but w is [{N}, {K2}]")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"gemm_small_m: operands must be bfloat16, got {x.dtype} and {w.dtype}")
    if not 1 <= M <= SMALL_M_MAX or K % 8:
        raise KernelError(f"gemm_small_m: needs 1..{SMALL_M_MAX} rows and K a multiple of 8, got M={M}, K={K}")
    ldo = N
    if swiglu:
        if N % 32:
            raise KernelError(f"gemm_small_m: the SwiGLU epilogue needs rows in groups of 32, got {N}")
        mode, ldo = 3, N // 2
        _need(out, "gemm out", torch.bfloat16, (M, N // 2))
    elif accumulate:
        mode = 2
        _need(out, "gemm out", torch.float32, (M, N))
    else:
        mode = 0 if out.dtype == torch.float32 else 1
        _need(out, "gemm out", None, (M, N))
        _dt(out)
    link = _link_args(x, M, N, K, mode, scale, emit, -(-N // gemm_small_m_tile_rows(N, 2)))
    _check(_fn("bf16", "mv_gemm_small_m")(
        _need(x, "gemm x"), _need(w, "gemm w"), _need(bias, "gemm bias", torch.float32, (N,), True),
        out.data_ptr(), mode, M, N, K, ldo, *link, *(ahead or (None, 0)), _stream()), "mv_gemm_small_m")
    _account_gemm(x, w, out, accumulate)
    return out


SHORTCONV_FUSED_MAX_ROWS = 8


def gemm_small_m_shortconv(x: torch.Tensor, w_in: torch.Tensor, b_in: Optional[torch.Tensor], taps: torch.Tensor,
                           b_conv: Optional[torch.Tensor], state: torch.Tensor, slots: torch.Tensor,
                           out: torch.Tensor, *, scale: Optional[NormLink] = None,
                           ahead: Optional[tuple] = None) -> torch.Tensor:
    """A decode step's gated short convolution together with its input projection, in one kernel:
    [B | C | x] = x @ w_in.T (+ b_in), out = C * conv(B * x) with the sequences' kept values in
    ``state`` [n_slots, k-1, H], which it shifts and updates for the rows' sequences (``slots[m]`` is
    row m's).  At most 8 rows, one a sequence; bfloat16 operands; ``scale`` and ``ahead`` as in
    ``gemm_small_m``."""
    M, K = x.shape
    H, k = taps.shape
    if tuple(w_in.shape) != (3 * H, K):
        raise KernelError(f"shortconv: in_proj weight is {tuple(w_in.shape)}, expected [{3 * H}, {K}]")
    if x.dtype != torch.bfloat16 or w_in.dtype != torch.bfloat16:
        raise KernelError(f"gemm_small_m_shortconv: operands must be bfloat16, got {x.dtype} and {w_in.dtype}")
    if not 1 <= M <= SHORTCONV_FUSED_MAX_ROWS or K % 8:
        raise KernelError(f"gemm_small_m_shortconv: needs 1..{SHORTCONV_FUSED_MAX_ROWS} rows and K a multiple "
                          f"of 8, got M={M}, K={K}")
    if not 1 <= k <= MAX_CONV_K:
        raise KernelError(f"shortconv: convolution width {k} is outside 1..{MAX_CONV_K}")
    _need(state, "shortconv state", torch.float32)
    if state.dim() != 3 or state.shape[1] != k - 1 or state.shape[2] != H:
        raise KernelError(f"shortconv: state shape {tuple(state.shape)}, expected [slots, {k - 1}, {H}]")
    if slots.numel() < M:
        raise KernelError(f"shortconv: {slots.numel()} slots for {M} rows")
    sp, n_sp, s_stride, dim, eps = _link_args(x, M, 3 * H, K, 1, scale, None, 0)[:5]
    _check(_fn("bf16", "mv_gemm_small_m_shortconv")(
        _need(x, "gemm x"), _need(w_in, "gemm w"), _need(b_in, "in_proj bias", torch.float32, (3 * H,), True),
        _need(taps, "shortconv taps", torch.float32), _need(b_conv, "shortconv bias", torch.float32, (H,), True),
        state.data_ptr(), _need(slots, "slots", torch.int32), _need(out, "shortconv out", torch.bfloat16, (M, H)),
        M, H, K, k, sp, n_sp, s_stride, dim, eps, *(ahead or (None, 0)), _stream()), "mv_gemm_small_m_shortconv")
    _account_gemm(x, w_in, out, False)
    return out


HEADS_FUSED_HEAD_DIM = 64


def gemm_small_m_heads(x: torch.Tensor, w_qkv: torch.Tensor, wq: Optional[torch.Tensor], wk: Optional[torch.Tensor],
                       eps: float, inv_freq: Optional[torch.Tensor], half_split: bool, positions, seq_of,
                       page_table, pool: torch.Tensor, q_out: torch.Tensor, nh: int, nkv: int, *,
                       scale: Optional[NormLink] = None, ahead: Optional[tuple] = None) -> torch.Tensor:
    """The fused q/k/v projection together with what ``qk_prepare`` does, in one kernel, for steps of
    at most 8 tokens, heads of 64 and a bfloat16 cache: q comes out normed and rotated in ``q_out``,
    k (normed, rotated) and v go into the tokens' rows of the paged cache.  ``scale`` and ``ahead``
    as in ``gemm_small_m``."""
    M, K = x.shape
    hd = HEADS_FUSED_HEAD_DIM
    if tuple(w_qkv.shape) != ((nh + 2 * nkv) * hd, K):
        raise KernelError(f"gemm_small_m_heads: weight is {tuple(w_qkv.shape)}, expected "
                          f"[{(nh + 2 * nkv) * hd}, {K}] ({nh} + 2 x {nkv} heads of {hd})")
    if x.dtype != torch.bfloat16 or w_qkv.dtype != torch.bfloat16 or pool.dtype != torch.bfloat16:
        raise KernelError(f"gemm_small_m_heads: operands and cache must be bfloat16, got {x.dtype}, "
                          f"{w_qkv.dtype} and {pool.dtype}")
    if not 1 <= M <= SHORTCONV_FUSED_MAX_ROWS or K % 8:
        raise KernelError(f"gemm_small_m_heads: needs 1..{SHORTCONV_FUSED_MAX_ROWS} rows and K a multiple "
                          f"of 8, got M={M}, K={K}")
    page_size = pool.shape[3]
    _check_kv(pool, nkv, hd, page_size, "gemm_small_m_heads")
    _need(page_table, "page table", torch.int32)
    sp, n_sp, s_stride, dim, eps_norm = _link_args(x, M, (nh + 2 * nkv) * hd, K, 1, scale, None, 0)[:5]
    _check(_fn("bf16", "mv_gemm_small_m_heads")(
        _need(x, "gemm x"), _need(w_qkv, "gemm w"), _need(wq, "q norm weight", torch.float32, (hd,), True),
        _need(wk, "k norm weight", torch.float32, (hd,), True), float(eps),
        _need(inv_freq, "inv_freq", torch.float32, (hd // 2,), True), int(half_split),
        _need(positions, "positions", torch.int32), _need(seq_of, "seq_of", torch.int32),
        page_table.data_ptr(), page_table.shape[1], page_size, _need(pool, "cache pool"), pool.stride(0),
        _need(q_out, "q out", torch.bfloat16, (M, nh * hd)), M, nh, nkv, K, sp, n_sp, s_stride, dim, eps_norm,
        *(ahead or (None, 0)), _stream()), "mv_gemm_small_m_heads")
    _account_gemm(x, w_qkv, q_out, False)
    return q_out


def _link_args(x, M: int, N: int, K: int, mode: int, scale: Optional[NormLink], emit: Optional[NormLink],
               tiles: int):
    """The nine arguments that carry a norm through a product: (partials, count, stride, dim, eps)
    of the link it consumes and (weight, rows, partials, stride) of the link it emits, which
    writes ``tiles`` sums a row."""
    sp, n_sp, s_stride, dim, eps, eg, ex, ep, e_stride = None, 0, 0, 0, 0.0, None, None, None, 0
    if scale is not None:
        if scale.n_partials <= 0 or scale.dim != K or x.data_ptr() != scale.xg.data_ptr():
            raise KernelError("gemm: the scaled input must be the rows that the norm link's producer wrote")
        _need(scale.partials, "norm partials", torch.float32)
        sp, n_sp, s_stride = scale.partials.data_ptr(), scale.n_partials, scale.partials.shape[1]
        dim, eps = scale.dim, float(scale.eps)
    if emit is not None:
        if mode != 2 or emit.dim != N:
            raise KernelError("gemm: only a product that adds into the residual stream can emit a norm")
        _need(emit.weight, "norm weight", torch.float32, (N,))
        _need(emit.xg, "normed rows", torch.bfloat16, (M, N))
        _need(emit.partials, "norm partials", torch.float32)
        if emit.partials.dim() != 2 or emit.partials.shape[0] < M or emit.partials.shape[1] < tiles:
            raise KernelError(f"gemm: norm partials [{tuple(emit.partials.shape)}] cannot hold {tiles} tile "
                              f"sums for each of {M} rows")
        eg, ex, ep, e_stride = emit.weight.data_ptr(), emit.xg.data_ptr(), emit.partials.data_ptr(), emit.partials.shape[1]
        emit.n_partials = tiles
    return sp, n_sp, s_stride, dim, eps, eg, ex, ep, e_stride


_error_flags = {}
_error_mirrors = {}
_ERROR_ROLES = {1: "the TMA producer", 2: "the MMA issuer", 3: "the epilogue", 4: "a guarded index"}


def _error_flag(device) -> torch.Tensor:
    """One int per device that a kernel sets when one of its bounded waits ran out (or, in a build
    with index checks, when an index lay outside its bounds)."""
    key = torch.device(device).index or 0
    if key not in _error_flags:
        _error_flags[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _error_flags[key]


def _error_text(key: int, code: int) -> str:
    role = _ERROR_ROLES.get(code, f"code {code}")
    if code == 4:
        return (f"a kernel on cuda:{key} was handed an index outside its bounds (a page or a slot); it skipped "
                f"the access and its output is not valid")
    return (f"a tensor-core kernel on cuda:{key} gave up waiting on a barrier in {role}; "
            f"its output is not valid")


def note_device_errors(device) -> None:
    """Enqueue a copy of the device's error flag into pinned host memory, on the current stream
    (may be recorded into a CUDA graph).  ``raise_seen_device_errors`` looks at that copy."""
    key = torch.device(device).index or 0
    mirror = _error_mirrors.get(key)
    if mirror is None:
        mirror = torch.zeros(1, dtype=torch.int32).pin_memory()
        _error_mirrors[key] = mirror
    code = _fn("core", "mv_copy_to_host")(mirror.data_ptr(), _error_flag(device).data_ptr(), 4, _stream())
    if code != 0:
        raise KernelError(f"copying the error flag to the host failed with CUDA error {code}")


def raise_seen_device_errors(device) -> None:
    """Raise if a copy of the error flag that has arrived on the host is set; does not wait for the
    device.  Exact where the host has just waited for work enqueued after ``note_device_errors``."""
    key = torch.device(device).index or 0
    mirror = _error_mirrors.get(key)
    if mirror is None:
        return
    code = int(mirror[0])
    if code:
        torch.cuda.synchronize(device)
        _error_flags[key].zero_()
        torch.cuda.synchronize(device)
        mirror.zero_()
        raise KernelError(_error_text(key, code))


def raise_device_error(device, code: int) -> None:
    """A kernel's fault arrived on the host by another way than the mirror (with the sampled tokens):
    clear the flag and raise."""
    key = torch.device(device).index or 0
    torch.cuda.synchronize(device)
    _error_flag(device).zero_()
    torch.cuda.synchronize(device)
    if key in _error_mirrors:
        _error_mirrors[key].zero_()
    raise KernelError(_error_text(key, int(code)))


def check_device_errors() -> None:
    """Raise if a kernel reported a fault (synchronises the device)."""
    for key, flag in _error_flags.items():
        code = int(flag.item())
        if code:
            flag.zero_()
            if key in _error_mirrors:
                torch.cuda.synchronize(flag.device)
                _error_mirrors[key].zero_()
            raise KernelError(_error_text(key, code))


_PREFILL_GEMM = os.environ.get("MIVI_PREFILL_GEMM", "auto")      # pair | single | auto


def gemm_tc_pair_takes(M: int, N: int) -> bool:
    """Shapes for which two multiprocessors share a 256 x 256 tile (``gemm_tc_pair.cu``): more than
    128 rows, and enough tiles that most pairs of the device get one."""
    if _PREFILL_GEMM == "single" or M <= 128 or N < 128:
        return False
    tiles = -(-M // 256) * -(-N // 256)
    return _PREFILL_GEMM == "pair" or tiles >= 48 * n_sms() // 148


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, bias: Optional[torch.Tensor] = None,
            accumulate: bool = False, swiglu: bool = False, pair: Optional[bool] = None,
            scale: Optional[NormLink] = None, emit: Optional[NormLink] = None) -> torch.Tensor:
    """out = x @ w.T, bfloat16 operands, on the tcgen05 tensor cores (TMA
    loads, accumulator in tensor memory): the matrix product of prefill.
    ``pair``: True: the kernel in which two multiprocessors share a 256 x 256 tile, False: the
    one-multiprocessor kernels, None: by shape (``gemm_tc_pair_takes``).  ``scale`` / ``emit``: the two
    ends of a :class:`NormLink`; every kernel here applies a scale, only the pair kernel emits (N in
    steps of 32)."""
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelError(f"gemm: x is [{M}, {K}] but w is [{N}, {K2}]")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"gemm_tc: operands must be bfloat16, got {x.dtype} and {w.dtype}")
    if K % 8 or K < 8:
        raise KernelError(f"gemm_tc: K must be a multiple of 8 (16-byte rows for TMA), got {K}")
    ldo = N
    if swiglu:
        if N % 32:
            raise KernelError(f"gemm_tc: the SwiGLU epilogue needs rows in groups of 32, got {N}")
        mode, ldo = 3, N // 2
        _need(out, "gemm out", torch.bfloat16, (M, N // 2))
    elif accumulate:
        mode = 2
        _need(out, "gemm out", torch.float32, (M, N))
    else:
        mode = 0 if out.dtype == torch.float32 else 1
        _need(out, "gemm out", None, (M, N))
        _dt(out)
    if pair is None:
        pair = gemm_tc_pair_takes(M, N) or (emit is not None and M > 128 and N >= 128)
    elif pair and (M <= 128 or N < 128):
        raise KernelError(f"gemm_tc: the pair kernel needs more than 128 rows and at least 128 columns, got {M} x {N}")
    if pair:
        if emit is not None and N % 32:
            raise KernelError(f"gemm_tc: a product that emits a norm needs N in steps of 32, got {N}")
        link = _link_args(x, M, N, K, mode, scale, emit, -(-N // 256))
        _check(_fn("bf16", "mv_gemm_tc_pair")(
            _need(x, "gemm x"), _need(w, "gemm w"), _need(bias, "gemm bias", torch.float32, (N,), True),
            out.data_ptr(), mode, M, N, K, ldo, *link, _error_flag(x.device).data_ptr(), _stream()), "mv_gemm_tc_pair")
        _account_gemm(x, w, out, accumulate)
        return out
    if emit is not None:
        raise KernelError("gemm_tc: only the kernel of two multiprocessors a tile emits a norm")
    link = _link_args(x, M, N, K, mode, scale, None, 0)
    entry = "mv_gemm_tc"
    _check(_fn("bf16", entry)(
        _need(x, "gemm x"), _need(w, "gemm w"), _need(bias, "gemm bias", torch.float32, (N,), True),
        out.data_ptr(), mode, M, N, K, ldo, *link[:5], _error_flag(x.device).data_ptr(), _stream()), entry)
    _account_gemm(x, w, out, accumulate)
    return out


def gemm_tc_swap(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, bias: Optional[torch.Tensor] = None,
                 accumulate: bool = False, swiglu: bool = False, scale: Optional[NormLink] = None,
                 emit: Optional[NormLink] = None, ahead: Optional[tuple] = None) -> torch.Tensor:
    """out = x @ w.T on the tcgen05 tensor cores with the operands' roles swapped (rows of w
    on the MMA's M side, up to 256 tokens a tile on its N side): a TMA pipeline that streams w
    once, K cut over the blocks of a cluster.  Same contract as ``gemm_small_m``, for any number of
    rows: the kernel of steps whose cost is reading the weights."""
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelError(f"gemm: x is [{M}, {K}] but w is [{N}, {K2}]")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"gemm_tc_swap: operands must be bfloat16, got {x.dtype} and {w.dtype}")
    if M < 1 or K % 8 or K < 8:
        raise KernelError(f"gemm_tc_swap: needs at least one row and K a multiple of 8, got M={M}, K={K}")
    ldo = N
    if swiglu:
        if N % 32:
            raise KernelError(f"gemm_tc_swap: the SwiGLU epilogue needs rows in groups of 32, got {N}")
        mode, ldo = 3, N // 2
        _need(out, "gemm out", torch.bfloat16, (M, N // 2))
    elif accumulate:
        mode = 2
        _need(out, "gemm out", torch.float32, (M, N))
    else:
        mode = 0 if out.dtype == torch.float32 else 1
        _need(out, "gemm out", None, (M, N))
        _dt(out)
    link = _link_args(x, M, N, K, mode, scale, emit, -(-N // 128))
    _check(_fn("bf16", "mv_gemm_tc_swap")(
        _need(x, "gemm x"), _need(w, "gemm w"), _need(bias, "gemm bias", torch.float32, (N,), True),
        out.data_ptr(), mode, M, N, K, ldo, *link, *(ahead or (None, 0)), _error_flag(x.device).data_ptr(), _stream()),
        "mv_gemm_tc_swap")
    _account_gemm(x, w, out, accumulate)
    return out


def gemm_tc_swap_shortconv(x: torch.Tensor, w_in: torch.Tensor, b_in: Optional[torch.Tensor], taps: torch.Tensor,
                           b_conv: Optional[torch.Tensor], state: torch.Tensor, slots: torch.Tensor,
                           out: torch.Tensor, *, scale: Optional[NormLink] = None,
                           ahead: Optional[tuple] = None) -> torch.Tensor:
    """``gemm_small_m_shortconv`` for up to 64 rows, on the tcgen05 kernel with swapped operands.  The rows
    of ``w_in`` come regrouped by :func:`group_conv_rows` (32 channels' B, C and x rows together; the width a
    multiple of 32), so that a block's one tile holds all three of its channels."""
    M, K = x.shape
    H, k = taps.shape
    if H % CONV_ROW_GROUP:
        raise KernelError(f"shortconv: regrouped rows need a width in steps of {CONV_ROW_GROUP}, got {H}")
    if tuple(w_in.shape) != (3 * H, K):
        raise KernelError(f"shortconv: in_proj weight is {tuple(w_in.shape)}, expected [{3 * H}, {K}]")
    if x.dtype != torch.bfloat16 or w_in.dtype != torch.bfloat16:
        raise KernelError(f"gemm_tc_swap_shortconv: operands must be bfloat16, got {x.dtype} and {w_in.dtype}")
    if not 1 <= M <= SMALL_M_MAX or K % 8 or K < 8:
        raise KernelError(f"gemm_tc_swap_shortconv: needs 1..{SMALL_M_MAX} rows and K a multiple of 8, got M={M}, K={K}")
    if not 1 <= k <= MAX_CONV_K:
        raise KernelError(f"shortconv: convolution width {k} is outside 1..{MAX_CONV_K}")
    _need(state, "shortconv state", torch.float32)
    if state.dim() != 3 or state.shape[1] != k - 1 or state.shape[2] != H:
        raise KernelError(f"shortconv: state shape {tuple(state.shape)}, expected [slots, {k - 1}, {H}]")
    if slots.numel() < M:
        raise KernelError(f"shortconv: {slots.numel()} slots for {M} rows")
    sp, n_sp, s_stride, dim, eps = _link_args(x, M, 3 * H, K, 1, scale, None, 0)[:5]
    entry = "mv_gemm_tc_swap_shortconv"
    _check(_fn("bf16", entry)(
        _need(x, "gemm x"), _need(w_in, "gemm w"), _need(b_in, "in_proj bias", torch.float32, (3 * H,), True),
        _need(taps, "shortconv taps", torch.float32), _need(b_conv, "shortconv bias", torch.float32, (H,), True),
        state.data_ptr(), _need(slots, "slots", torch.int32), _need(out, "shortconv out", torch.bfloat16, (M, H)),
        M, H, K, k, sp, n_sp, s_stride, dim, eps, *(ahead or (None, 0)), _error_flag(x.device).data_ptr(), _stream()),
        entry)
    _account_gemm(x, w_in, out, False)
    return out


CONV_ROW_GROUP = 32


def group_conv_rows(w_in: torch.Tensor) -> torch.Tensor:
    """The rows of a short convolution's input projection [3 H, K] (B rows, C rows, x rows) regrouped for
    ``gemm_tc_swap_shortconv``: the B rows of channels 0..31, their C rows, their x rows, then
    the same of channels 32..63, and so on.  A copy; H a multiple of 32."""
    H3, K = w_in.shape
    H = H3 // 3
    if H3 != 3 * H or H % CONV_ROW_GROUP:
        raise KernelError(f"shortconv: cannot regroup the rows of a [{H3}, {K}] projection by {CONV_ROW_GROUP} channels")
    g = CONV_ROW_GROUP
    return w_in.view(3, H // g, g, K).permute(1, 0, 2, 3).reshape(H3, K).contiguous()


def gemm_tc_swap_heads(x: torch.Tensor, w_qkv: torch.Tensor, wq: Optional[torch.Tensor], wk: Optional[torch.Tensor],
                       eps: float, inv_freq: Optional[torch.Tensor], positions, seq_of, page_table,
                       pool: torch.Tensor, q_out: torch.Tensor, nh: int, nkv: int, *,
                       scale: Optional[NormLink] = None, ahead: Optional[tuple] = None) -> torch.Tensor:
    """``gemm_small_m_heads`` for up to 64 tokens, on the tcgen05 kernel with swapped operands (heads of 64,
    the pairs (2i, 2i+1) only): a tile of 128 rows is two heads, a half-warp finishes one for a token."""
    M, K = x.shape
    hd = HEADS_FUSED_HEAD_DIM
    if tuple(w_qkv.shape) != ((nh + 2 * nkv) * hd, K):
        raise KernelError(f"gemm_tc_swap_heads: weight is {tuple(w_qkv.shape)}, expected "
                          f"[{(nh + 2 * nkv) * hd}, {K}] ({nh} + 2 x {nkv} heads of {hd})")
    if x.dtype != torch.bfloat16 or w_qkv.dtype != torch.bfloat16 or pool.dtype != torch.bfloat16:
        raise KernelError(f"gemm_tc_swap_heads: operands and cache must be bfloat16, got {x.dtype}, "
                          f"{w_qkv.dtype} and {pool.dtype}")
    if not 1 <= M <= SMALL_M_MAX or K % 8 or K < 8:
        raise KernelError(f"gemm_tc_swap_heads: needs 1..{SMALL_M_MAX} rows and K a multiple of 8, got M={M}, K={K}")
    page_size = pool.shape[3]
    _check_kv(pool, nkv, hd, page_size, "gemm_tc_swap_heads")
    _need(page_table, "page table", torch.int32)
    sp, n_sp, s_stride, dim, eps_norm = _link_args(x, M, (nh + 2 * nkv) * hd, K, 1, scale, None, 0)[:5]
    _check(_fn("bf16", "mv_gemm_tc_swap_heads")(
        _need(x, "gemm x"), _need(w_qkv, "gemm w"), _need(wq, "q norm weight", torch.float32, (hd,), True),
        _need(wk, "k norm weight", torch.float32, (hd,), True), float(eps),
        _need(inv_freq, "inv_freq", torch.float32, (hd // 2,), True),
        _need(positions, "positions", torch.int32), _need(seq_of, "seq_of", torch.int32),
        page_table.data_ptr(), page_table.shape[1], page_size, _need(pool, "cache pool"), pool.stride(0),
        _need(q_out, "q out", torch.bfloat16, (M, nh * hd)), M, nh, nkv, K, sp, n_sp, s_stride, dim, eps_norm,
        *(ahead or (None, 0)), _error_flag(x.device).data_ptr(), _stream()), "mv_gemm_tc_swap_heads")
    _account_gemm(x, w_qkv, q_out, False)
    return q_out


def shortconv(p: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor,
              positions, seq_of, cu, slots, starts, lens, out: torch.Tensor, n_seqs: int,
              decode: bool = False) -> torch.Tensor:
    """Gated short convolution between its projections; updates ``state``
    [n_slots, k-1, H] in place for the ``n_seqs`` sequences of the step.
    ``decode``: every sequence brings exactly one token (one fused kernel)."""
    N, H3 = p.shape
    H, k = w.shape
    if H3 != 3 * H:
        raise KernelError(f"shortconv: projection width {H3} is not 3 x {H}")
    if not 1 <= k <= MAX_CONV_K:
        raise KernelError(f"shortconv: convolution width {k} is outside 1..{MAX_CONV_K}")
    _need(state, "shortconv state", torch.float32)
    if state.dim() != 3 or state.shape[1] != k - 1 or state.shape[2] != H:
        raise KernelError(f"shortconv: state shape {tuple(state.shape)}, expected [slots, {k - 1}, {H}]")
    _guard("core", "shortconv", p.device, n_slots=state.shape[0])
    if N == n_seqs and decode:
        _check(_fn("core", "mv_shortconv_decode")(
            _need(p, "shortconv p", torch.float32), _need(w, "shortconv taps", torch.float32),
            _need(bias, "shortconv bias", torch.float32, (H,), True), state.data_ptr(),
            _need(slots, "slots", torch.int32), _need(out, "shortconv out", None, (N, H)), _dt(out), N, H, k,
            _stream()), "mv_shortconv_decode")
        account(_nbytes(p, out) + 2 * N * (k - 1) * H * 4)
        return out
    _check(_fn("core", "mv_shortconv")(
        _need(p, "shortconv p", torch.float32), _need(w, "shortconv taps", torch.float32),
        _need(bias, "shortconv bias", torch.float32, (H,), True), state.data_ptr(),
        _need(positions, "positions", torch.int32), _need(seq_of, "seq_of", torch.int32),
        _need(cu, "cu", torch.int32), _need(slots, "slots", torch.int32),
        _need(starts, "starts", torch.int32), _need(lens, "lens", torch.int32),
        _need(out, "shortconv out", None, (N, H)), _dt(out), N, n_seqs, H, k, _stream()), "mv_shortconv")
    account(_nbytes(p, out) + 2 * n_seqs * (k - 1) * H * 4)
    return out


def _check_kv(pool: torch.Tensor, nkv: int, hd: int, page_size: int, what: str):
    if pool.dim() != 5 or tuple(pool.shape[1:]) != (2, nkv, page_size, hd):
        raise KernelError(f"{what}: cache pool shape {tuple(pool.shape)}, expected "
                          f"[pages, 2, {nkv}, {page_size}, {hd}]")
    if page_size & (page_size - 1):
        raise KernelError(f"{what}: page size {page_size} is not a power of two")


def qk_prepare(qkv: torch.Tensor, wq: Optional[torch.Tensor], wk: Optional[torch.Tensor], eps: float,
               inv_freq: Optional[torch.Tensor], half_split: bool, positions, seq_of, page_table,
               pool: torch.Tensor, q_out: torch.Tensor, nh: int, nkv: int, hd: int,
               append: bool = True) -> torch.Tensor:
    """Per-head RMSNorm of q and k, rotation, and the write of k and v into
    the paged cache; q comes out in the model's dtype."""
    N = qkv.shape[0]
    if hd % 2 or hd > MAX_HEAD_DIM:
        raise KernelError(f"qk_prepare: head size {hd} must be even and at most {MAX_HEAD_DIM}")
    page_size = pool.shape[3]
    _check_kv(pool, nkv, hd, page_size, "qk_prepare")
    if pool.dtype != q_out.dtype:
        raise KernelError(f"qk_prepare: cache is {pool.dtype} but q is {q_out.dtype}")
    _need(page_table, "page table", torch.int32)
    _guard("core", "attention", qkv.device, n_pages=pool.shape[0])
    _check(_fn("core", "mv_qk_prepare")(
        _need(qkv, "qkv", torch.float32, (N, (nh + 2 * nkv) * hd)),
        _need(wq, "q norm weight", torch.float32, (hd,), True),
        _need(wk, "k norm weight", torch.float32, (hd,), True), float(eps),
        _need(inv_freq, "inv_freq", torch.float32, (hd // 2,), True), int(half_split),
        _need(positions, "positions", torch.int32), _need(seq_of, "seq_of", torch.int32),
        page_table.data_ptr(), page_table.shape[1], page_size, _need(pool, "cache pool"),
        pool.stride(0), int(append), _need(q_out, "q out", None, (N, nh * hd)), _dt(q_out), N, nh, nkv, hd,
        _stream()), "mv_qk_prepare")
    account(_nbytes(qkv, q_out) + N * 2 * nkv * hd * pool.element_size())
    return q_out


def qk_prepare_q_only(qkv: torch.Tensor, wq: Optional[torch.Tensor], eps: float,
                      inv_freq: Optional[torch.Tensor], half_split: bool, positions, q_out: torch.Tensor,
                      nh: int, hd: int) -> torch.Tensor:
    """The same for a layer that has queries only (it reads another layer's cache)."""
    N = qkv.shape[0]
    if hd % 2 or hd > MAX_HEAD_DIM:
        raise KernelError(f"qk_prepare: head size {hd} must be even and at most {MAX_HEAD_DIM}")
    _check(_fn("core", "mv_qk_prepare")(
        _need(qkv, "q", torch.float32, (N, nh * hd)), _need(wq, "q norm weight", torch.float32, (hd,), True),
        None, float(eps), _need(inv_freq, "inv_freq", torch.float32, (hd // 2,), True), int(half_split),
        _need(positions, "positions", torch.int32), None, None, 0, 1, None, 0, 0,
        _need(q_out, "q out", None, (N, nh * hd)), _dt(q_out), N, nh, 0, hd, _stream()), "mv_qk_prepare")
    return q_out


def attention_generic(q: torch.Tensor, pool: torch.Tensor, page_table, positions, seq_of,
                      out: torch.Tensor, nh: int, nkv: int, hd: int, scale: float, window: int = 0):
    """Causal attention of every token of the step over its sequence's cache
    (which already holds the step's own keys), optional sliding window."""
    N = q.shape[0]
    if hd % 8 or hd > MAX_HEAD_DIM:
        raise KernelError(f"attention: head size {hd} must be a multiple of 8 and at most {MAX_HEAD_DIM}")
    if nh % nkv:
        raise KernelError(f"attention: {nh} heads are not a multiple of {nkv} kv heads")
    page_size = pool.shape[3]
    _check_kv(pool, nkv, hd, page_size, "attention")
    if q.dtype != pool.dtype or out.dtype != q.dtype:
        raise KernelError(f"attention: q {q.dtype}, cache {pool.dtype}, out {out.dtype} must agree")
    _guard("core", "attention", q.device, n_pages=pool.shape[0])
    _check(_fn("core", "mv_attention_generic")(
        _need(q, "q", None, (N, nh * hd)), _need(pool, "cache pool"), pool.stride(0),
        _need(page_table, "page table", torch.int32), page_table.shape[1], page_size,
        _need(positions, "positions", torch.int32), _need(seq_of, "seq_of", torch.int32),
        _need(out, "attention out", None, (N, nh * hd)), _dt(q), N, nh, nkv, hd, float(scale), int(window),
        _stream()), "mv_attention_generic")
    return out


_n_sms = {}


def n_sms(device=None) -> int:
    """Multiprocessors of the device (asked once); 148 where no device can be asked (planning on a CPU)."""
    if device is None and _n_sms:
        if len(_n_sms) == 1:                      # the usual case, asked many times a step
            return next(iter(_n_sms.values()))
    if not torch.cuda.is_available():
        return 148
    key = torch.cuda.current_device() if device is None else (torch.device(device).index or 0)
    if key not in _n_sms:
        _n_sms[key] = torch.cuda.get_device_properties(key).multi_processor_count
    return _n_sms[key]


DECODE_ATTENTION_MAX_TOKENS = 128      # steps with more query tokens split the work over the queries,
DECODE_ATTENTION_MAX_QUERIES = 2       # unless no sequence brings more than this many (a large decode batch)


def attention_decode_plan(N: int, nh: int, nkv: int, context_cap: int = 0):
    """(query heads per block, head tiles per kv head, key splits) for a step of N
    query tokens.  Enough blocks to fill the GPU twice over; more when the cache
    can be long (``context_cap`` tokens, the reach of the step's page table), so
    that a warp has about eight runs of 32 keys.  The count depends on the page
    table's width, not on the lengths: a decode step's launches are recorded once
    per width and replayed as the cache grows."""
    G = nh // nkv
    gt = 1 if G <= 1 else (2 if G <= 2 else (4 if G <= 4 else 8))
    head_tiles = -(-G // gt)
    splits = -(-2 * n_sms() // max(1, N * nkv * head_tiles))
    splits = max(splits, -(-context_cap // (32 * 4 * 8)))
    return gt, head_tiles, max(1, min(32, splits))


def attention_decode(q: torch.Tensor, pool: torch.Tensor, page_table, positions, seq_of, out: torch.Tensor,
                     nh: int, nkv: int, hd: int, scale: float, window: int, ws, splits: Optional[int] = None):
    """The same contract as ``attention_generic``, for steps with few query
    tokens: work is split over the keys, and the heads of a group share the
    loads.  ``ws`` (a Workspace) supplies the scratch for the key splits."""
    N = q.shape[0]
    if hd % 8 or hd > MAX_HEAD_DIM:
        raise KernelError(f"attention: head size {hd} must be a multiple of 8 and at most {MAX_HEAD_DIM}")
    if nh % nkv:
        raise KernelError(f"attention: {nh} heads are not a multiple of {nkv} kv heads")
    page_size = pool.shape[3]
    _check_kv(pool, nkv, hd, page_size, "attention")
    if q.dtype != pool.dtype or out.dtype != q.dtype:
        raise KernelError(f"attention: q {q.dtype}, cache {pool.dtype}, out {out.dtype} must agree")
    gt, head_tiles, auto = attention_decode_plan(N, nh, nkv, page_table.shape[1] * page_size)
    splits = auto if splits is None else int(splits)
    part_o = ws.get("attn_part_o", (N * nh * splits * hd,), torch.float32)
    part_ml = ws.get("attn_part_ml", (N * nh * splits * 2,), torch.float32)
    tickets = ws.get_zeroed("attn_tickets", (N * nkv * head_tiles,), torch.int32)
    _guard("core", "attention_decode", q.device, n_pages=pool.shape[0])
    _check(_fn("core", "mv_attention_decode")(
        _need(q, "q", None, (N, nh * hd)), _need(pool, "cache pool"), pool.stride(0),
        _need(page_table, "page table", torch.int32), page_table.shape[1], page_size,
        _need(positions, "positions", torch.int32), _need(seq_of, "seq_of", torch.int32),
        _need(out, "attention out", None, (N, nh * hd)), _dt(q), part_o.data_ptr(), part_ml.data_ptr(),
        tickets.data_ptr(), N, nh, nkv, hd, float(scale), int(window), splits, gt, head_tiles, _stream()),
        "mv_attention_decode")
    return out


def attention_decode_tc_plan(N: int, nkv: int, context_cap: int) -> int:
    """Key splits for the tcgen05 decode attention: as many as it takes to give each of the
    GPU's multiprocessors its two blocks (more blocks than that only add set-up and merging:
    at 64 tokens of 520 cached ones, 29 us unsplit against 39 us in two), at least two key
    blocks of 128 a split.  Like ``attention_decode_plan`` it depends on the page table's
    reach, not on the lengths."""
    blocks = max(1, -(-context_cap // 128))
    want = (2 * n_sms()) // max(1, N * nkv)
    if blocks <= 8:
        return 1          # up to 1,024 cached tokens a split saves less than its merge kernel costs
    return max(1, min(64, want, blocks // 2))


DECODE_TC_MAX_GROUP = 16


def attention_decode_tc_supported(dtype: torch.dtype, hd: int, pool: torch.Tensor, window: int, nh: int,
                                  nkv: int) -> bool:
    """What the tcgen05 decode attention takes: as the tcgen05 prefill attention, and at most 16
    query heads a kv head (they are the 16 columns of its transposed scores)."""
    return (attention_prefill_tc_supported(dtype, hd, pool, window) and nkv > 0 and nh % nkv == 0
            and nh // nkv <= DECODE_TC_MAX_GROUP)


def attention_decode_tc(q: torch.Tensor, pool: torch.Tensor, page_table, positions, seq_of, out: torch.Tensor,
                        nh: int, nkv: int, hd: int, scale: float, ws, splits: Optional[int] = None):
    """Attention of single query tokens over long caches, both products on tcgen05 (bfloat16,
    head size 64, pages of 64 tokens, no window).  Same arguments and result as
    :func:`attention_decode`."""
    N = q.shape[0]
    if not attention_decode_tc_supported(q.dtype, hd, pool, 0, nh, nkv):
        raise KernelError(f"attention_decode_tc: needs bfloat16, head size 64, a dense pool of 64-token pages and "
                          f"at most 16 heads a kv head, got {q.dtype}, {hd}, pool {tuple(pool.shape)}, {nh}/{nkv}")
    _check_kv(pool, nkv, hd, 64, "attention")
    if q.dtype != pool.dtype or out.dtype != q.dtype:
        raise KernelError(f"attention: q {q.dtype}, cache {pool.dtype}, out {out.dtype} must agree")
    splits = attention_decode_tc_plan(N, nkv, page_table.shape[1] * 64) if splits is None else int(splits)
    part_o = ws.get("attn_part_o", (N * nh * splits * hd,), torch.float32)
    part_ml = ws.get("attn_part_ml", (N * nh * splits * 2,), torch.float32)
    _check(_fn("bf16", "mv_attention_decode_tc")(
        _need(q, "q", None, (N, nh * hd)), _need(pool, "cache pool"), pool.shape[0] * 2 * nkv * 64,
        _need(page_table, "page table", torch.int32), page_table.shape[1],
        _need(positions, "positions", torch.int32), _need(seq_of, "seq_of", torch.int32),
        _need(out, "attention out", None, (N, nh * hd)), part_o.data_ptr(), part_ml.data_ptr(), N, nh, nkv,
        float(scale), splits, _error_flag(q.device).data_ptr(), _stream()), "mv_attention_decode_tc")
    if splits > 1:
        add_launches(1)                    # the kernel that merges the splits
    return out


PREFILL_ATTENTION_MAX_HEAD_DIM = 128


def attention_prefill_supported(dtype: torch.dtype, hd: int) -> bool:
    return dtype == torch.bfloat16 and hd % 16 == 0 and hd <= PREFILL_ATTENTION_MAX_HEAD_DIM


def attention_prefill(q: torch.Tensor, pool: torch.Tensor, page_table, cu, starts, out: torch.Tensor,
                      n_seqs: int, nh: int, nkv: int, hd: int, scale: float, window: int = 0):
    """Causal attention of a step with many query tokens on the tensor cores
    (bfloat16, head sizes 16..128 in steps of 16).  The step's tokens are packed
    sequence by sequence (``cu``), sequence b starting at position ``starts[b]``."""
    N = q.shape[0]
    if not attention_prefill_supported(q.dtype, hd):
        raise KernelError(f"attention_prefill: needs bfloat16 and a head size 16..128 in steps of 16, "
                          f"got {q.dtype}, {hd}")
    if nh % nkv:
        raise KernelError(f"attention: {nh} heads are not a multiple of {nkv} kv heads")
    page_size = pool.shape[3]
    _check_kv(pool, nkv, hd, page_size, "attention")
    if q.dtype != pool.dtype or out.dtype != q.dtype:
        raise KernelError(f"attention: q {q.dtype}, cache {pool.dtype}, out {out.dtype} must agree")
    _guard("bf16", "attention_prefill", q.device, n_pages=pool.shape[0])
    _check(_fn("bf16", "mv_attention_prefill")(
        _need(q, "q", None, (N, nh * hd)), _need(pool, "cache pool"), pool.stride(0),
        _need(page_table, "page table", torch.int32), page_table.shape[1], page_size,
        _need(cu, "cu", torch.int32), _need(starts, "starts", torch.int32),
        _need(out, "attention out", None, (N, nh * hd)), N, n_seqs, nh, nkv, hd, float(scale), int(window),
        _stream()), "mv_attention_prefill")
    return out


def attention_prefill_tc_supported(dtype: torch.dtype, hd: int, pool: torch.Tensor, window: int) -> bool:
    """What the tcgen05 prefill attention takes: bfloat16, head size 64, no window, and a
    dense cache pool [pages, 2, kv heads, 64, 64] that a 2-D tensor map can describe."""
    if DEBUG_CHECKS:
        return False            # a build with index checks runs the kernels that have them
    if dtype != torch.bfloat16 or hd != 64 or window != 0 or pool.dim() != 5 or pool.shape[3] != 64:
        return False
    rows = pool.shape[0] * 2 * pool.shape[2] * 64
    return pool.is_contiguous() and rows < 2 ** 31 and pool.data_ptr() % 16 == 0


def attention_prefill_tc(q: torch.Tensor, pool: torch.Tensor, page_table, cu, starts, out: torch.Tensor,
                         n_seqs: int, nh: int, nkv: int, hd: int, scale: float):
    """Causal attention of a step with many query tokens, both products on tcgen05
    (bfloat16, head size 64, pages of 64 tokens, no window).  Same arguments and
    result as :func:`attention_prefill`."""
    N = q.shape[0]
    if not attention_prefill_tc_supported(q.dtype, hd, pool, 0):
        raise KernelError(f"attention_prefill_tc: needs bfloat16, head size 64 and a dense pool of 64-token pages, "
                          f"got {q.dtype}, {hd}, pool {tuple(pool.shape)}")
    if nh % nkv:
        raise KernelError(f"attention: {nh} heads are not a multiple of {nkv} kv heads")
    _check_kv(pool, nkv, hd, 64, "attention")
    if q.dtype != pool.dtype or out.dtype != q.dtype:
        raise KernelError(f"attention: q {q.dtype}, cache {pool.dtype}, out {out.dtype} must agree")
    _check(_fn("bf16", "mv_attention_prefill_tc")(
        _need(q, "q", None, (N, nh * hd)), _need(pool, "cache pool"), pool.shape[0] * 2 * nkv * 64,
        _need(page_table, "page table", torch.int32), page_table.shape[1],
        _need(cu, "cu", torch.int32), _need(starts, "starts", torch.int32),
        _need(out, "attention out", None, (N, nh * hd)), N, n_seqs, nh, nkv, float(scale),
        _error_flag(q.device).data_ptr(), _stream()), "mv_attention_prefill_tc")
    return out


def sample_scratch_width(V: int) -> int:
    """Floats of scratch a row of V logits needs: V rounded up to the sampling block's 1,024 threads."""
    return -(-int(V) // 1024) * 1024


def sample(logits: torch.Tensor, work: torch.Tensor, out: torch.Tensor, *, temperature: float,
           top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0, repetition_penalty: float = 1.0,
           presence_penalty: float = 0.0, frequency_penalty: float = 0.0,
           recent: Optional[torch.Tensor] = None, n_recent: Optional[torch.Tensor] = None, seed: int = 0,
           streams: Optional[torch.Tensor] = None, steps: Optional[torch.Tensor] = None,
           ring: Optional[torch.Tensor] = None, ring_rows: Optional[torch.Tensor] = None,
           flag_to: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of ``logits`` [B, V] (float32, rows may be strided).  ``work``: scratch of
    ``sample_scratch_width(V)`` floats a row.  The recent tokens that the penalties look at come
    either from the caller (``recent`` [B, 64], ``n_recent``) or from ``ring`` [states, 128], which the
    kernel keeps itself: row b uses state ``ring_rows[b]``, looks at the places of its last
    min(steps[b], 64) steps and writes the token it samples to place steps[b] mod 128.
    ``flag_to`` (int32 [1] on the device): the kernel also copies the device's error flag there, so
    that it reaches the host with the tokens."""
    B, V = logits.shape
    if not logits.is_cuda or logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 on a CUDA device with unit column stride")
    if work.dim() != 2 or work.shape[0] < B:
        raise KernelError(f"sample: scratch {tuple(work.shape)} has fewer rows than the {B} rows of logits")
    if ring is not None and (steps is None or recent is not None):
        raise KernelError("sample: a ring of recent tokens needs the rows' steps, and excludes a caller's recent tokens")
    if recent is not None and (recent.shape != (B, RECENT_MAX)):
        raise KernelError(f"sample: recent tokens shape {tuple(recent.shape)}, expected [{B}, {RECENT_MAX}]")
    _check(_fn("core", "mv_sample")(
        logits.data_ptr(), logits.stride(0),
        _need(work, "sample scratch", torch.float32, (None, sample_scratch_width(V))), B, V,
        float(temperature), int(top_k), float(top_p), float(min_p), float(repetition_penalty),
        float(presence_penalty), float(frequency_penalty),
        _need(recent, "recent", torch.int32, optional=True),
        _need(n_recent, "n_recent", torch.int32, (B,), True), int(seed) & ((1 << 64) - 1),
        _need(streams, "streams", torch.int32, (B,), True), _need(steps, "steps", torch.int32, (B,), True),
        _need(ring, "recent ring", torch.int32, (None, RECENT_RING), True),
        _need(ring_rows, "ring rows", torch.int32, (B,), ring is None),
        _need(out, "sample out", torch.int32, (B,)),
        _error_flag(logits.device).data_ptr() if flag_to is not None else None,
        _need(flag_to, "flag copy", torch.int32, (1,), True), _stream()), "mv_sample")
    account(B * V * 4)
    return out
