"""The matrix product of a layer, y = x W^T: picks the kernel for the operands'
dtype and shape.  All kernels are this library's own; none is a vendor library
call.

float32 operands always take the CUDA-core kernel (true 32-bit products and
sums).  bfloat16 operands take the tensor-core kernels where their shape
rules hold and the CUDA-core kernel otherwise.  A weight that the checkpoint
stores in 32-bit stays so; a bfloat16 activation is widened for it.
"""
from __future__ import annotations

import contextlib
from typing import Optional

import torch

from . import kernels as K


import os

_DECODE_GEMM = os.environ.get("MIVI_DECODE_GEMM", "auto")
MMA_MAX_ROWS = 8


class WeightOrder:
    """The weights that the products of a step read, in order.  A step that will be replayed
    many times (a decode step) is first run once with ``recording()``; recorded again under
    ``looking_ahead()``, each product of few rows is told what the next product will read and
    asks the L2 cache for it while it finishes.  A step whose products come in another order
    than the recorded one simply gets no hints from the first difference on."""

    def __init__(self):
        self.seen = []           # (address, bytes) of each product's weight
        self.at = None           # position while looking ahead; None while recording
        self.lasting = None      # address -> bytes of memory that outlives the recording, or None: any

    def next_after(self, w: torch.Tensor):
        here = (w.data_ptr(), w.numel() * w.element_size())
        if self.at is None:
            self.seen.append(here)
            return None
        i = self.at
        if i < 0 or i >= len(self.seen) or self.seen[i] != here:
            self.at = -1         # not the recorded order: no more hints
            return None
        self.at = i + 1
        ptr, size = self.seen[(i + 1) % len(self.seen)]       # after the last one comes the next step's first
        if self.lasting is not None and self.lasting.get(ptr, 0) < size:
            return None          # not a tensor of the model: it may be gone when the recording is replayed
        size = min(size, _AHEAD_BYTES)
        return (ptr, size) if size >= 128 else None


_order: Optional[WeightOrder] = None
# The most that one product requests ahead (MIVI_AHEAD_MB, 0 turns it off).  Measured on decode steps
# of the 1.2B-parameter shape at 8 sequences: 735 us without, 729 with 2 MB, 712 with 8, 714 with 16,
# 746 with 32, 760 with 64 (the requests then stand in the way of the kernel's own last loads and stores).
_AHEAD_BYTES = int(float(os.environ.get("MIVI_AHEAD_MB", "8")) * (1 << 20))


@contextlib.contextmanager
def recording():
    """Products issued inside note their weights; yields the ``WeightOrder``."""
    global _order
    prev, _order = _order, WeightOrder()
    try:
        yield _order
    finally:
        _order = prev


@contextlib.contextmanager
def looking_ahead(order: WeightOrder, lasting: Optional[dict] = None):
    """Products issued inside, if they come in ``order``'s order, prefetch their successor's weights.
    ``lasting``: address -> bytes of the tensors that will still be there whenever the launches recorded
    inside are replayed (a model's parameters); other weights are not requested ahead."""
    global _order
    prev, _order = _order, order
    order.at = 0 if _AHEAD_BYTES > 0 and order.seen else -1
    order.lasting = lasting
    try:
        yield
    finally:
        _order = prev


def _ahead(w: torch.Tensor, fn) -> dict:
    """The ``ahead`` argument for a product with ``w``, if its kernel takes one."""
    if _order is None:
        return {}
    nxt = _order.next_after(w)
    return {"ahead": nxt} if nxt is not None and (fn is K.gemm_small_m or fn is K.gemm_tc_swap) else {}


def _small_m(m: int):
    """The kernel for at most 64 rows.  Two exist: the mma.sync kernel that streams W
    through registers, and the tcgen05 kernel with swapped operands (TMA ring,
    accumulator in tensor memory).  Measured on whole decode steps of the
    1.2B-parameter shape, the first wins up to 8 rows (a short product does not repay
    the pipeline's set-up), the second from 16 rows on (1.3 ms against 1.4 at 16 rows,
    1.7 ms against 2.7 at 64), where the first is bound by re-reading X.
    MIVI_DECODE_GEMM=mma|tc forces one."""
    if _DECODE_GEMM == "tc" or (_DECODE_GEMM != "mma" and m > MMA_MAX_ROWS):
        return K.gemm_tc_swap
    return K.gemm_small_m


def tensor_core_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the bfloat16 tensor-core kernels take these operands."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


_PREFILL_CARRY = os.environ.get("MIVI_CARRY_NORMS_PREFILL", "0") == "1"
_MID_GEMM = os.environ.get("MIVI_MID_GEMM", "auto")              # swap | tc | auto


def swap_takes(n_rows: int, w: torch.Tensor) -> bool:
    """Whether a product of more than 64 rows with ``w`` goes to the kernel with swapped operands
    (``gemm_tc_swap``: a block has 128 rows of w and 128 tokens, K cut over a cluster) rather than to
    the prefill kernels: while its blocks are few enough that cutting K is what fills the device.
    Measured on the five products of the 1.2B-parameter shape at 65 to 1,024 rows; the down projection
    (K = 8,192: 16 us against 50 at 128 rows, 23 against 47 at 512) gains most.  MIVI_MID_GEMM=swap|tc
    forces one."""
    if _MID_GEMM != "auto":
        return _MID_GEMM == "swap"
    blocks = -(-w.shape[0] // 128) * -(-n_rows // 128)
    return blocks <= 100 or (blocks <= 148 and (n_rows <= 96 or w.shape[1] >= 4096))


def norm_link_ok(n_rows: int, w: torch.Tensor, x_dtype: torch.dtype = torch.bfloat16, emits: bool = False) -> bool:
    """Whether a product of ``n_rows`` rows with ``w`` takes a kernel that can carry a
    norm (``scale`` of :func:`linear`, or ``emit`` with ``emits``): the weight-streaming kernels do
    both; the prefill kernels apply a scale for nothing, but as the one that emits, the kernel of two
    multiprocessors a tile measured slower than the norm kernel it saves (4.70 against 4.59 ms for a
    prompt of 2,048 tokens: with one tile a pair the epilogue's reading of the old rows is exposed),
    so it emits only with MIVI_CARRY_NORMS_PREFILL=1."""
    if not (x_dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] % 8 == 0 and w.data_ptr() % 16 == 0):
        return False
    if 1 <= n_rows <= K.SMALL_M_MAX or swap_takes(n_rows, w) or not emits:
        return True
    return _PREFILL_CARRY and w.shape[0] % 32 == 0 and K.gemm_tc_pair_takes(n_rows, w.shape[0])


_FUSED_CONV = os.environ.get("MIVI_FUSED_CONV", "1") != "0"
# From 9 rows on the fused kernel is the tcgen05 one over a copy of the projection whose rows are regrouped by 32
# channels (``kernels.gemm_tc_swap_shortconv``, ``kernels.group_conv_rows``; the mixer keeps the copy).  It takes
# ten launches out of a decode step of the 1.2B-parameter shape and leaves its time where it was (64 sequences:
# 1,053 us with it, 1,047 without; 32: 0.99 against 0.96 ms): the convolution kernels it replaces run under the
# products' tails anyway.  So it is off, and MIVI_FUSED_CONV_TC=1 turns it on.  (An earlier form, three
# accumulators a block of 128 channels, was 15 % slower than the two kernels: its blocks were alone on a
# multiprocessor.)
_FUSED_CONV_TC = os.environ.get("MIVI_FUSED_CONV_TC", "0") == "1"


def conv_rows_grouped(n_rows: int, w_in: torch.Tensor) -> bool:
    """Whether the fused convolution of a step of ``n_rows`` rows reads the projection's rows regrouped
    (``kernels.group_conv_rows``): the tcgen05 kernel's range."""
    return _small_m(n_rows) is K.gemm_tc_swap


def shortconv_decode_fused_ok(n_rows: int, x: torch.Tensor, w_in: torch.Tensor) -> bool:
    """Whether a decode step's gated short convolution can run as the epilogue of its input
    projection (``kernels.gemm_small_m_shortconv``): the steps whose products take the
    register-streaming kernel, bfloat16 operands.  One launch less a layer; MIVI_FUSED_CONV=0
    keeps the two kernels."""
    if not (_FUSED_CONV and not K.DEBUG_CHECKS and 1 <= n_rows <= K.SMALL_M_MAX and tensor_core_ok(x, w_in)):
        return False
    if _small_m(n_rows) is K.gemm_small_m:
        return n_rows <= K.SHORTCONV_FUSED_MAX_ROWS
    return _FUSED_CONV_TC and (w_in.shape[0] // 3) % K.CONV_ROW_GROUP == 0


def linear_shortconv_decode(x: torch.Tensor, w_in: torch.Tensor, b_in, taps, b_conv, state, slots, out, *,
                            scale: Optional[K.NormLink] = None, grouped: bool = False) -> torch.Tensor:
    """The input projection and the convolution of a decode step in one kernel (the register-streaming
    one up to 8 rows, the tcgen05 one from there to 64); needs ``shortconv_decode_fused_ok``.  ``grouped``:
    ``w_in`` is the regrouped copy that ``conv_rows_grouped`` asks for."""
    ahead = {}
    if _order is not None:
        nxt = _order.next_after(w_in)
        ahead = {"ahead": nxt} if nxt is not None else {}
    if _small_m(x.shape[0]) is K.gemm_tc_swap:
        if not grouped:
            raise K.KernelError("linear_shortconv_decode: the tcgen05 kernel reads the regrouped projection")
        return K.gemm_tc_swap_shortconv(x, w_in, b_in, taps, b_conv, state, slots, out, scale=scale, **ahead)
    return K.gemm_small_m_shortconv(x, w_in, b_in, taps, b_conv, state, slots, out, scale=scale, **ahead)


_FUSED_QK = os.environ.get("MIVI_FUSED_QK", "1") != "0"


def heads_fused_ok(n_rows: int, x: torch.Tensor, w_qkv: torch.Tensor, head_dim: int, pool: torch.Tensor,
                   half_split: bool = False) -> bool:
    """Whether the preparation of q, k and v (per-head norm, rotation, append to the cache) can run
    as the epilogue of their projection (``kernels.gemm_small_m_heads`` up to 8 rows,
    ``kernels.gemm_tc_swap_heads`` from there to 64, which pairs the elements (2i, 2i+1) only): heads of 64,
    bfloat16 cache.  MIVI_FUSED_QK=0 keeps the two kernels."""
    if not (_FUSED_QK and not K.DEBUG_CHECKS and 1 <= n_rows <= K.SMALL_M_MAX and head_dim == K.HEADS_FUSED_HEAD_DIM
            and pool.dtype == torch.bfloat16 and tensor_core_ok(x, w_qkv)):
        return False
    if _small_m(n_rows) is K.gemm_tc_swap:
        return not half_split
    return n_rows <= K.SHORTCONV_FUSED_MAX_ROWS


def linear_heads(x: torch.Tensor, w_qkv: torch.Tensor, wq, wk, eps: float, inv_freq, half_split: bool, positions,
                 seq_of, page_table, pool, q_out, nh: int, nkv: int, *, scale: Optional[K.NormLink] = None):
    """The q/k/v projection and the preparation of its heads in one kernel; needs ``heads_fused_ok``."""
    ahead = {}
    if _order is not None:
        nxt = _order.next_after(w_qkv)
        ahead = {"ahead": nxt} if nxt is not None else {}
    if _small_m(x.shape[0]) is K.gemm_tc_swap:
        return K.gemm_tc_swap_heads(x, w_qkv, wq, wk, eps, inv_freq, positions, seq_of, page_table, pool, q_out, nh,
                                    nkv, scale=scale, **ahead)
    return K.gemm_small_m_heads(x, w_qkv, wq, wk, eps, inv_freq, half_split, positions, seq_of, page_table, pool,
                                q_out, nh, nkv, scale=scale, **ahead)


def end_norms_carried(n_rows: int) -> bool:
    """Whether the norms at the two ends of the model (after the embedding, before the head) ride on
    their neighbours too, like the ones between products.  Measured on the 1.2B-parameter shape:
    702 -> 700 us a step at 8 sequences (two launches fewer), but 1084 -> 1105 us at 64, where the
    norm kernels run under the tails of their predecessors anyway; so only in steps of few rows."""
    return 1 <= n_rows <= MMA_MAX_ROWS and _DECODE_GEMM != "tc"


def linear_swiglu(x: torch.Tensor, w_grouped: torch.Tensor, out: torch.Tensor, *,
                  scale: Optional[K.NormLink] = None) -> torch.Tensor:
    """out = silu(gate) * up where [gate | up] = x @ w_grouped.T and the rows of
    ``w_grouped`` alternate in groups of 16 (gate rows, then the up rows of the
    same features): the activation runs in the product's epilogue, so gate and
    up never go to memory.  Needs ``tensor_core_ok``."""
    if x.shape[0] <= K.SMALL_M_MAX:
        fn = _small_m(x.shape[0])
        return fn(x, w_grouped, out, swiglu=True, scale=scale, **_ahead(w_grouped, fn))
    if swap_takes(x.shape[0], w_grouped):
        return K.gemm_tc_swap(x, w_grouped, out, swiglu=True, scale=scale, **_ahead(w_grouped, K.gemm_tc_swap))
    if _order is not None:
        _order.next_after(w_grouped)
    return K.gemm_tc(x, w_grouped, out, swiglu=True, scale=scale)


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, bias: Optional[torch.Tensor] = None,
           accumulate: bool = False, scale: Optional[K.NormLink] = None,
           emit: Optional[K.NormLink] = None) -> torch.Tensor:
    """out = x @ w.T (+ bias); with ``accumulate`` the product is added to
    ``out`` (float32), which is how a layer's result joins the residual
    stream without a separate pass.  ``scale`` / ``emit`` (see ``NormLink``) need
    ``norm_link_ok`` for these operands."""
    if scale is not None or emit is not None:
        if not norm_link_ok(x.shape[0], w, x.dtype, emits=emit is not None) or x.data_ptr() % 16:
            raise K.KernelError("linear: these operands cannot carry a norm; ask norm_link_ok first")
        if x.shape[0] > K.SMALL_M_MAX and swap_takes(x.shape[0], w):
            return K.gemm_tc_swap(x, w, out, bias=bias, accumulate=accumulate, scale=scale, emit=emit,
                                  **_ahead(w, K.gemm_tc_swap))
        if x.shape[0] > K.SMALL_M_MAX:
            if _order is not None:
                _order.next_after(w)
            return K.gemm_tc(x, w, out, bias=bias, accumulate=accumulate, scale=scale, emit=emit,
                             pair=True if emit is not None else None)
        fn = _small_m(x.shape[0])
        return fn(x, w, out, bias=bias, accumulate=accumulate, scale=scale, emit=emit, **_ahead(w, fn))
    if w.dtype == torch.float32 and x.dtype != torch.float32:
        x = x.float()
    if (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
        if x.shape[0] <= K.SMALL_M_MAX:
            fn = _small_m(x.shape[0])
            return fn(x, w, out, bias=bias, accumulate=accumulate, **_ahead(w, fn))
        if swap_takes(x.shape[0], w):
            return K.gemm_tc_swap(x, w, out, bias=bias, accumulate=accumulate, **_ahead(w, K.gemm_tc_swap))
        if _order is not None:
            _order.next_after(w)
        return K.gemm_tc(x, w, out, bias=bias, accumulate=accumulate)
    if _order is not None:
        _order.next_after(w)
    return K.gemm_simt(x, w, out, bias=bias, accumulate=accumulate)
