"""The matrix product of a layer, y = x W^T: picks the kernel for the operands'
dtype and shape.  All kernels are this library's own; none is a vendor library
call.

float32 operands always take the CUDA-core kernel (true 32-bit products and
sums).  bfloat16 operands take the tensor-core kernels where their shape
rules hold and the CUDA-core kernel otherwise.  A weight that the checkpoint
stores in 32-bit stays so; a bfloat16 activation is widened for it.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import kernels as K


import os

_DECODE_GEMM = os.environ.get("MIVI_DECODE_GEMM", "auto")
MMA_MAX_ROWS = 8


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


def norm_link_ok(n_rows: int, w: torch.Tensor, x_dtype: torch.dtype = torch.bfloat16) -> bool:
    """Whether a product of ``n_rows`` rows with ``w`` takes a kernel that can carry a
    norm (``scale`` / ``emit`` of :func:`linear`): one of the two of at most 64 rows.  (In the
    tcgen05 kernel of more rows the epilogue is on the critical path: carrying the norm there
    measured 8 % slower than the norm kernels it saved.)"""
    return (1 <= n_rows <= K.SMALL_M_MAX and x_dtype == torch.bfloat16
            and w.dtype == torch.bfloat16 and w.shape[1] % 8 == 0 and w.data_ptr() % 16 == 0)


def linear_swiglu(x: torch.Tensor, w_grouped: torch.Tensor, out: torch.Tensor, *,
                  scale: Optional[K.NormLink] = None) -> torch.Tensor:
    """out = silu(gate) * up where [gate | up] = x @ w_grouped.T and the rows of
    ``w_grouped`` alternate in groups of 16 (gate rows, then the up rows of the
    same features): the activation runs in the product's epilogue, so gate and
    up never go to memory.  Needs ``tensor_core_ok``."""
    if scale is not None:
        return _small_m(x.shape[0])(x, w_grouped, out, swiglu=True, scale=scale)
    if x.shape[0] <= K.SMALL_M_MAX:
        return _small_m(x.shape[0])(x, w_grouped, out, swiglu=True)
    return K.gemm_tc(x, w_grouped, out, swiglu=True)


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, bias: Optional[torch.Tensor] = None,
           accumulate: bool = False, scale: Optional[K.NormLink] = None,
           emit: Optional[K.NormLink] = None) -> torch.Tensor:
    """out = x @ w.T (+ bias); with ``accumulate`` the product is added to
    ``out`` (float32), which is how a layer's result joins the residual
    stream without a separate pass.  ``scale`` / ``emit`` (see ``NormLink``) need
    ``norm_link_ok`` for these operands."""
    if scale is not None or emit is not None:
        if not norm_link_ok(x.shape[0], w, x.dtype) or x.data_ptr() % 16:
            raise K.KernelError("linear: these operands cannot carry a norm; ask norm_link_ok first")
        return _small_m(x.shape[0])(x, w, out, bias=bias, accumulate=accumulate, scale=scale, emit=emit)
    if w.dtype == torch.float32 and x.dtype != torch.float32:
        x = x.float()
    if (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
        if x.shape[0] <= K.SMALL_M_MAX:
            return _small_m(x.shape[0])(x, w, out, bias=bias, accumulate=accumulate)
        return K.gemm_tc(x, w, out, bias=bias, accumulate=accumulate)
    return K.gemm_simt(x, w, out, bias=bias, accumulate=accumulate)
