"""The allocation-free decode-attention entry point, called through its
exported C symbol (as a C program that links the library would), against the
ordinary entry point that takes scratch from the caller.

Who this entry point is for: callers that cannot obtain device memory at the
moment of the call - code running where the CUDA allocator must not be entered,
or a program that links the library without PyTorch.  Its scratch is a device
array inside the library (about 4 MiB on every GPU that loads it), so calls
share it: the test makes two calls in a row on one stream and checks both, and
it checks that a call too large for the array is refused with a message
instead of being served some other way.

This file sorts last on purpose: a run that stops at the first failure has then
already run every other test.  It passes alone in a fresh process and after the
other tests.
"""
import ctypes
import math

import pytest
import torch

from test_kernels_gpu import build_cache, ints, plain_attend

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def static_entry():
    from mivi_v4_b200.ops.build import compile_library
    lib = ctypes.CDLL(compile_library("core"))
    fn = lib.mv_attention_decode_static
    P, I, F, Q = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
    fn.argtypes = [P, P, Q, P, I, I, P, P, P, I, I, I, I, I, F, I, I, P, ctypes.c_char_p, I]
    fn.restype = I
    return fn


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_static_scratch_entry_matches_the_allocating_one(dtype):
    from mivi_v4_b200.engine.step import Workspace
    from mivi_v4_b200.ops import kernels as K
    fn = static_entry()
    nh, nkv, hd, page = 8, 2, 64, 64
    scale = 1.0 / math.sqrt(hd)
    tol = 2e-5 if dtype == torch.float32 else 1.5e-2
    stream = torch.cuda.current_stream().cuda_stream
    err = ctypes.create_string_buffer(256)
    for call, (lengths, splits) in enumerate([([300, 64, 129, 1], 5), ([33, 700], 9)]):
        pool, table, dense = build_cache(lengths, nkv, hd, page, dtype, seed=call)
        queries = [(b, n - 1) for b, n in enumerate(lengths)]
        g = torch.Generator().manual_seed(call)
        q = torch.randn(len(queries), nh, hd, generator=g).to(dtype)
        qd = q.reshape(len(queries), nh * hd).contiguous().to(DEV)
        seq_of, positions = ints([b for b, _ in queries]), ints([p for _, p in queries])
        want = torch.empty_like(qd)
        K.attention_decode(qd, pool, table, positions, seq_of, want, nh, nkv, hd, scale, 0, Workspace(DEV),
                           splits=splits)
        got = torch.full_like(qd, float("nan"))
        rc = fn(qd.data_ptr(), pool.data_ptr(), pool.stride(0), table.data_ptr(), table.shape[1], page,
                positions.data_ptr(), seq_of.data_ptr(), got.data_ptr(), 0 if dtype == torch.float32 else 1,
                len(queries), nh, nkv, hd, scale, 0, splits, stream, err, len(err))
        assert rc == 0, err.value.decode()
        torch.cuda.synchronize()
        assert torch.allclose(got.double(), want.double(), rtol=tol, atol=tol), (call, (got - want).abs().max())
        for i, (b, p) in enumerate(queries):        # and both are right
            ref = plain_attend(q[i], dense[b][0], dense[b][1], p, nh, nkv, scale, 0)
            assert torch.allclose(got[i].reshape(nh, hd).double().cpu(), ref, rtol=tol, atol=tol)


def test_static_scratch_entry_refuses_what_does_not_fit():
    fn = static_entry()
    err = ctypes.create_string_buffer(256)
    dummy = torch.zeros(16, device=DEV)
    d = dummy.data_ptr()
    # 4096 tokens x 32 heads x 8 splits x 66 floats is far beyond the built-in array
    rc = fn(d, d, 0, d, 1, 64, d, d, d, 1, 4096, 32, 8, 64, 0.125, 0, 8, None, err, len(err))
    assert rc == 2 and b"built-in scratch" in err.value
    rc = fn(d, d, 0, d, 1, 64, d, d, d, 1, 4, 5, 2, 64, 0.125, 0, 1, None, err, len(err))
    assert rc == 1 and b"multiple" in err.value
    # bad arguments are named as such (1), before anything is enqueued: a head size, a page size, a pointer
    rc = fn(d, d, 0, d, 1, 64, d, d, d, 1, 4, 8, 2, 60, 0.125, 0, 2, None, err, len(err))
    assert rc == 1 and b"head size 60" in err.value
    rc = fn(d, d, 0, d, 1, 48, d, d, d, 1, 4, 8, 2, 64, 0.125, 0, 2, None, err, len(err))
    assert rc == 1 and b"page size 48" in err.value
    rc = fn(d, d, 0, d, 1, 64, d, d, None, 1, 4, 8, 2, 64, 0.125, 0, 2, None, err, len(err))
    assert rc == 1 and b"null" in err.value


def test_static_scratch_entry_leaves_device_memory_alone():
    """It allocates nothing: the device's free memory is the same before and after calls, and an
    unsplit call of many tokens needs none of the built-in scratch."""
    from mivi_v4_b200.ops import kernels as K
    from mivi_v4_b200.engine.step import Workspace
    fn = static_entry()
    nh, nkv, hd, page = 4, 2, 32, 16
    scale = 1.0 / math.sqrt(hd)
    lengths = [37] * 20
    pool, table, dense = build_cache(lengths, nkv, hd, page, torch.float32, seed=5)
    N = 20000                                   # beyond the counters of the built-in array: fine when unsplit
    g = torch.Generator().manual_seed(5)
    qd = torch.randn(N, nh * hd, generator=g).to(DEV)
    seq_of = ints([i % 20 for i in range(N)])
    positions = ints([36] * N)
    want = torch.empty_like(qd)
    K.attention_decode(qd, pool, table, positions, seq_of, want, nh, nkv, hd, scale, 0, Workspace(DEV), splits=1)
    got = torch.full_like(qd, float("nan"))
    err = ctypes.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    free0 = None
    for call in range(3):
        if call == 1:                           # the first call may load the library's device code
            torch.cuda.synchronize()
            free0, _ = torch.cuda.mem_get_info()
        rc = fn(qd.data_ptr(), pool.data_ptr(), pool.stride(0), table.data_ptr(), table.shape[1], page,
                positions.data_ptr(), seq_of.data_ptr(), got.data_ptr(), 0, N, nh, nkv, hd, scale, 0, 1, stream,
                err, len(err))
        assert rc == 0, err.value.decode()
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0
    assert torch.allclose(got, want, rtol=2e-5, atol=2e-5)
