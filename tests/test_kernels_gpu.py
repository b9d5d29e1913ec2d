"""Each kernel alone against a plain PyTorch float32/float64 expression of the
same operation, at sizes other than the engine's."""
import math

import pytest
import torch

import plain_lfm2 as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def K():
    from mivi_v4_b200.ops import kernels
    return kernels


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def ints(vals):
    return torch.tensor(vals, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("V,H,N", [(37, 24, 5), (301, 200, 3)])
def test_embed(dtype, V, H, N):
    table = rnd(V, H, dtype=dtype)
    tok = ints([V - 1, 0, 7][:N] + [3] * max(0, N - 3))
    out = torch.empty(tok.numel(), H, device=DEV)
    K().embed(table, tok, out)
    assert torch.equal(out, table[tok.long()].float())


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,H,eps", [(1, 16, 1e-5), (7, 200, 1e-6), (3, 2048, 1e-5), (2, 5000, 1e-3)])
def test_rmsnorm(out_dtype, n, H, eps):
    x, w = rnd(n, H, scale=3.0), rnd(H) + 1.0
    out = torch.empty(n, H, dtype=out_dtype, device=DEV)
    K().rmsnorm(x, w, eps, out)
    want = P.plain_rms_norm(x.double(), w.double(), eps)
    tol = 1e-5 if out_dtype == torch.float32 else 1e-2
    assert torch.allclose(out.double(), want, rtol=tol, atol=tol)
    rows = ints([n - 1, 0])
    out2 = torch.empty(2, H, dtype=out_dtype, device=DEV)
    K().rmsnorm(x, w, eps, out2, rows)
    assert torch.equal(out2, out[rows.long()])


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_swiglu(out_dtype):
    N, F = 5, 144
    gu = rnd(N, 2 * F, scale=4.0)
    gu[0, 0] = -90.0
    out = torch.empty(N, F, dtype=out_dtype, device=DEV)
    K().swiglu(gu, out)
    a, b = gu[:, :F].double(), gu[:, F:].double()
    want = a / (1 + torch.exp(-a)) * b
    tol = 1e-6 if out_dtype == torch.float32 else 1e-2
    assert torch.allclose(out.double(), want, rtol=tol, atol=tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,Kd", [(1, 1, 1), (3, 70, 33), (65, 64, 64), (130, 301, 200), (8, 2048, 96)])
def test_gemm_simt(dtype, M, N, Kd):
    x, w, bias = rnd(M, Kd, dtype=dtype), rnd(N, Kd, dtype=dtype, seed=1), rnd(N, seed=2)
    want = x.double() @ w.double().T
    out = torch.empty(M, N, device=DEV)
    K().gemm_simt(x, w, out)
    assert torch.allclose(out.double(), want, rtol=1e-5, atol=1e-4)
    K().gemm_simt(x, w, out, bias=bias)
    assert torch.allclose(out.double(), want + bias.double(), rtol=1e-5, atol=1e-4)
    base = rnd(M, N, seed=3)
    acc = base.clone()
    K().gemm_simt(x, w, acc, accumulate=True)
    assert torch.allclose(acc.double(), want + base.double(), rtol=1e-5, atol=1e-4)
    ob = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    K().gemm_simt(x, w, ob)
    assert torch.allclose(ob.double(), want, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("M", [1, 2, 7, 8, 9, 16, 17, 31, 33, 64])
@pytest.mark.parametrize("N,Kd", [(16, 8), (1, 64), (50, 40), (301, 240), (2048, 2048), (300, 8200), (9600, 96)])
def test_gemm_small_m(M, N, Kd):
    x, w = rnd(M, Kd, dtype=torch.bfloat16), rnd(N, Kd, dtype=torch.bfloat16, seed=1)
    bias = rnd(N, seed=2)
    want = x.double() @ w.double().T
    tol = dict(rtol=1e-4, atol=1e-3 * math.sqrt(Kd / 64))
    out = torch.full((M, N), float("nan"), device=DEV)
    K().gemm_small_m(x, w, out)
    assert torch.allclose(out.double(), want, **tol)
    base = rnd(M, N, seed=3)
    acc = base.clone()
    K().gemm_small_m(x, w, acc, bias=bias, accumulate=True)
    assert torch.allclose(acc.double(), want + base.double() + bias.double(), **tol)
    again = base.clone()
    K().gemm_small_m(x, w, again, bias=bias, accumulate=True)
    assert torch.equal(acc, again)               # the same bits in every run


def test_gemm_small_m_refuses_what_it_cannot_do():
    x, w = rnd(65, 64, dtype=torch.bfloat16), rnd(8, 64, dtype=torch.bfloat16)
    with pytest.raises(K().KernelError):
        K().gemm_small_m(x, w, torch.empty(65, 8, device=DEV))
    with pytest.raises(K().KernelError):
        K().gemm_small_m(rnd(2, 12, dtype=torch.bfloat16), rnd(8, 12, dtype=torch.bfloat16),
                         torch.empty(2, 8, device=DEV))
    with pytest.raises(K().KernelError):
        K().gemm_simt(rnd(2, 8).cpu(), rnd(8, 8).cpu(), torch.empty(2, 8))
