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
@pytest.mark.parametrize("n,H,eps", [(1, 16, 1e-5), (7, 200, 1e-6), (3, 2048, 1e-5), (2, 5000, 1e-3),
                                     (600, 2048, 1e-5), (513, 516, 1e-6)])       # many rows: a warp a row
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
    if n < 512:
        assert torch.equal(out2, out[rows.long()])
    else:       # many rows take another kernel, which adds the squares in another order
        assert torch.allclose(out2.double(), out[rows.long()].double(), rtol=tol, atol=tol)


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


@pytest.mark.parametrize("kernel,M", [(k, M) for k in ("gemm_small_m", "gemm_tc_swap")
                                      for M in (1, 2, 7, 8, 9, 16, 17, 31, 33, 64)] +
                         # the kernel with swapped operands takes any number of rows: tiles of 128 tokens
                         [("gemm_tc_swap", M) for M in (65, 128, 129, 300, 1000)])
@pytest.mark.parametrize("N,Kd", [(16, 8), (1, 64), (50, 40), (301, 240), (2048, 2048), (300, 8200), (9600, 96)])
def test_gemm_small_m(kernel, M, N, Kd):
    fn = getattr(K(), kernel)
    x, w = rnd(M, Kd, dtype=torch.bfloat16), rnd(N, Kd, dtype=torch.bfloat16, seed=1)
    bias = rnd(N, seed=2)
    want = x.double() @ w.double().T
    tol = dict(rtol=1e-4, atol=1e-3 * math.sqrt(Kd / 64))
    out = torch.full((M, N), float("nan"), device=DEV)
    fn(x, w, out)
    assert torch.allclose(out.double(), want, **tol)
    base = rnd(M, N, seed=3)
    acc = base.clone()
    fn(x, w, acc, bias=bias, accumulate=True)
    assert torch.allclose(acc.double(), want + base.double() + bias.double(), **tol)
    again = base.clone()
    fn(x, w, again, bias=bias, accumulate=True)
    assert torch.equal(acc, again)               # the same bits in every run
    ob = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    fn(x, w, ob)
    assert torch.allclose(ob.double(), want, rtol=1e-2, atol=1e-2 * math.sqrt(Kd / 64))
    K().check_device_errors()


@pytest.mark.parametrize("kernel,M,H,F,swiglu",
                         [(k, M, H, F, sw) for k in ("gemm_small_m", "gemm_tc_swap") for M in (1, 5, 8, 17, 64)
                          for H, F, sw in ((64, 48, False), (200, 96, True), (2048, 160, False), (9600, 64, True))] +
                         [("gemm_tc_swap", M, H, F, sw) for M in (65, 200, 515)
                          for H, F, sw in ((200, 96, True), (2048, 160, False))] +
                         # the one-multiprocessor prefill kernels only apply a scale: the swapped kernel emits
                         [("gemm_tc_one", M, H, F, sw) for M in (65, 200, 1000)
                          for H, F, sw in ((200, 96, True), (2048, 48, False), (2048, 4096, True))] +
                         # the prefill product of two multiprocessors a tile: more than 128 rows, an emitting
                         # product's width in steps of 32, a consuming one's at least 128
                         [("gemm_tc_pair", M, H, F, sw) for M in (129, 300, 1000)
                          for H, F, sw in ((128, 208, True), (256, 160, True), (2048, 384, False), (9600, 128, False),
                                           (2048, 8192, True))])
def test_gemm_carries_a_norm(kernel, M, H, F, swiglu):
    """x_new = x + z Wo^T; y = rmsnorm(x_new) * g, then y W1^T (or its SwiGLU): the first product
    writes the rows bf16(x_new * g) and the tile sums, the second applies the scale."""
    import functools
    gemm = functools.partial(K().gemm_tc, pair=True) if kernel == "gemm_tc_pair" else \
        functools.partial(K().gemm_tc, pair=False) if kernel == "gemm_tc_one" else getattr(K(), kernel)
    emitter = K().gemm_tc_swap if kernel == "gemm_tc_one" else gemm
    from mivi_v4_b200.ops.linear import linear
    eps = 1e-5
    z, wo = rnd(M, 72, dtype=torch.bfloat16), rnd(H, 72, dtype=torch.bfloat16, seed=1)
    x = rnd(M, H, scale=2.0, seed=2)
    g = rnd(H, seed=3) + 1.0
    w1 = rnd(2 * F if swiglu else F, H, dtype=torch.bfloat16, seed=4)
    bias = None if swiglu else rnd(F, seed=5)
    link = K().NormLink(None, g, eps, H, torch.empty(M, H, dtype=torch.bfloat16, device=DEV),
                        torch.full((M, -(-H // 64) * 4), float("nan"), device=DEV))
    resid = x.clone()
    emitter(z, wo, resid, accumulate=True, emit=link)
    K().check_device_errors()
    x_new = x.double() + z.double() @ wo.double().T
    assert torch.allclose(resid.double(), x_new, rtol=1e-5, atol=1e-4)
    assert link.n_partials == {"gemm_small_m": -(-H // (32 if H >= 9472 else 16)), "gemm_tc_swap": -(-H // 128),
                               "gemm_tc_one": -(-H // 128), "gemm_tc_pair": -(-H // 256)}[kernel]
    ss = link.partials[:, :link.n_partials].double().sum(1)
    assert torch.allclose(ss, (x_new ** 2).sum(1), rtol=1e-5)
    # the rows handed on are x_new * g, rounded once to bfloat16 (x_new itself is a float32 sum: 1e-5)
    xg_want = x_new * g.double()
    xg_err = (link.xg.double() - xg_want).abs() - (2.0 ** -8 * xg_want.abs() + 1e-5)
    assert (xg_err <= 0).all(), xg_err.max()
    y = P.plain_rms_norm(x_new, g.double(), eps)
    own = link.xg.double() * torch.rsqrt(ss / H + eps)[:, None]      # what the consumer multiplies, exactly
    if swiglu:
        out = torch.empty(M, F, dtype=torch.bfloat16, device=DEV)
        gemm(link.xg, w1, out, swiglu=True, scale=link)

        def glu(rows):
            gu = (rows @ w1.double().T).view(M, F // 16, 2, 16)
            a, b = gu[:, :, 0].reshape(M, F), gu[:, :, 1].reshape(M, F)
            return a / (1 + torch.exp(-a)) * b, a, b
        want, a, b = glu(y)
        want_own, a_own, b_own = glu(own)
        # from the rows it was given: float32 sums (2^-20 of the terms' size) and one rounding to bfloat16
        tight = 2.0 ** -8 * want_own.abs() + 1e-4 * math.sqrt(H) * (a_own.abs() + b_own.abs() + 1)
    else:
        out = torch.empty(M, F, device=DEV)
        gemm(link.xg, w1, out, bias=bias, scale=link)
        want = y @ w1.double().T + bias.double()
        want_own = own @ w1.double().T + bias.double()
        tight = 1e-5 * want_own.abs() + 1e-4 * math.sqrt(H)
    K().check_device_errors()
    assert ((out.double() - want_own).abs() <= tight).all(), ((out.double() - want_own).abs() - tight).max()
    # against the norm in full precision: rounding x_new * g to bfloat16 moves a dot product of H terms by
    # about 2^-9 sqrt(H) a term of size 1, delta being six times its standard deviation; silu(a) b moves by
    # about (|a| + |b|) delta.  Over the millions of values of the large cases a few lie further out.
    delta = 1e-2 * math.sqrt(H)
    bound = delta * (a.abs() + b.abs() + 1) + 1e-2 * want.abs() if swiglu else delta + 1e-2 * want.abs()
    err = (out.double().cpu() - want.cpu()).abs()
    if err.numel() <= 64 * 1024:
        assert (err <= bound.cpu()).all(), (err - bound.cpu()).max()
    else:
        assert (err <= 2 * bound.cpu()).all() and (err > bound.cpu()).double().mean() < 1e-4
    # the same through the norm kernel and a plain product, for the size of the difference
    u = torch.empty(M, H, dtype=torch.bfloat16, device=DEV)
    K().rmsnorm(resid, g, eps, u)
    if not swiglu:
        ref = torch.empty(M, F, device=DEV)
        linear(u, w1, ref, bias=bias)
        assert (out - ref).abs().max() <= 2 * (ref.double() - want).abs().max() + 1e-3


def test_gemm_small_m_refuses_what_it_cannot_do():
    x, w = rnd(65, 64, dtype=torch.bfloat16), rnd(8, 64, dtype=torch.bfloat16)
    with pytest.raises(K().KernelError):
        K().gemm_small_m(x, w, torch.empty(65, 8, device=DEV))
    with pytest.raises(K().KernelError):
        K().gemm_small_m(rnd(2, 12, dtype=torch.bfloat16), rnd(8, 12, dtype=torch.bfloat16),
                         torch.empty(2, 8, device=DEV))
    with pytest.raises(K().KernelError):
        K().gemm_simt(rnd(2, 8).cpu(), rnd(8, 8).cpu(), torch.empty(2, 8))


# ---------------------------------------------------------------- attention
def build_cache(lengths, nkv, hd, page_size, dtype, seed=0):
    """Random keys and values of sequences with these lengths, laid into pages
    handed out in a shuffled order; returns pool, page table, and the dense
    copies [len, nkv, hd] for the plain expression."""
    g = torch.Generator().manual_seed(seed)
    blocks = [-(-n // page_size) for n in lengths]
    n_pages = sum(blocks) + 3
    order = torch.randperm(n_pages, generator=g).tolist()
    pool = torch.zeros(n_pages, 2, nkv, page_size, hd, dtype=dtype)
    table = torch.zeros(len(lengths), max(blocks) + 2, dtype=torch.int32)
    dense = []
    for b, n in enumerate(lengths):
        k = torch.randn(n, nkv, hd, generator=g).to(dtype)
        v = torch.randn(n, nkv, hd, generator=g).to(dtype)
        dense.append((k, v))
        for blk in range(blocks[b]):
            page = order.pop()
            table[b, blk] = page
            lo, hi = blk * page_size, min(n, (blk + 1) * page_size)
            pool[page, 0, :, :hi - lo] = k[lo:hi].permute(1, 0, 2)
            pool[page, 1, :, :hi - lo] = v[lo:hi].permute(1, 0, 2)
    return pool.to(DEV), table.to(DEV), dense


def plain_attend(q, k, v, pos, nh, nkv, scale, window):
    """softmax(q.k / sqrt(hd)) v over keys t <= pos (and t > pos - window), float64."""
    q, k, v = q.double(), k.double(), v.double()
    hd = q.shape[-1]
    out = torch.zeros(nh, hd, dtype=torch.float64)
    lo = max(0, pos - window + 1) if window > 0 else 0
    for h in range(nh):
        g = h // (nh // nkv)
        s = (k[lo:pos + 1, g] @ q[h]) * scale
        out[h] = torch.softmax(s, 0) @ v[lo:pos + 1, g]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("kernel", ["generic", "decode", "decode_1split", "decode_7splits"])
@pytest.mark.parametrize("nh,nkv,hd,page,window", [
    (4, 2, 16, 16, 0), (3, 1, 32, 64, 0), (5, 5, 48, 32, 0), (32, 8, 64, 64, 0), (12, 1, 128, 64, 0),
    (2, 2, 256, 8, 0), (8, 2, 64, 64, 37), (6, 3, 80, 16, 64)])
def test_attention_kernels(dtype, kernel, nh, nkv, hd, page, window):
    from mivi_v4_b200.engine.step import Workspace
    lengths = [1, 33, 300, 64, 129]
    pool, table, dense = build_cache(lengths, nkv, hd, page, dtype, seed=nh + hd)
    # query tokens: the last position of every sequence, and some in the middle (a step may
    # bring several tokens of one sequence, each sees the keys up to its own position)
    queries = [(b, n - 1) for b, n in enumerate(lengths)] + [(2, 0), (2, 31), (2, 32), (2, 255), (4, 64), (4, 63)]
    g = torch.Generator().manual_seed(1)
    q = torch.randn(len(queries), nh, hd, generator=g)
    # make one far key of the longest sequence stand out for head 0, so that a kernel that
    # loses it (a wrong page, a dropped run, a bad split) cannot pass
    far = 5
    k2 = dense[2][0]
    q[2, 0] = (k2[far, 0].float() / k2[far, 0].float().norm()) * 6.0 * (hd ** 0.25)
    q = q.to(dtype)
    scale = 1.0 / math.sqrt(hd)
    seq_of, positions = ints([b for b, _ in queries]), ints([p for _, p in queries])
    qd = q.reshape(len(queries), nh * hd).contiguous().to(DEV)
    out = torch.empty_like(qd)
    if kernel == "generic":
        K().attention_generic(qd, pool, table, positions, seq_of, out, nh, nkv, hd, scale, window)
    else:
        ws = Workspace(DEV)
        splits = {"decode": None, "decode_1split": 1, "decode_7splits": 7}[kernel]
        for _ in range(2):          # twice: the ticket counters must be back at zero
            out.fill_(float("nan"))
            K().attention_decode(qd, pool, table, positions, seq_of, out, nh, nkv, hd, scale, window, ws,
                                 splits=splits)
    tol = 2e-5 if dtype == torch.float32 else 1.5e-2
    for i, (b, p) in enumerate(queries):
        want = plain_attend(q[i], dense[b][0], dense[b][1], p, nh, nkv, scale, window)
        got = out[i].reshape(nh, hd).double().cpu()
        assert torch.allclose(got, want, rtol=tol, atol=tol), (kernel, i, b, p, (got - want).abs().max())
    if window == 0:
        w = torch.softmax((dense[2][0][:, 0].double() @ q[2, 0].double()) * scale, 0)
        assert w[far] > 0.5          # the far key does dominate


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("style", ["interleaved", "half_split"])
@pytest.mark.parametrize("nh,nkv,hd,eps,theta", [(4, 2, 16, 1e-5, 1e4), (3, 1, 32, 1e-6, 1e6), (5, 5, 48, 1e-5, 5e4)])
def test_qk_prepare(dtype, style, nh, nkv, hd, eps, theta):
    page = 16
    lengths = [40, 7]
    pool = torch.zeros(8, 2, nkv, page, hd, dtype=dtype, device=DEV)
    table = ints([[3, 5, 1], [6, 0, 0]])
    toks = [(0, p) for p in (0, 15, 16, 39)] + [(1, 6)]
    qkv = rnd(len(toks), (nh + 2 * nkv) * hd, scale=2.0)
    wq, wk = rnd(hd) + 1.0, rnd(hd, seed=1) + 1.0
    inv = (1.0 / (torch.tensor(theta, dtype=torch.float64) ** (2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd)))
    q_out = torch.empty(len(toks), nh * hd, dtype=dtype, device=DEV)
    K().qk_prepare(qkv, wq, wk, eps, inv.float().to(DEV), style == "half_split", ints([p for _, p in toks]),
                   ints([b for b, _ in toks]), table, pool, q_out, nh, nkv, hd)
    pos = torch.tensor([p for _, p in toks])
    x = qkv.double().cpu()
    qw = P.plain_rope(P.plain_rms_norm(x[:, :nh * hd].reshape(-1, nh, hd), wq.double().cpu(), eps), pos, theta, style)
    kw = P.plain_rope(P.plain_rms_norm(x[:, nh * hd:(nh + nkv) * hd].reshape(-1, nkv, hd), wk.double().cpu(), eps),
                      pos, theta, style)
    vw = x[:, (nh + nkv) * hd:].reshape(-1, nkv, hd)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(q_out.double().cpu().reshape(-1, nh, hd), qw, rtol=tol, atol=tol)
    tab = table.cpu()
    for i, (b, p) in enumerate(toks):
        pg = int(tab[b, p // page])
        assert torch.allclose(pool[pg, 0, :, p % page].double().cpu(), kw[i], rtol=tol, atol=tol)
        assert torch.allclose(pool[pg, 1, :, p % page].double().cpu(), vw[i], rtol=tol, atol=tol)
    written = sum(1 for _ in toks) * 2 * nkv * hd
    assert int((pool != 0).sum()) <= written     # nothing was written anywhere else


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("nh,nkv,normed,rotated", [(32, 8, True, True), (3, 1, True, True), (5, 2, False, True),
                                                   (4, 4, True, False), (7, 3, False, False)])
@pytest.mark.parametrize("lengths", [[301, 260], [40, 31], [2000, 900]], ids=["561", "71", "2900"])
def test_qk_prepare_many_tokens_heads_of_64(dtype, nh, nkv, normed, rotated, lengths):
    """Steps of 65 tokens and more with heads of 64 take a kernel of their own (a warp a token, two heads a
    round; with few tokens a token's heads go to several warps): odd head counts, so that the two halves of
    a warp hold heads of different kinds; two sequences whose tokens lie in shuffled pages; with and without
    the norm and the rotation."""
    hd, page, eps, theta = 64, 16, 1e-5, 10000.0
    g = torch.Generator().manual_seed(nh * 10 + nkv)
    blocks = [-(-n // page) for n in lengths]
    order = torch.randperm(sum(blocks) + 2, generator=g).tolist()
    table = torch.zeros(2, max(blocks), dtype=torch.int32)
    for b in range(2):
        for blk in range(blocks[b]):
            table[b, blk] = order.pop()
    pool = torch.zeros(sum(blocks) + 2, 2, nkv, page, hd, dtype=dtype, device=DEV)
    toks = [(0, p) for p in range(lengths[0])] + [(1, p) for p in range(lengths[1])]
    qkv = rnd(len(toks), (nh + 2 * nkv) * hd, scale=2.0)
    wq, wk = (rnd(hd) + 1.0, rnd(hd, seed=1) + 1.0) if normed else (None, None)
    inv = (1.0 / (torch.tensor(theta, dtype=torch.float64) ** (2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd)))
    q_out = torch.full((len(toks), nh * hd), float("nan"), dtype=dtype, device=DEV)
    K().qk_prepare(qkv, wq, wk, eps, inv.float().to(DEV) if rotated else None, False, ints([p for _, p in toks]),
                   ints([b for b, _ in toks]), table.to(DEV), pool, q_out, nh, nkv, hd)
    pos = torch.tensor([p for _, p in toks])
    x = qkv.double().cpu()
    qw, kw = x[:, :nh * hd].reshape(-1, nh, hd), x[:, nh * hd:(nh + nkv) * hd].reshape(-1, nkv, hd)
    if normed:
        qw, kw = P.plain_rms_norm(qw, wq.double().cpu(), eps), P.plain_rms_norm(kw, wk.double().cpu(), eps)
    if rotated:
        def rotate(v):
            # the angle as the kernels define it, a float32 product of position and frequency (at position 2,000
            # that differs from the exact product by 2e-4 rad); up to a few hundred tokens the plain rotation
            # with exact angles agrees within the tolerance and is what is compared
            if max(lengths) <= 512:
                return P.plain_rope(v, pos, theta, "interleaved")
            ang = (pos.float()[:, None] * inv.float()[None, :]).double()
            c, sn = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
            out = torch.empty_like(v)
            out[..., 0::2] = v[..., 0::2] * c - v[..., 1::2] * sn
            out[..., 1::2] = v[..., 0::2] * sn + v[..., 1::2] * c
            return out
        qw, kw = rotate(qw), rotate(kw)
    vw = x[:, (nh + nkv) * hd:].reshape(-1, nkv, hd)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(q_out.double().cpu().reshape(-1, nh, hd), qw, rtol=tol, atol=tol * 4)
    got_k = torch.stack([pool[int(table[b, p // page]), 0, :, p % page] for b, p in toks]).double().cpu()
    got_v = torch.stack([pool[int(table[b, p // page]), 1, :, p % page] for b, p in toks]).double().cpu()
    assert torch.allclose(got_k, kw, rtol=tol, atol=tol * 4) and torch.allclose(got_v, vw, rtol=tol, atol=tol * 4)
    assert int((pool != 0).sum()) <= len(toks) * 2 * nkv * hd        # nothing was written anywhere else


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("H,k,bias", [(8, 3, False), (200, 4, True), (64, 2, False), (16, 1, True), (24, 7, False),
                                      (10, 3, True), (2048, 3, False)])
def test_shortconv_any_cut(out_dtype, H, k, bias):
    """Whole sequences against the plain loop, then the same sequences cut at
    every place: the state carries the left context."""
    T = [9, 4, 1]
    g = torch.Generator().manual_seed(H + k)
    p_all = [torch.randn(t, 3 * H, generator=g) for t in T]
    w = torch.randn(H, k, generator=g)
    b = torch.randn(H, generator=g) if bias else None

    def plain(p):
        bx = p[:, :H].double() * p[:, 2 * H:].double()
        y = torch.zeros_like(bx)
        for t in range(p.shape[0]):
            for j in range(k):
                src = t - (k - 1) + j
                if src >= 0:
                    y[t] += w[:, j].double() * bx[src]
        if b is not None:
            y = y + b.double()
        return p[:, H:2 * H].double() * y

    want = [plain(p) for p in p_all]
    tol = 1e-5 if out_dtype == torch.float32 else 2e-2
    wd, bd = w.to(DEV), (b.to(DEV) if bias else None)

    def run(cuts):
        """cuts[b] = list of chunk lengths of sequence b; chunk i of every sequence runs in step i."""
        state = torch.zeros(5, k - 1, H, device=DEV)
        slots = [3, 0, 4]
        done = [0, 0, 0]
        got = [[] for _ in T]
        for step in range(max(len(c) for c in cuts)):
            live = [s for s in range(len(T)) if step < len(cuts[s])]
            lens = [cuts[s][step] for s in live]
            rows = torch.cat([p_all[s][done[s]:done[s] + n] for s, n in zip(live, lens)]).to(DEV).contiguous()
            cu = [0]
            for n in lens:
                cu.append(cu[-1] + n)
            out = torch.empty(rows.shape[0], H, dtype=out_dtype, device=DEV)
            K().shortconv(rows, wd, bd, state, ints([done[s] + i for s, n in zip(live, lens) for i in range(n)]),
                          ints([j for j, n in enumerate(lens) for _ in range(n)]), ints(cu),
                          ints([slots[s] for s in live]), ints([done[s] for s in live]), ints(lens), out, len(live),
                          decode=all(n == 1 for n in lens))       # one token each: the fused kernel
            for j, (s, n) in enumerate(zip(live, lens)):
                got[s].append(out[cu[j]:cu[j] + n])
                done[s] += n
        return [torch.cat(x).double().cpu() for x in got], state

    whole, st_whole = run([[t] for t in T])
    for a, b_ in zip(whole, want):
        assert torch.allclose(a, b_, rtol=tol, atol=tol)
    for cuts in ([[5, 4], [1, 3], [1]], [[1] * 9, [2, 2], [1]], [[8, 1], [4], [1]], [[2, 1, 6], [1, 1, 2], [1]]):
        part, st = run(cuts)
        for a, b_ in zip(part, want):
            assert torch.allclose(a, b_, rtol=tol, atol=tol), cuts
        assert torch.equal(st, st_whole), cuts       # the same state whatever the cut


@pytest.mark.parametrize("M,N,Kd", [(65, 16, 8), (128, 128, 64), (129, 130, 72), (300, 301, 240), (256, 64, 200),
                                    (1000, 2048, 2048), (2048, 512, 8192), (70, 9600, 96),
                                    # wide enough for the persistent 128 x 256 kernel, ragged in every dimension
                                    (2048, 2048, 512), (1500, 4100, 264), (4096, 6144, 2048), (12300, 300, 72),
                                    (2048, 2048, 8192), (129, 128, 64), (257, 257, 136), (5000, 1100, 392)])
@pytest.mark.parametrize("pair", [False, True], ids=["one_sm", "pair"])
def test_gemm_tc(M, N, Kd, pair):
    """Both tcgen05 products of many rows: one multiprocessor a tile, and two on a 256 x 256 tile."""
    if pair and (M <= 128 or N < 128):
        pytest.skip("the pair kernel takes more than 128 rows and at least 128 columns")
    x, w = rnd(M, Kd, dtype=torch.bfloat16), rnd(N, Kd, dtype=torch.bfloat16, seed=1)
    bias = rnd(N, seed=2)
    want = x.double() @ w.double().T
    tol = dict(rtol=1e-4, atol=1e-3 * math.sqrt(Kd / 64))
    out = torch.full((M, N), float("nan"), device=DEV)
    K().gemm_tc(x, w, out, pair=pair)
    K().check_device_errors()
    assert torch.allclose(out.double(), want, **tol), (out.double() - want).abs().max()
    base = rnd(M, N, seed=3)
    acc = base.clone()
    K().gemm_tc(x, w, acc, bias=bias, accumulate=True, pair=pair)
    assert torch.allclose(acc.double(), want + base.double() + bias.double(), **tol)
    ob = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    K().gemm_tc(x, w, ob, pair=pair)
    assert torch.allclose(ob.double(), want, rtol=1e-2, atol=1e-2 * math.sqrt(Kd / 64))
    K().check_device_errors()


@pytest.mark.parametrize("nh,nkv,hd,page,window", [
    (4, 2, 16, 16, 0), (3, 1, 32, 64, 0), (5, 5, 48, 32, 0), (8, 2, 64, 64, 0), (2, 1, 128, 64, 0),
    (4, 4, 96, 128, 0), (8, 2, 64, 64, 37), (6, 3, 80, 16, 64), (2, 2, 112, 64, 100)])
def test_attention_prefill(nh, nkv, hd, page, window):
    """Chunks of several sequences in one step: (tokens already cached, tokens of this step)."""
    dtype = torch.bfloat16
    chunks = [(0, 1), (0, 200), (130, 70), (5, 64), (63, 66), (300, 3)]
    lengths = [s + n for s, n in chunks]
    pool, table, dense = build_cache(lengths, nkv, hd, page, dtype, seed=nh * hd)
    N = sum(n for _, n in chunks)
    g = torch.Generator().manual_seed(2)
    q = torch.randn(N, nh, hd, generator=g)
    # one far key stands out for the last token of the second sequence
    row_last_b1 = chunks[0][1] + chunks[1][1] - 1
    far = 3
    kf = dense[1][0][far, 0].float()
    q[row_last_b1, 0] = kf / kf.norm() * 6.0 * (hd ** 0.25)
    q = q.to(dtype)
    cu = [0]
    for _, n in chunks:
        cu.append(cu[-1] + n)
    out = torch.full((N, nh * hd), float("nan"), dtype=dtype, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    K().attention_prefill(q.reshape(N, nh * hd).contiguous().to(DEV), pool, table, ints(cu),
                          ints([s for s, _ in chunks]), out, len(chunks), nh, nkv, hd, scale, window)
    tol = 1.5e-2
    for b, (s, n) in enumerate(chunks):
        for i in list(range(0, n, 7)) + [n - 1]:
            want = plain_attend(q[cu[b] + i], dense[b][0], dense[b][1], s + i, nh, nkv, scale, window)
            got = out[cu[b] + i].reshape(nh, hd).double().cpu()
            assert torch.allclose(got, want, rtol=tol, atol=tol), (b, i, (got - want).abs().max())
    assert not torch.isnan(out.float()).any()


@pytest.mark.parametrize("nh,nkv", [(8, 2), (3, 1), (5, 5)])
def test_attention_prefill_tc(nh, nkv):
    """The tcgen05 kernel (head size 64, pages of 64): chunks that start anywhere, span several
    query tiles and key blocks, and end in the middle of a page."""
    dtype, hd, page = torch.bfloat16, 64, 64
    chunks = [(0, 1), (0, 700), (130, 270), (5, 64), (63, 66), (1000, 300), (64, 128), (0, 128)]
    lengths = [s + n for s, n in chunks]
    pool, table, dense = build_cache(lengths, nkv, hd, page, dtype, seed=nh)
    N = sum(n for _, n in chunks)
    g = torch.Generator().manual_seed(2)
    q = torch.randn(N, nh, hd, generator=g)
    cu = [0]
    for _, n in chunks:
        cu.append(cu[-1] + n)
    # one far key stands out for the last token of the second and of the sixth sequence
    for b, far in ((1, 3), (5, 200)):
        kf = dense[b][0][far, 0].float()
        q[cu[b + 1] - 1, 0] = kf / kf.norm() * 6.0 * (hd ** 0.25)
    q = q.to(dtype)
    out = torch.full((N, nh * hd), float("nan"), dtype=dtype, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    K().attention_prefill_tc(q.reshape(N, nh * hd).contiguous().to(DEV), pool, table, ints(cu),
                             ints([s for s, _ in chunks]), out, len(chunks), nh, nkv, hd, scale)
    K().check_device_errors()
    tol = 1.5e-2
    for b, (s, n) in enumerate(chunks):
        for i in sorted(set(list(range(0, n, 7)) + [n - 1] + [x for x in (63, 64, 127, 128, 129) if x < n])):
            want = plain_attend(q[cu[b] + i], dense[b][0], dense[b][1], s + i, nh, nkv, scale, 0)
            got = out[cu[b] + i].reshape(nh, hd).double().cpu()
            assert torch.allclose(got, want, rtol=tol, atol=tol), (b, i, (got - want).abs().max())
    assert not torch.isnan(out.float()).any()


@pytest.mark.parametrize("splits", [None, 1, 3, 7])
@pytest.mark.parametrize("nh,nkv", [(8, 2), (3, 1), (5, 5), (12, 2), (16, 1)])
def test_attention_decode_tc(nh, nkv, splits):
    """The tcgen05 decode kernel (head size 64, pages of 64): single tokens at the end and in the
    middle of caches of many lengths, any number of key splits, with one far key that stands out."""
    from mivi_v4_b200.engine.step import Workspace
    dtype, hd, page = torch.bfloat16, 64, 64
    lengths = [1, 33, 300, 64, 129, 1000, 128, 2500]
    pool, table, dense = build_cache(lengths, nkv, hd, page, dtype, seed=nh + 1)
    queries = [(b, n - 1) for b, n in enumerate(lengths)] + [(2, 0), (2, 127), (2, 128), (5, 511), (7, 1300)]
    g = torch.Generator().manual_seed(1)
    q = torch.randn(len(queries), nh, hd, generator=g)
    for row, far in ((5, 7), (7, 1900)):                     # sequences 5 and 7, last position
        kf = dense[queries[row][0]][0][far, 0].float()
        q[row, 0] = kf / kf.norm() * 6.0 * (hd ** 0.25)
    q = q.to(dtype)
    N = len(queries)
    out = torch.full((N, nh * hd), float("nan"), dtype=dtype, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    K().attention_decode_tc(q.reshape(N, nh * hd).contiguous().to(DEV), pool, table, ints([p for _, p in queries]),
                            ints([b for b, _ in queries]), out, nh, nkv, hd, scale, Workspace(DEV), splits=splits)
    K().check_device_errors()
    assert not torch.isnan(out.float()).any()
    for i, (b, pos) in enumerate(queries):
        want = plain_attend(q[i], dense[b][0], dense[b][1], pos, nh, nkv, scale, 0)
        got = out[i].reshape(nh, hd).double().cpu()
        assert torch.allclose(got, want, rtol=1.5e-2, atol=1.5e-2), (i, b, pos, (got - want).abs().max())


def grouped(w1, w3, G=16):
    F, H = w1.shape
    return torch.stack([w1.view(F // G, G, H), w3.view(F // G, G, H)], dim=1).reshape(2 * F, H).contiguous()


def test_swiglu_grouped_columns():
    N, F = 5, 48
    gu = rnd(N, 2 * F, scale=3.0)
    out = torch.empty(N, F, device=DEV)
    K().swiglu(gu, out, 16)
    v = gu.view(N, F // 16, 2, 16).double()
    a, b = v[:, :, 0].reshape(N, F), v[:, :, 1].reshape(N, F)
    assert torch.allclose(out.double(), a / (1 + torch.exp(-a)) * b, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("M", [1, 8, 9, 33, 64, 65, 200, 1000, 3000])
@pytest.mark.parametrize("F,Kd", [(16, 8), (48, 72), (256, 96), (8192, 2048), (1040, 200)])
def test_gemm_swiglu_epilogue(M, F, Kd):
    """gate and up never reach memory: the product's epilogue applies silu(gate) * up."""
    x = rnd(M, Kd, dtype=torch.bfloat16)
    w1, w3 = rnd(F, Kd, dtype=torch.bfloat16, scale=0.2, seed=1), rnd(F, Kd, dtype=torch.bfloat16, scale=0.2, seed=2)
    a, b = x.double() @ w1.double().T, x.double() @ w3.double().T
    want = a / (1 + torch.exp(-a)) * b
    out = torch.full((M, F), float("nan"), dtype=torch.bfloat16, device=DEV)
    scale = max(1.0, want.abs().max().item())
    import functools
    many = [functools.partial(K().gemm_tc, pair=False), K().gemm_tc_swap] + \
        ([functools.partial(K().gemm_tc, pair=True)] if M > 128 and 2 * F >= 128 else [])
    for fn in ([K().gemm_small_m, K().gemm_tc_swap] if M <= 64 else many):
        out.fill_(float("nan"))
        fn(x, grouped(w1, w3), out, swiglu=True)
        K().check_device_errors()
        assert (out.double() - want).abs().max().item() <= 1e-2 * scale, fn


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("H,k,bias", [(200, 3, False), (136, 4, True), (64, 1, False), (40, 6, True)])
def test_shortconv_long_steps(out_dtype, H, k, bias):
    """Steps with hundreds of tokens of several sequences (the vectorised kernel where the width allows);
    sequences begin anywhere among the packed rows, and a prompt may arrive in two steps."""
    T = [300, 77, 5, 130]
    g = torch.Generator().manual_seed(H * k)
    p_all = [torch.randn(t, 3 * H, generator=g) for t in T]
    w = torch.randn(H, k, generator=g)
    b = torch.randn(H, generator=g) if bias else None
    wd, bd = w.to(DEV), (b.to(DEV) if bias else None)

    def plain(p):
        bx = (p[:, :H] * p[:, 2 * H:]).double()
        y = torch.zeros_like(bx)
        for j in range(k):
            shift = k - 1 - j
            y[shift:] += w[:, j].double() * bx[:bx.shape[0] - shift] if shift else w[:, j].double() * bx
        if b is not None:
            y = y + b.double()
        return p[:, H:2 * H].double() * y

    want = [plain(p) for p in p_all]
    tol = 1e-5 if out_dtype == torch.float32 else 2e-2
    for cuts in ([[t] for t in T], [[260, 40], [77], [1, 4], [2, 128]]):
        state = torch.zeros(6, k - 1, H, device=DEV)
        slots, done, got = [5, 0, 3, 1], [0] * 4, [[] for _ in T]
        for step in range(max(len(c) for c in cuts)):
            live = [s for s in range(len(T)) if step < len(cuts[s])]
            lens = [cuts[s][step] for s in live]
            rows = torch.cat([p_all[s][done[s]:done[s] + n] for s, n in zip(live, lens)]).to(DEV).contiguous()
            cu = [0]
            for n in lens:
                cu.append(cu[-1] + n)
            out = torch.full((rows.shape[0], H), float("nan"), dtype=out_dtype, device=DEV)
            K().shortconv(rows, wd, bd, state, ints([done[s] + i for s, n in zip(live, lens) for i in range(n)]),
                          ints([j for j, n in enumerate(lens) for _ in range(n)]), ints(cu),
                          ints([slots[s] for s in live]), ints([done[s] for s in live]), ints(lens), out, len(live))
            for j, (s, n) in enumerate(zip(live, lens)):
                got[s].append(out[cu[j]:cu[j] + n])
                done[s] += n
        for a, b_ in zip(got, want):
            assert torch.allclose(torch.cat(a).double().cpu(), b_, rtol=tol, atol=tol), cuts


_CONV_SHAPES = [(16, 8, 3, False, False), (200, 72, 4, True, True), (40, 2048, 1, True, False),
                (2048, 2048, 3, False, True), (24, 8200, 7, False, False), (300, 264, 2, True, True)]
# the tcgen05 kernel over regrouped rows: widths in steps of 32
_CONV_SHAPES_GROUPED = [(32, 8, 3, False, False), (96, 72, 4, True, True), (64, 2048, 1, True, False),
                        (2048, 2048, 3, False, True), (160, 8200, 7, False, False), (1536, 264, 2, True, True)]


@pytest.mark.parametrize("kernel,M,H,Kd,k,bias,scaled",
                         [("mma", M) + sh for M in (1, 3, 8) for sh in _CONV_SHAPES] +
                         [("tc", M) + sh for M in (1, 8, 9, 20, 33, 64) for sh in _CONV_SHAPES_GROUPED])
def test_gemm_small_m_shortconv(kernel, M, H, Kd, k, bias, scaled):
    """The decode step's convolution as the epilogue of its input projection (the register-streaming
    kernel up to 8 rows; the tcgen05 kernel up to 64, over rows regrouped by 32 channels): several steps in a row over slots in any order, against a float64 expression
    and against the two separate kernels (same outputs within rounding, same kind of state)."""
    from mivi_v4_b200.ops.kernels import NormLink
    fused = K().gemm_small_m_shortconv if kernel == "mma" else K().gemm_tc_swap_shortconv
    g = torch.Generator().manual_seed(H + Kd + k + M)
    w_in = (torch.randn(3 * H, Kd, generator=g) / math.sqrt(Kd)).to(torch.bfloat16).to(DEV)
    w_fused = w_in
    if kernel == "tc":
        w_fused = K().group_conv_rows(w_in)
        assert torch.equal(w_fused[32:64], w_in[H:H + 32]) and torch.equal(w_fused[64:96], w_in[2 * H:2 * H + 32])
    taps = torch.randn(H, k, generator=g).to(DEV)
    b_in = torch.randn(3 * H, generator=g).to(DEV) if bias else None
    b_conv = torch.randn(H, generator=g).to(DEV) if bias else None
    n_slots = M + 3
    slots = ints(torch.randperm(n_slots, generator=g).tolist()[:M])
    state = torch.zeros(n_slots, k - 1, H, device=DEV)
    state_two = torch.zeros_like(state)
    hist = torch.zeros(M, k - 1, H, dtype=torch.float64)           # the plain side's kept values of B * x
    n_part = 3
    for step in range(k + 2):
        x = torch.randn(M, Kd, generator=g).to(torch.bfloat16).to(DEV)
        link = None
        if scaled:
            # the rows come with partial sums of squares whose total sets a scale per row
            parts = torch.rand(M, n_part + 2, generator=g).to(DEV) * Kd
            link = NormLink(norm=None, weight=torch.ones(Kd, device=DEV), eps=1e-5, dim=Kd, xg=x, partials=parts, n_partials=n_part)
            rs = 1.0 / torch.sqrt(parts[:, :n_part].double().sum(1) / Kd + 1e-5)
        p = x.double() @ w_in.double().T
        if scaled:
            p = p * rs[:, None]
        if bias:
            p = p + b_in.double()
        p = p.cpu()
        bx = p[:, :H] * p[:, 2 * H:]
        y = taps[:, k - 1].double().cpu() * bx
        for j in range(k - 1):
            y = y + taps[:, j].double().cpu() * hist[:, j]
        if bias:
            y = y + b_conv.double().cpu()
        want = p[:, H:2 * H] * y
        hist = torch.cat([hist[:, 1:], bx[:, None]], dim=1) if k > 1 else hist

        out = torch.empty(M, H, dtype=torch.bfloat16, device=DEV)
        fused(x, w_fused, b_in, taps, b_conv, state, slots, out, scale=link)
        K().check_device_errors()
        tol = dict(rtol=2e-2, atol=2e-2 * float(want.abs().max()))
        assert torch.allclose(out.double().cpu(), want, **tol), step
        # the separate kernels
        p32 = torch.empty(M, 3 * H, device=DEV)
        (K().gemm_small_m if kernel == "mma" else K().gemm_tc_swap)(x, w_in, p32, bias=b_in, scale=link)
        out_two = torch.empty(M, H, dtype=torch.bfloat16, device=DEV)
        K().shortconv(p32, taps, b_conv, state_two, None, None, None, slots, None, None, out_two, M, decode=True)
        assert torch.allclose(out.float(), out_two.float(), rtol=2e-2, atol=2e-2 * float(want.abs().max())), step
        if k > 1:
            assert torch.allclose(state, state_two, rtol=1e-4, atol=1e-4 * float(bx.abs().max())), step
            assert torch.allclose(state[slots.long()].double().cpu(), hist, rtol=1e-3, atol=1e-3 * float(bx.abs().max()))
    untouched = [s for s in range(n_slots) if s not in slots.tolist()]
    assert not state[untouched].any()                               # other sequences' state is left alone


@pytest.mark.parametrize("kernel,style,M", [("mma", "interleaved", 7), ("mma", "half_split", 7), ("tc", "interleaved", 7),
                                            ("tc", "interleaved", 9), ("tc", "interleaved", 40), ("tc", "interleaved", 64)])
@pytest.mark.parametrize("nh,nkv,Kd,eps,theta,normed,scaled", [
    (4, 2, 64, 1e-5, 1e4, True, False), (3, 1, 200, 1e-6, 1e6, True, True), (5, 5, 2048, 1e-5, 5e4, False, False),
    (32, 8, 2048, 1e-5, 1e6, True, True), (2, 2, 8200, 1e-5, 1e6, True, False)])
def test_gemm_small_m_heads(kernel, style, M, nh, nkv, Kd, eps, theta, normed, scaled):
    """Norm, rotation and append as the epilogue of the q/k/v projection (heads of 64; the register-streaming
    kernel up to 8 tokens, the tcgen05 kernel, two heads a tile, up to 64): against the plain expressions on a
    float64 product, and against the two separate kernels."""
    from mivi_v4_b200.ops.kernels import NormLink
    hd, page = 64, 16
    pool = torch.zeros(8, 2, nkv, page, hd, dtype=torch.bfloat16, device=DEV)
    pool_two = torch.zeros_like(pool)
    table = ints([[3, 5, 1], [6, 0, 0], [2, 7, 4]])
    toks = [(0, p) for p in (0, 15, 16, 39)] + [(1, 6), (2, 47), (2, 31)]
    # more tokens: further positions of the three sequences, each (sequence, position) once
    more = [(b, p) for p in range(48) for b in (0, 2) if (b, p) not in toks] + [(1, p) for p in range(16) if p != 6]
    toks = (toks + more)[:M]
    x = rnd(M, Kd, dtype=torch.bfloat16)
    w = (rnd((nh + 2 * nkv) * hd, Kd, seed=1) * (2.0 / math.sqrt(Kd))).to(torch.bfloat16)
    wq, wk = (rnd(hd) + 1.0, rnd(hd, seed=1) + 1.0) if normed else (None, None)
    inv = (1.0 / (torch.tensor(theta, dtype=torch.float64) ** (2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd)))
    inv_d = inv.float().to(DEV)
    positions, seq_of = ints([p for _, p in toks]), ints([b for b, _ in toks])
    link = None
    qkv = x.double() @ w.double().T
    if scaled:
        parts = torch.rand(M, 6, device=DEV) * Kd
        link = NormLink(norm=None, weight=torch.ones(Kd, device=DEV), eps=1e-5, dim=Kd, xg=x, partials=parts, n_partials=4)
        qkv = qkv * (1.0 / torch.sqrt(parts[:, :4].double().sum(1) / Kd + 1e-5))[:, None]
    qkv = qkv.cpu()
    q_out = torch.empty(M, nh * hd, dtype=torch.bfloat16, device=DEV)
    if kernel == "mma":
        K().gemm_small_m_heads(x, w, wq, wk, eps, inv_d, style == "half_split", positions, seq_of, table, pool, q_out,
                               nh, nkv, scale=link)
    else:
        K().gemm_tc_swap_heads(x, w, wq, wk, eps, inv_d, positions, seq_of, table, pool, q_out, nh, nkv, scale=link)
    K().check_device_errors()
    pos = torch.tensor([p for _, p in toks])
    qh, kh = qkv[:, :nh * hd].reshape(-1, nh, hd), qkv[:, nh * hd:(nh + nkv) * hd].reshape(-1, nkv, hd)
    if normed:
        qh, kh = P.plain_rms_norm(qh, wq.double().cpu(), eps), P.plain_rms_norm(kh, wk.double().cpu(), eps)
    qw, kw = P.plain_rope(qh, pos, theta, style), P.plain_rope(kh, pos, theta, style)
    vw = qkv[:, (nh + nkv) * hd:].reshape(-1, nkv, hd)
    tol = dict(rtol=2e-2, atol=2e-2 * float(qw.abs().max()))
    assert torch.allclose(q_out.double().cpu().reshape(-1, nh, hd), qw, **tol)
    tab = table.cpu()
    for i, (b, p) in enumerate(toks):
        pg = int(tab[b, p // page])
        assert torch.allclose(pool[pg, 0, :, p % page].double().cpu(), kw[i], **tol)
        assert torch.allclose(pool[pg, 1, :, p % page].double().cpu(), vw[i], **tol)
    assert int((pool != 0).sum()) <= M * 2 * nkv * hd     # nothing was written anywhere else
    # the separate kernels
    p32 = torch.empty(M, (nh + 2 * nkv) * hd, device=DEV)
    (K().gemm_small_m if kernel == "mma" else K().gemm_tc_swap)(x, w, p32, scale=link)
    q_two = torch.empty_like(q_out)
    K().qk_prepare(p32, wq, wk, eps, inv_d, style == "half_split", positions, seq_of, table, pool_two, q_two, nh, nkv, hd)
    assert torch.allclose(q_out.float(), q_two.float(), rtol=2e-2, atol=tol["atol"])
    assert torch.allclose(pool.float(), pool_two.float(), rtol=2e-2, atol=tol["atol"])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("V,H,N", [(37, 24, 5), (301, 200, 3), (50, 2048, 8)])
def test_embed_hands_on_the_first_norm(dtype, V, H, N):
    """The embedding kernel can also write what the product after it needs to apply the first norm
    itself: the rows bf16(x * weight) and partial sums of x^2 that add up to each row's sum."""
    from mivi_v4_b200.ops.kernels import NormLink
    table = rnd(V, H, dtype=dtype)
    tok = ints([V - 1, 0, 7][:N] + [3] * max(0, N - 3))
    g = rnd(H, seed=3) + 1.0
    link = NormLink(norm=None, weight=g, eps=1e-5, dim=H, xg=torch.empty(N, H, dtype=torch.bfloat16, device=DEV),
                    partials=torch.full((N + 1, -(-H // 64) * 4), 7.0, device=DEV))
    out = torch.empty(N, H, device=DEV)
    K().embed(table, tok, out, link)
    want = table[tok.long()].float()
    assert torch.equal(out, want)
    assert torch.equal(link.xg, (want * g).to(torch.bfloat16))
    assert link.n_partials in (4, 8)
    sums = link.partials[:N, :link.n_partials].double().sum(1)
    assert torch.allclose(sums, (want.double() ** 2).sum(1), rtol=1e-5)
    assert bool((link.partials[N] == 7.0).all())                      # no row beyond the step's
    # and a product that takes the link gives what the norm kernel and a plain product give
    w = rnd(48, H, dtype=torch.bfloat16, seed=5)
    if H % 8 == 0:
        y = torch.empty(N, 48, device=DEV)
        K().gemm_small_m(link.xg, w, y, scale=link)
        normed = P.plain_rms_norm(want.double(), g.double(), 1e-5)
        ref = normed @ w.double().T
        assert torch.allclose(y.double(), ref, rtol=2e-2, atol=2e-2 * float(ref.abs().max()))
