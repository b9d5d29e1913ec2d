"""The sampling kernel against the plain sampler on the same logits."""
import pytest
import torch

import plain_lfm2 as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def run_kernel(logits, seed, streams, steps, recent, **kw):
    from mivi_v4_b200.ops import kernels as K
    B, V = logits.shape
    lg = logits.to(DEV)
    work = torch.empty(B, K.sample_scratch_width(V), device=DEV)
    out = torch.empty(B, dtype=torch.int32, device=DEV)
    rec = torch.zeros(B, 64, dtype=torch.int32)
    nrec = torch.zeros(B, dtype=torch.int32)
    for b, r in enumerate(recent):
        r = list(r)[-64:]
        rec[b, :len(r)] = torch.tensor(r, dtype=torch.int32)
        nrec[b] = len(r)
    K.sample(lg, work, out, recent=rec.to(DEV), n_recent=nrec.to(DEV), seed=seed,
             streams=torch.tensor(streams, dtype=torch.int32, device=DEV),
             steps=torch.tensor(steps, dtype=torch.int32, device=DEV), **kw)
    assert torch.equal(lg.cpu(), logits)              # the caller's logits are left alone
    return out.tolist()


CASES = [
    dict(temperature=0.0),
    dict(temperature=0.0, repetition_penalty=1.3, presence_penalty=0.2, frequency_penalty=0.1),
    dict(temperature=0.8),
    dict(temperature=1.5, top_k=5),
    dict(temperature=0.7, top_p=0.9),
    dict(temperature=1.0, min_p=0.05),
    dict(temperature=0.9, top_k=40, top_p=0.9, min_p=0.02, repetition_penalty=1.1),
    dict(temperature=0.2, top_k=40, top_p=0.9, repetition_penalty=1.05),        # the reference's defaults
    dict(temperature=2.0, top_p=0.3),
]


@pytest.mark.parametrize("kw", CASES, ids=[str(i) for i in range(len(CASES))])
@pytest.mark.parametrize("V", [301, 4100, 65536])
def test_sample_matches_plain(kw, V):
    g = torch.Generator().manual_seed(V)
    B = 6
    logits = torch.randn(B, V, generator=g) * 3.0
    logits[1, 7] = logits[1].max() + 0.0                 # a tie for the maximum: the first one wins
    logits[1, 3] = logits[1, 7]
    logits[2] = torch.round(logits[2])                   # many exact ties inside the distribution
    seed, streams, steps = 1234, [0, 1, 2, 3, 70000, 5], [0, 5, 9, 2, 1, 63]
    recent = [[], [3, 3, 7, 9], list(range(80)), [V - 1], [5] * 10, [1, 2, 3]]
    got = run_kernel(logits, seed, streams, steps, recent, **kw)
    for b in range(B):
        want = P.plain_sample(logits[b], recent=recent[b][-64:], u=P.plain_uniform(seed, streams[b], steps[b]), **kw)
        assert got[b] == want, (b, kw, got[b], want)


def test_draw_depends_on_stream_and_step_not_on_the_batch():
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(1, 500, generator=g).repeat(8, 1)
    a = run_kernel(logits, 9, [4] * 8, list(range(8)), [[]] * 8, temperature=1.0)
    assert len(set(a)) > 3                                # different steps draw different tokens
    b = run_kernel(logits[:3], 9, [4] * 3, [5, 6, 7], [[]] * 3, temperature=1.0)
    assert b == a[5:8]                                    # the same (stream, step) in another batch
    c = run_kernel(logits, 10, [4] * 8, list(range(8)), [[]] * 8, temperature=1.0)
    assert c != a


def test_distribution_of_draws():
    p = torch.tensor([0.5, 0.25, 0.125, 0.125])
    logits = p.log().repeat(4000, 1)
    got = run_kernel(logits, 3, list(range(4000)), [0] * 4000, [[]] * 4000, temperature=1.0)
    freq = torch.bincount(torch.tensor(got), minlength=4).double() / 4000
    assert (freq - p.double()).abs().max() < 0.03
    got = run_kernel(logits, 3, list(range(4000)), [0] * 4000, [[]] * 4000, temperature=1.0, top_p=0.7)
    freq = torch.bincount(torch.tensor(got), minlength=4).double() / 4000
    assert freq[2] == 0 and freq[3] == 0 and abs(freq[0] - 2 / 3) < 0.03


def test_large_vocabulary():
    g = torch.Generator().manual_seed(5)
    logits = torch.randn(2, 65536, generator=g) * 2
    assert run_kernel(logits, 0, [0, 1], [0, 0], [[], []], temperature=0.0) == logits.argmax(1).tolist()
    got = run_kernel(logits, 0, [0, 1], [0, 0], [[], []], temperature=1.0, top_k=3)
    top3 = logits.topk(3, dim=1).indices.tolist()
    assert got[0] in top3[0] and got[1] in top3[1]
    want = [P.plain_sample(logits[b], temperature=1.0, top_k=3, u=P.plain_uniform(0, b, 0)) for b in range(2)]
    assert got == want


@pytest.mark.parametrize("kw", [dict(temperature=0.0, repetition_penalty=1.5, frequency_penalty=0.3),
                                dict(temperature=0.9, top_k=30, top_p=0.95, repetition_penalty=1.3, presence_penalty=0.4)])
def test_recent_tokens_kept_on_the_device(kw):
    """The kernel keeps the recent tokens in a ring of its own: over 200 steps (the window of 64 wraps
    three times) it samples what it samples when the caller hands it the last 64 tokens; two rows use
    states that are not their row numbers; a step run twice gives the same token twice."""
    from mivi_v4_b200.ops import kernels as K
    V, B, steps_n = 97, 2, 200
    g = torch.Generator().manual_seed(3)
    base = torch.randn(B, V, generator=g)
    ring = torch.full((6, K.RECENT_RING), -7, dtype=torch.int32, device=DEV)       # stale contents
    rows = torch.tensor([4, 1], dtype=torch.int32, device=DEV)
    work = torch.empty(B, K.sample_scratch_width(V), device=DEV)
    out = torch.empty(B, dtype=torch.int32, device=DEV)
    streams = torch.tensor([11, 12], dtype=torch.int32, device=DEV)
    history = [[], []]
    for s in range(steps_n):
        logits = (base + 0.3 * torch.randn(B, V, generator=g)).to(DEV)
        st = torch.tensor([s, s], dtype=torch.int32, device=DEV)
        K.sample(logits, work, out, seed=5, streams=streams, steps=st, ring=ring, ring_rows=rows, **kw)
        got = out.tolist()
        if s % 37 == 5:                                   # the same step once more: the same tokens
            K.sample(logits, work, out, seed=5, streams=streams, steps=st, ring=ring, ring_rows=rows, **kw)
            assert out.tolist() == got
        want = run_kernel(logits.cpu(), 5, [11, 12], [s, s], [h[-64:] for h in history], **kw)
        assert got == want, (s, got, want)
        for b in range(B):
            history[b].append(got[b])
    assert len(set(history[0])) > 5                       # the penalties did spread the tokens


@pytest.mark.parametrize("kw", [dict(temperature=1.0, top_k=5, top_p=0.9), dict(temperature=1.0, top_p=0.9),
                                dict(temperature=0.7), dict(temperature=1.0, top_k=2000, top_p=0.33333)],
                         ids=["top_k_top_p", "top_p", "temperature", "large_top_k"])
@pytest.mark.parametrize("V", [4100, 70000, 131072, 140001])
def test_top_k_with_a_wall_of_ties(V, kw):
    """More values tie at the k-th place than the kernel's list of survivors holds (rows of equal
    logits, and a row with 2,000 equal maxima): the row is then sampled the slow way, with the same result.
    Without top_k the nucleus' edge falls into the wall, and the ties are counted in index order across
    the blocks that share a row; the largest vocabulary is one that those blocks cannot hold."""
    logits = torch.zeros(3, V)
    logits[1, ::2] = 1.0
    g = torch.Generator().manual_seed(1)
    logits[2] = torch.randn(V, generator=g)
    logits[2, 100:2100] = 9.0
    seed, streams, steps = 7, [0, 1, 2], [3, 4, 5]
    got = run_kernel(logits, seed, streams, steps, [[], [], []], **kw)
    for b in range(3):
        want = P.plain_sample(logits[b], recent=[], u=P.plain_uniform(seed, streams[b], steps[b]), **kw)
        assert got[b] == want, (b, got[b], want)


@pytest.mark.parametrize("kw", [dict(temperature=0.2, top_k=40, top_p=0.9, repetition_penalty=1.05),
                                dict(temperature=0.8, top_p=0.9), dict(temperature=1.1)],
                         ids=["defaults", "top_p", "temperature"])
@pytest.mark.parametrize("V", [4100, 30001])
def test_many_rows(V, kw):
    """More rows than take eight blocks each: they are sampled by four blocks a row, with the same tokens."""
    g = torch.Generator().manual_seed(V + 1)
    B = 20
    logits = torch.randn(B, V, generator=g) * 2.5
    logits[3] = torch.round(logits[3] * 2) / 2
    seed, streams, steps = 77, list(range(100, 100 + B)), [3 * b for b in range(B)]
    recent = [[(7 * b + j) % V for j in range(b)] for b in range(B)]
    got = run_kernel(logits, seed, streams, steps, recent, **kw)
    for b in range(B):
        want = P.plain_sample(logits[b], recent=recent[b][-64:], u=P.plain_uniform(seed, streams[b], steps[b]), **kw)
        assert got[b] == want, (b, got[b], want)
