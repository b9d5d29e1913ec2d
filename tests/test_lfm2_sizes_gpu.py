"""The engine at the layer sizes of LFM2.5-1.2B (width 2,048, 32 heads on 8 kv heads of 64, feed-forward
8,192 from block_ff_dim 12,288, vocabulary 65,536, tied head, convolution width 3), four layers deep, against
the plain implementation in float32 and in bfloat16, under every way of cutting the work.

At these sizes the engine takes kernels that no tiny model reaches inside the engine: the persistent tcgen05
product with 128x256 tiles, the tcgen05 decode product with K cut over a cluster, norms carried over 2,048
columns, the look-ahead into real weight extents, four query heads a kv head in the tcgen05 decode attention.
The model is the one that ``bench.py`` measures, with fewer layers; its weights go through a model folder, so
the safetensors path sees tensors of real size too.

With N(0, 0.02) matrices at width 2,048 every part moves the residual stream by about as much as it holds,
so a fault in any one part shows (``test_a_fault_would_show_at_these_sizes``).
"""
import pytest
import torch

import plain_lfm2 as P
from helpers import (assert_close, check_cache, forget_view, mutated_logits, plain_logits, plain_noise, plain_view64, would_fail,
                     write_model)
from tiny_configs import ARCH, prompts

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]
IDS = ["f32", "bf16"]

WIDE = dict(
    architectures=ARCH, model_type="lfm2", hidden_size=2048, num_hidden_layers=4, num_attention_heads=32,
    num_key_value_heads=8, vocab_size=65536, block_ff_dim=12288, block_auto_adjust_ff_dim=True,
    block_multiple_of=256, block_ffn_dim_multiplier=1.0,
    layer_types=["conv", "conv", "full_attention", "conv"], rope_theta=1000000.0, norm_eps=1e-5,
    conv_L_cache=3, conv_bias=False, tie_embedding=True)
V = WIDE["vocab_size"]


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    d = write_model(tmp_path_factory.mktemp("wide"), WIDE, 7)
    yield d
    forget_view(d)


_models = {}


@pytest.fixture(scope="module")
def models(folder):
    """The model in each dtype, loaded once for the module."""
    from mivi_v4_b200 import load_model

    def get(dtype):
        if dtype not in _models:
            _models[dtype] = load_model(folder, dtype, "cuda:0")
        return _models[dtype]
    yield get
    _models.clear()


def make_engine(models, dtype, max_tokens=4096, **kw):
    from mivi_v4_b200 import Engine
    return Engine(models(dtype), max_tokens=max_tokens, **kw)


def check(got, folder, toks, dtype, what, rows=None):
    want = plain_logits(folder, toks)
    assert_close(got, want if rows is None else want[rows], dtype, what, noise=plain_noise(folder, toks, dtype))


def test_ff_width_follows_the_rule(models):
    assert models(torch.bfloat16).config.ff_dim == 8192


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_whole_prompts(folder, models, dtype):
    eng = make_engine(models, dtype)
    for toks in prompts(V, [1, 65, 130, 200], seed=3):
        s = eng.open()
        got = eng.step([(s, toks)], "all")
        eng.close(s)
        check(got, folder, toks, dtype, f"whole, {len(toks)} tokens")
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_a_prompt_of_several_row_tiles(folder, models, dtype):
    """700 tokens: three row tiles of the product that pairs two multiprocessors (every projection is wide
    enough for it at this length), the tcgen05 attention over several key blocks; whole, and as chunks of 300
    and 400 tokens beside a second, short sequence."""
    eng = make_engine(models, dtype)
    a, b = prompts(V, [700, 45], seed=6)
    s = eng.open()
    got = eng.step([(s, a)], "all")
    eng.close(s)
    check(got, folder, a, dtype, "700 tokens whole")
    sa, sb = eng.open(), eng.open()
    first = eng.step([(sa, a[:300]), (sb, b[:20])], "all")
    second = eng.step([(sb, b[20:]), (sa, a[300:])], "all")
    eng.close(sa), eng.close(sb)
    check(torch.cat([first[:300], second[25:]]), folder, a, dtype, "700 tokens in chunks of 300 and 400")
    check(torch.cat([first[300:], second[:25]]), folder, b, dtype, "the short sequence beside it")
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_last_32_one_by_one(folder, models, dtype):
    eng = make_engine(models, dtype)
    for toks in prompts(V, [1, 65, 130, 200], seed=3)[2:]:
        s = eng.open()
        cut = len(toks) - 32
        rows = [eng.step([(s, toks[:cut])], "all")]
        rows += [eng.step([(s, [t])], "last") for t in toks[cut:]]
        eng.close(s)
        check(torch.cat(rows), folder, toks, dtype, f"last 32 of {len(toks)} one by one")
    assert eng.graph_replays > 0


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_unequal_batches_through_a_cache_that_holds_one(folder, models, dtype):
    """A batch of 3 and a batch of 11 (whose decode steps run on the products for 9 to 64 rows), prompts in
    one step, then one token each; shorter requests end earlier; the second batch takes the first one's
    slots and pages."""
    batches = [([40, 7, 101], [9, 4, 12]), ([33, 1, 64, 65, 12, 90, 5, 17, 128, 47, 70], [6, 11, 3, 10, 12, 2, 9, 7, 5, 12, 8])]
    eng = make_engine(models, dtype, max_tokens=11 * 192, max_batch=11)
    for round_, (lens, extra) in enumerate(batches):
        full = prompts(V, [n + d for n, d in zip(lens, extra)], seed=30 + round_)
        slots = [eng.open() for _ in full]
        got = [[] for _ in full]
        lg = eng.step([(s, t[:n]) for s, t, n in zip(slots, full, lens)], "all")
        off = 0
        for i, n in enumerate(lens):
            got[i].append(lg[off:off + n])
            off += n
        pos = list(lens)
        live = list(range(len(full)))
        while live:
            lg = eng.step([(slots[i], [full[i][pos[i]]]) for i in live], "last")
            for j, i in enumerate(live):
                got[i].append(lg[j:j + 1])
                pos[i] += 1
            for i in [i for i in live if pos[i] == len(full[i])]:
                eng.close(slots[i])
            live = [i for i in live if pos[i] < len(full[i])]
        for i in range(len(full)):
            check(torch.cat(got[i]), folder, full[i], dtype, f"batch {round_} request {i}")
        eng.cache.check()
        assert eng.cache.slots.held_count == 0
    assert eng.graph_replays > 0


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_tokens_and_tiles_agree(folder, models, dtype):
    """Prompts of 63, 64 and 65 tokens fed in tiles of 1, 2, 8 and 64: the same logits, keys, values and
    convolution state, then three greedy tokens, as the reference asks of its token and tile paths on a
    real model (crates/mivi-model/src/model.rs:2110-2182)."""
    from mivi_v4_b200 import SamplingParams
    cfg, weights = plain_view64(folder)
    eng = make_engine(models, dtype)
    for toks in prompts(V, [63, 64, 65], seed=5):
        for tile in (1, 2, 8, 64):
            s = eng.open()
            rows = [eng.step([(s, toks[lo:lo + tile])], "all") for lo in range(0, len(toks), tile)]
            check_cache(eng, s, folder, toks, dtype, f"{len(toks)} tokens in tiles of {tile}")
            eng.close(s)
            check(torch.cat(rows), folder, toks, dtype, f"{len(toks)} tokens in tiles of {tile}")
        out = eng.generate([toks], 3, SamplingParams.greedy(), stop_token_ids=[])[0]
        if dtype == torch.float32:
            assert out == P.plain_generate(cfg, weights, toks, 3)
        else:
            logits = plain_logits(folder, toks + out)
            noise = plain_noise(folder, toks + out, dtype)
            for i, tok in enumerate(out):
                row = logits[len(toks) + i - 1]
                assert row[tok] >= row.max() - 32 * noise, (i, tok, int(row.argmax()))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("B", [100, 200])
def test_decode_batches_beyond_a_token_tile(folder, models, dtype, B):
    """100 and 200 sequences at these widths: a prefill step of several hundred tokens (its products cut along K
    on the kernel with swapped operands, the norms carried from it into the prefill kernels) and decode steps of
    more rows than the 64 of the weight-streaming kernels and the 128 of a token tile.  Every seventeenth
    sequence is held against the plain implementation."""
    lens = [2 + (5 * i) % 9 for i in range(B)]
    seqs = prompts(V, [n + 3 for n in lens], seed=41)
    eng = make_engine(models, dtype, max_tokens=64 * B, max_batch=B)
    slots = [eng.open() for _ in range(B)]
    first = eng.step([(s, t[:n]) for s, t, n in zip(slots, seqs, lens)], "last")
    got = [first] + [eng.step([(s, [t[n + k]]) for s, t, n in zip(slots, seqs, lens)], "last") for k in range(3)]
    eng.check_errors()
    for b in range(0, B, 17):
        rows = torch.stack([g[b] for g in got])
        check(rows, folder, seqs[b], dtype, f"sequence {b} of {B}", rows=list(range(lens[b] - 1, lens[b] + 3)))
    for s in slots:
        eng.close(s)
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_decoding_from_500_to_1100_cached_tokens(folder, models, dtype):
    """Decode steps replayed from recorded launches while the cache grows past 512 tokens (the page table
    of the recording widens: another recording) and past 1,024 (the tcgen05 decode attention starts to
    split the keys and adds its merge kernel to the recording).  A second, short sequence rides along and
    ends early.  Every step's logits against the plain implementation."""
    from mivi_v4_b200.ops import kernels as K
    a, b = prompts(V, [1100, 140], seed=8)
    eng = make_engine(models, dtype, max_tokens=1152 + 192)
    sa, sb = eng.open(), eng.open()
    eng.step([(sa, a[:500]), (sb, b[:40])], None)
    rows_a, rows_b = [], []
    for i in range(600):
        items = [(sa, [a[500 + i]])] + ([(sb, [b[40 + i]])] if i < 100 else [])
        lg = eng.step(items, "last")
        rows_a.append(lg[0:1])
        if i < 100:
            rows_b.append(lg[1:2])
        if i == 99:
            eng.close(sb)
    eng.close(sa)
    check(torch.cat(rows_a), folder, a, dtype, "decoding 500..1100", rows=slice(500, 1100))
    check(torch.cat(rows_b), folder, b, dtype, "the short companion", rows=slice(40, 140))
    # two sequences under a page table of 512 and of 1,024 tokens, then one under 1,024 and 2,048
    assert eng.graphs_recorded >= 4 and any(key[1][0][1] == 32 for key in eng.graph_keys()), eng.graph_keys()
    assert eng.graph_replays >= 590
    if dtype == torch.bfloat16:
        assert K.attention_decode_tc_plan(1, WIDE["num_key_value_heads"], 1152) > 1
    eng.cache.check()


def test_a_fault_would_show_at_these_sizes(folder):
    toks = prompts(V, [1, 65, 130, 200], seed=3)[1]
    want = plain_logits(folder, toks)
    for dtype in DTYPES:
        noise = plain_noise(folder, toks, dtype)
        for i, kind in enumerate(WIDE["layer_types"]):
            pre = f"model.layers.{i}."
            n = pre + ("conv.out_proj.weight" if kind == "conv" else "self_attn.out_proj.weight")
            assert would_fail(mutated_logits(folder, toks, n), want, dtype, noise), (dtype, n)
