"""Ways of running the engine that the other files do not take: a step that mixes a prompt's chunk with
single tokens, a bfloat16 run over a checkpoint that stores some matrices in 32-bit, decoding under
replayed recordings across the page table's growth, and sampled generation in bfloat16 and with
penalties, against the plain implementation."""
import pytest
import torch

import plain_lfm2 as P
from helpers import assert_close, plain_logits, plain_noise, plain_view, write_model
from tiny_configs import TINY_B, TINY_F, all_folders, config_of, prompts

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]
IDS = ["f32", "bf16"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return all_folders(tmp_path_factory.mktemp("models"))


def engine(folder, dtype, **kw):
    from mivi_v4_b200 import Engine, load_model
    kw.setdefault("max_tokens", 4096)
    return Engine(load_model(folder, dtype, "cuda:0"), **kw)


def check(got, folder, toks, dtype, what, rows=None):
    want = plain_logits(folder, toks)
    assert_close(got, want if rows is None else want[rows], dtype, what, noise=plain_noise(folder, toks, dtype))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", ["AL", "BL", "C", "FL"])
def test_a_step_that_mixes_a_prompt_chunk_with_single_tokens(folders, name, dtype):
    """Two sequences are decoding; a third joins the same steps with its prompt in chunks of 30 and 1
    and 22 tokens.  (The generation loop never builds such a step, the step function allows it.)"""
    Vn = config_of(name)["vocab_size"]
    a, b, c = prompts(Vn, [20, 35, 53], seed=14)
    eng = engine(folders[name], dtype)
    sa, sb, sc = eng.open(), eng.open(), eng.open()
    got = {0: [], 1: [], 2: []}
    lg = eng.step([(sa, a[:10]), (sb, b[:31])], "all")
    got[0].append(lg[:10]), got[1].append(lg[10:])
    lg = eng.step([(sa, [a[10]]), (sc, c[:30]), (sb, [b[31]])], "all")
    got[0].append(lg[:1]), got[2].append(lg[1:31]), got[1].append(lg[31:])
    lg = eng.step([(sc, [c[30]]), (sa, [a[11]]), (sb, [b[32]])], "last")
    got[2].append(lg[0:1]), got[0].append(lg[1:2]), got[1].append(lg[2:3])
    lg = eng.step([(sa, [a[12]]), (sb, [b[33]]), (sc, c[31:])], [[0], [0], list(range(22))])
    got[0].append(lg[:1]), got[1].append(lg[1:2]), got[2].append(lg[2:])
    check(torch.cat(got[0]), folders[name], a[:13], dtype, f"{name}: first decoding sequence")
    check(torch.cat(got[1]), folders[name], b[:34], dtype, f"{name}: second decoding sequence")
    check(torch.cat(got[2]), folders[name], c, dtype, f"{name}: the sequence that joined in chunks")
    for s in (sa, sb, sc):
        eng.close(s)
    eng.cache.check()


@pytest.mark.parametrize("name,cfg,seed", [("B", TINY_B, 1), ("F", TINY_F, 5)])
def test_bfloat16_run_with_some_matrices_stored_in_32_bit(tmp_path, name, cfg, seed):
    """A checkpoint may keep single matrices in float32; they stay so, and their products run in true
    32-bit on bfloat16 activations widened for them.  Here: a feed-forward's w2, a convolution's in_proj,
    an attention's k_proj (the fused q/k/v matrix is then 32-bit as a whole) and the embedding table."""
    kinds = cfg["layer_types"]
    conv, attn = kinds.index("conv"), kinds.index("full_attention")
    over = {f"model.layers.{conv}.feed_forward.w2.weight": "float32",
            f"model.layers.{conv}.conv.in_proj.weight": "float32",
            f"model.layers.{attn}.self_attn.k_proj.weight": "float32",
            "model.embed_tokens.weight": "float32"}
    folder = write_model(tmp_path, cfg, seed, init="loud", store_overrides=over, tag="_mixed")
    eng = engine(folder, torch.bfloat16)
    assert eng.model.embedding.weight.dtype == torch.float32
    toks = prompts(cfg["vocab_size"], [70], seed=15)[0]
    s = eng.open()
    rows = [eng.step([(s, toks[:38])], "all")] + [eng.step([(s, [t])], "last") for t in toks[38:]]
    eng.close(s)
    check(torch.cat(rows), folder, toks, torch.bfloat16, f"{name} with mixed storage")


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_decoding_across_the_page_table_growth(folders, dtype):
    """Heads of 64 (in bfloat16: the tcgen05 decode attention): one token at a time from 500 to 1,100
    cached tokens under replayed recordings, three recordings of different page-table widths."""
    name = "FL"
    Vn = config_of(name)["vocab_size"]
    a, b = prompts(Vn, [1100, 600], seed=16)
    eng = engine(folders[name], dtype, max_tokens=1152 + 640)
    sa, sb = eng.open(), eng.open()
    eng.step([(sa, a[:500]), (sb, b[:3])], None)
    rows_a, rows_b = [], []
    for i in range(600):
        items = [(sa, [a[500 + i]])] + ([(sb, [b[3 + i]])] if 3 + i < len(b) else [])
        lg = eng.step(items, "last")
        rows_a.append(lg[0:1])
        if len(items) == 2:
            rows_b.append(lg[1:2])
    check(torch.cat(rows_a), folders[name], a, dtype, "decoding 500..1100", rows=slice(500, 1100))
    check(torch.cat(rows_b), folders[name], b, dtype, "its companion 3..600", rows=slice(3, 600))
    assert eng.graphs_recorded >= 3 and any(key[1][0][1] == 32 for key in eng.graph_keys()), eng.graph_keys()
    assert eng.graph_replays >= 590


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sp", ["greedy", "temperature", "penalties"])
def test_early_enqueue_changes_nothing_in_either_dtype(folders, sp, dtype):
    """With recorded decode steps the loop enqueues the next step before it has read this step's tokens;
    without, it runs step by step.  Same tokens, stops and unequal lengths included, more requests than
    slots so that slots are used again inside one call."""
    from mivi_v4_b200 import SamplingParams
    name = "BL"
    cfg, weights = plain_view(folders[name])
    ps = prompts(cfg["vocab_size"], [3, 20, 9, 41, 1, 6, 14], seed=9)
    params = {"greedy": SamplingParams.greedy(), "temperature": SamplingParams.plain_temperature(0.9, seed=5),
              "penalties": SamplingParams(temperature=0.7, top_k=20, top_p=0.95, repetition_penalty=1.2,
                                          presence_penalty=0.1, frequency_penalty=0.05, seed=5)}[sp]
    new = [12, 3, 1, 9, 2, 70, 5]
    kw = dict(max_tokens=3 * 128, max_batch=3)
    base = engine(folders[name], dtype, cuda_graphs=False, **kw).generate(ps, new, params, stop_token_ids=[])
    stop = base[0][5]
    want = engine(folders[name], dtype, cuda_graphs=False, **kw).generate(ps, new, params, stop_token_ids=[stop])
    eng = engine(folders[name], dtype, **kw)
    got = eng.generate(ps, new, params, stop_token_ids=[stop])
    assert got == want
    assert eng.graph_replays > 0
    eng.cache.check()
    assert eng.cache.slots.held_count == 0
    if dtype == "float32":
        # the plain loop with the plain sampler: penalties over the last 64 generated tokens, the draw of
        # (seed, request, step), stops
        skw = {k: v for k, v in vars(params).items() if k != "seed"}
        plain = [P.plain_generate(cfg, weights, p, n, stop_ids=[stop], seed=params.seed or 0, stream=i, **skw)
                 for i, (p, n) in enumerate(zip(ps, new))]
        assert got == plain


def test_temperature_generation_bfloat16_draws_from_the_plain_distribution(folders):
    """Every token that a bfloat16 run samples lies in the support that the plain implementation's
    logits give at that place (top-k 8 here), or within rounding of its edge."""
    from mivi_v4_b200 import SamplingParams
    name = "BL"
    cfg, weights = plain_view(folders[name])
    ps = prompts(cfg["vocab_size"], [5, 11, 17, 2], seed=17)
    sp = SamplingParams(temperature=1.0, top_k=8, seed=3)
    got = engine(folders[name], "bfloat16").generate(ps, 24, sp, stop_token_ids=[])
    for p, out in zip(ps, got):
        assert len(out) == 24
        logits = plain_logits(folders[name], p + out)
        noise = plain_noise(folders[name], p + out, torch.bfloat16)
        for i, tok in enumerate(out):
            row = logits[len(p) + i - 1]
            kth = torch.topk(row, 8).values[-1]
            assert row[tok] >= kth - 32 * noise, (i, tok)
    assert len({t for out in got for t in out}) > 8          # not one token over and over


def test_many_decode_shapes_share_one_workspace(folders):
    """Sequences that end one by one and grow past page-table widths make many decode shapes.  Their
    recordings work in one workspace and one graph memory pool: the device memory that the engine holds
    does not grow with their number, the least recently used are dropped beyond ``max_graphs``, and the
    logits stay those of the plain implementation throughout."""
    name = "FL"
    Vn = config_of(name)["vocab_size"]
    n = 12
    full = prompts(Vn, [530 + 9 * i for i in range(n)], seed=18)
    eng = engine(folders[name], torch.bfloat16, max_tokens=n * 640, max_batch=n, max_graphs=6)
    slots = [eng.open() for _ in full]
    start = 500
    eng.step([(s, t[:start]) for s, t in zip(slots, full)], None)
    got = [[] for _ in full]
    live = list(range(n))
    pos = start
    mem = []
    while live:
        lg = eng.step([(slots[i], [full[i][pos]]) for i in live], "last")
        for j, i in enumerate(live):
            got[i].append(lg[j:j + 1].cpu())
        pos += 1
        for i in [i for i in live if pos == len(full[i])]:
            eng.close(slots[i])
        live = [i for i in live if pos < len(full[i])]
        mem.append(torch.cuda.memory_allocated())
        assert len(eng.graph_keys()) <= 6
    for i in range(n):
        check(torch.cat(got[i]), folders[name], full[i], torch.bfloat16, f"request {i}", rows=slice(start, len(full[i])))
    assert eng.graphs_recorded >= n + 1                      # every batch size, and the wider page table
    # after the first step (which sized the workspace) nothing more is held, whatever the number of shapes
    assert max(mem) - mem[0] <= (1 << 20), (mem[0], max(mem))
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name,B", [("AL", 150), ("BL", 200), ("FL", 70)])
def test_decoding_more_sequences_than_a_token_tile(folders, name, B, dtype):
    """Batches of 70 to 200 sequences: their prompts in one step of several hundred tokens, then one token
    each for four steps (more rows than the 64 of the weight-streaming kernels and the 128 of a token
    tile; the attention of a decode step stays with the kernel that takes every query token on its own)."""
    Vn = config_of(name)["vocab_size"]
    lens = [3 + (7 * i) % 11 for i in range(B)]
    seqs = prompts(Vn, [n + 4 for n in lens], seed=31)
    eng = engine(folders[name], dtype, max_tokens=64 * B, max_batch=B)
    slots = [eng.open() for _ in range(B)]
    eng.step([(s, t[:n]) for s, t, n in zip(slots, seqs, lens)], None)
    got = []
    for k in range(4):
        got.append(eng.step([(s, [t[n + k]]) for s, t, n in zip(slots, seqs, lens)], "last"))
    eng.check_errors()
    for b in range(0, B, 13):                  # every thirteenth sequence against the plain implementation
        rows = torch.stack([g[b] for g in got])
        check(rows, folders[name], seqs[b], dtype, f"{name}: sequence {b} of {B}",
              rows=list(range(lens[b], lens[b] + 4)))
    for s in slots:
        eng.close(s)
    eng.cache.check()
