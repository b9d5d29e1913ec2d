"""The engine against the plain implementation on a GPU, in 32-bit and in
bfloat16: each request alone and whole; with the last tokens one by one; in
batches of unequal lengths whose shorter requests end earlier, one batch after
another so that slots are used again."""
import pytest
import torch

from helpers import assert_close, check_cache, plain_logits, plain_noise
from tiny_configs import CONFIGS, LOUD_CONFIGS, all_folders, config_of, prompts

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]
NAMES = list(CONFIGS) + list(LOUD_CONFIGS)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return all_folders(tmp_path_factory.mktemp("models"))


def check(got, folder, toks, dtype, what):
    assert_close(got, plain_logits(folder, toks), dtype, what, noise=plain_noise(folder, toks, dtype))


def make_engine(folder, dtype, max_tokens=4096, **kw):
    from mivi_v4_b200 import Engine, load_model
    return Engine(load_model(folder, dtype, "cuda:0"), max_tokens=max_tokens, **kw)


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompt(folders, name, dtype):
    eng = make_engine(folders[name], dtype)
    V = config_of(name)["vocab_size"]
    for toks in prompts(V, [1, 2, 5, 33, 64, 65, 130], seed=3):
        s = eng.open()
        got = eng.step([(s, toks)], "all")
        eng.close(s)
        check(got, folders[name], toks, dtype, f"{name} whole len {len(toks)}")
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", NAMES)
def test_last_tokens_one_by_one(folders, name, dtype):
    eng = make_engine(folders[name], dtype)
    V = config_of(name)["vocab_size"]
    for toks in prompts(V, [33, 70, 100], seed=4):
        s = eng.open()
        cut = max(1, len(toks) - 32)
        rows = [eng.step([(s, toks[:cut])], "all")]
        for t in toks[cut:]:
            rows.append(eng.step([(s, [t])], "last"))
        eng.close(s)
        check(torch.cat(rows), folders[name], toks, dtype, f"{name} last32 len {len(toks)}")


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_slots_reused(folders, name, dtype):
    """Two batches one after another through a cache that is just large
    enough for one: prompts in one step, then one token each; shorter requests
    end earlier."""
    V = config_of(name)["vocab_size"]
    eng = make_engine(folders[name], dtype, max_tokens=4 * 128, max_batch=4)
    for round_, lens in enumerate([[5, 11, 17, 40], [1, 7, 19, 32]]):
        full = prompts(V, [n + d for n, d in zip(lens, [3, 9, 6, 12])], seed=10 + round_)
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
            check(torch.cat(got[i]), folders[name], full[i], dtype, f"{name} batch {round_} request {i}")
        eng.cache.check()
        assert eng.cache.slots.held_count == 0


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["A", "B", "D", "AL", "BL"])
def test_cache_contents_do_not_depend_on_the_cut(folders, name, dtype):
    """Not only the logits: the keys, values and convolution state that a sequence leaves in the cache are
    the plain implementation's whether it came whole, token by token or in uneven pieces (the reference checks the same for
    its token and tile paths: crates/mivi-model/src/ssm.rs:455-541, transformer.rs:612-753)."""
    eng = make_engine(folders[name], dtype, page_size=16)
    V = config_of(name)["vocab_size"]
    toks = prompts(V, [53], seed=12)[0]
    for cuts in ([53], [1] * 53, [7, 30, 1, 15], [16, 16, 21]):
        s = eng.open()
        done = 0
        for n in cuts:
            eng.step([(s, toks[done:done + n])], None)
            done += n
        check_cache(eng, s, folders[name], toks, dtype, f"{name} in pieces of {cuts[:4]}")
        eng.close(s)


@pytest.mark.parametrize("name", ["F", "FL"])
@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_long_prompts_in_chunks(folders, name, dtype):
    """Prompts of hundreds of tokens with heads of 64 (in bfloat16 the tcgen05 attention
    kernel runs them): two unequal prompts in one step, and one prompt in two chunks, the
    second of which starts in the middle of a page."""
    eng = make_engine(folders[name], dtype, max_tokens=4096)
    V = config_of(name)["vocab_size"]
    a, b = prompts(V, [700, 300], seed=11)
    sa, sb = eng.open(), eng.open()
    got = eng.step([(sa, a), (sb, b)], "all")
    eng.close(sa), eng.close(sb)
    check(got[:700], folders[name], a, dtype, "two prompts, the longer")
    check(got[700:], folders[name], b, dtype, "two prompts, the shorter")
    s = eng.open()
    first = eng.step([(s, a[:230])], "all")
    second = eng.step([(s, a[230:])], "all")
    eng.close(s)
    check(torch.cat([first, second]), folders[name], a, dtype, "one prompt in chunks of 230 and 470")
    # chunks of 100 tokens: steps of few tokens with many tokens of one sequence each (in bfloat16 the
    # tcgen05 decode attention, a block a token), two sequences side by side
    sa, sb = eng.open(), eng.open()
    rows_a, rows_b = [], []
    for lo in range(0, 700, 50):
        items = [(sa, a[lo:lo + 50])] + ([(sb, b[lo:lo + 50])] if lo < 300 else [])
        got = eng.step(items, "all")
        rows_a.append(got[:50])
        if lo < 300:
            rows_b.append(got[50:])
    eng.close(sa), eng.close(sb)
    check(torch.cat(rows_a), folders[name], a, dtype, "chunks of 50, the longer")
    check(torch.cat(rows_b), folders[name], b, dtype, "chunks of 50, the shorter")
    eng.cache.check()

