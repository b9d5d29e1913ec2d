"""Generation through the Python entry point against the plain implementation."""
import pytest
import torch

import plain_lfm2 as P
from helpers import assert_close, plain_logits, plain_noise, plain_view
from tiny_configs import all_folders, prompts

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return all_folders(tmp_path_factory.mktemp("models"))


def engine(folder, dtype, **kw):
    from mivi_v4_b200 import Engine, load_model
    kw.setdefault("max_tokens", 4096)
    return Engine(load_model(folder, dtype, "cuda:0"), **kw)


@pytest.mark.parametrize("name,lens,new", [("A", [5, 11, 17], 8), ("B", [1, 7, 19, 32], 12), ("C", [3, 64, 65], 6)])
def test_greedy_generation_float32(folders, name, lens, new):
    from mivi_v4_b200 import SamplingParams
    cfg, weights = plain_view(folders[name])
    ps = prompts(cfg["vocab_size"], lens, seed=1)
    got = engine(folders[name], "float32").generate(ps, new, SamplingParams.greedy(), stop_token_ids=[])
    want = [P.plain_generate(cfg, weights, p, new) for p in ps]
    assert got == want


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_bfloat16_follows_the_plain_logits(folders, name):
    """bfloat16 may pick another token where two logits nearly tie; every token it picks must be
    (nearly) the best one under the plain implementation, given the tokens before it."""
    from mivi_v4_b200 import SamplingParams
    cfg, weights = plain_view(folders[name])
    ps = prompts(cfg["vocab_size"], [5, 11, 17], seed=2)
    got = engine(folders[name], "bfloat16").generate(ps, 8, SamplingParams.greedy(), stop_token_ids=[])
    for p, out in zip(ps, got):
        assert len(out) == 8
        logits = P.plain_forward(cfg, weights, p + out)
        for i, tok in enumerate(out):
            row = logits[len(p) + i - 1]
            assert row[tok] >= row.max() - 0.05 * max(1.0, row.abs().max().item()), (i, tok, int(row.argmax()))


def test_temperature_generation_float32(folders):
    from mivi_v4_b200 import SamplingParams
    cfg, weights = plain_view(folders["B"])
    ps = prompts(cfg["vocab_size"], [1, 7, 19, 32], seed=3)
    sp = SamplingParams.plain_temperature(0.8, seed=11)
    got = engine(folders["B"], "float32").generate(ps, 12, sp, stop_token_ids=[])
    want = [P.plain_generate(cfg, weights, p, 12, seed=11, stream=i, temperature=0.8) for i, p in enumerate(ps)]
    assert got == want
    # each request alone draws the same tokens as in the batch when it keeps its stream
    eng = engine(folders["B"], "float32")
    again = eng.generate(ps, 12, sp, stop_token_ids=[])
    assert again == got


def test_stop_tokens_and_more_requests_than_slots(folders):
    from mivi_v4_b200 import SamplingParams
    cfg, weights = plain_view(folders["A"])
    ps = prompts(cfg["vocab_size"], [4, 9, 2, 30, 7, 12, 1], seed=4)
    free_run = [P.plain_generate(cfg, weights, p, 10) for p in ps]
    stop = free_run[1][3]                                 # a token that request 1 emits as its 4th
    want = [P.plain_generate(cfg, weights, p, 10, stop_ids=[stop]) for p in ps]
    assert len(want[1]) <= 3
    eng = engine(folders["A"], "float32", max_tokens=3 * 64, max_batch=3)     # three slots, one page each
    reqs = eng.generate(ps, 10, SamplingParams.greedy(), stop_token_ids=[stop], return_requests=True)
    assert [r.output for r in reqs] == want
    assert [r.finish_reason for r in reqs] == ["stop" if len(w) < 10 else "length" for w in want]
    eng.cache.check()
    assert eng.cache.slots.held_count == 0 and eng.cache.pages[eng.cache.kv_groups[0]].held_count == 0


@pytest.mark.parametrize("name", ["A", "AL"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(folders, name, dtype):
    """300 tokens decoded one by one after a short prompt, across several pages."""
    cfg, weights = plain_view(folders[name])
    toks = prompts(cfg["vocab_size"], [310], seed=5)[0]
    eng = engine(folders[name], dtype)
    s = eng.open()
    rows = [eng.step([(s, toks[:10])], "all")]
    for t in toks[10:]:
        rows.append(eng.step([(s, [t])], "last"))
    got = torch.cat(rows)
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    assert_close(got, plain_logits(folders[name], toks), td, "long decoding", noise=plain_noise(folders[name], toks, td))
    assert eng.graph_replays > 250                         # the decode steps did replay a captured graph


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "AL", "BL"])
def test_first_tokens_one_by_one(folders, name, dtype):
    """The first tokens of a sequence, fed singly from an empty cache (the convolution's zero
    left context, the first key of attention)."""
    cfg, _ = plain_view(folders[name])
    toks = prompts(cfg["vocab_size"], [6], seed=6)[0]
    eng = engine(folders[name], dtype)
    s = eng.open()
    got = torch.cat([eng.step([(s, [t])], "last") for t in toks])
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    assert_close(got, plain_logits(folders[name], toks), td, f"{name} first tokens",
                 noise=plain_noise(folders[name], toks, td))


def test_step_errors(folders):
    from mivi_v4_b200 import StepError
    eng = engine(folders["A"], "float32", max_tokens=128, max_batch=2)
    s = eng.open()
    with pytest.raises(StepError, match="vocabulary"):
        eng.step([(s, [1, 999])])
    with pytest.raises(StepError, match="not assigned"):
        eng.step([(s + 1, [1])])
    with pytest.raises(StepError, match="twice"):
        eng.step([(s, [1]), (s, [2])])
    with pytest.raises(StepError, match="wanted place"):
        eng.step([(s, [1, 2])], [[2]])
    with pytest.raises(StepError, match="full"):
        eng.step([(s, list(range(200)))])
    with pytest.raises(StepError, match="known are"):
        eng.step([(s, [1])], "first")
    with pytest.raises(StepError, match="integer places"):
        eng.step([(s, [1])], [["x"]])
    with pytest.raises(StepError, match="integer token ids"):
        eng.step([(s, ["a"])])
    with pytest.raises(StepError, match="vocabulary"):
        eng.step([(s, [-1])], "last")                       # a decode-shaped step takes another path in
    assert eng.length(s) == 0                              # a refused step leaves the sequence alone
    eng.step([(s, [1, 2, 3])], None)
    assert eng.length(s) == 3


def test_big_step_is_cut_invisibly(folders):
    cfg, _ = plain_view(folders["B"])
    ps = prompts(cfg["vocab_size"], [70, 3, 45], seed=8)
    eng = engine(folders["B"], "float32", max_step_tokens=32)
    slots = [eng.open() for _ in ps]
    got = eng.step(list(zip(slots, ps)), [[0, 69], [2], [44, 10]])
    want = torch.cat([plain_logits(folders["B"], ps[0])[[0, 69]], plain_logits(folders["B"], ps[1])[[2]],
                      plain_logits(folders["B"], ps[2])[[44, 10]]])
    assert_close(got, want, torch.float32, "cut step")


def test_command_line_generate(folders, capsys):
    from mivi_v4_b200.cli import main
    cfg, weights = plain_view(folders["A"])
    rc = main(["generate", "-m", folders["A"], "--prompt-ids", "5,6,7", "--prompt-ids", "9", "-n", "5", "-t", "0",
               "-r", "1.0", "--dtype", "float32", "--stop-ids", ""])
    assert rc == 0
    lines = [l for l in capsys.readouterr().out.strip().splitlines()]
    assert [[int(t) for t in l.split()] for l in lines] == [P.plain_generate(cfg, weights, p, 5) for p in ([5, 6, 7], [9])]


@pytest.mark.parametrize("sp", ["greedy", "temperature", "penalties"])
def test_early_enqueue_changes_nothing(folders, sp):
    """The loop enqueues the next step before it has read the current step's tokens (when no penalty
    needs them on the host).  The tokens must be those of the plain loop, stops and unequal lengths included."""
    from mivi_v4_b200 import SamplingParams
    cfg, weights = plain_view(folders["B"])
    ps = prompts(cfg["vocab_size"], [3, 20, 9, 41, 1], seed=9)
    params = {"greedy": SamplingParams.greedy(), "temperature": SamplingParams.plain_temperature(0.9, seed=5),
              "penalties": SamplingParams(temperature=0.7, top_k=20, top_p=0.95, repetition_penalty=1.2, seed=5)}[sp]
    new = [12, 3, 1, 9, 2]
    base = engine(folders["B"], "float32", cuda_graphs=False).generate(ps, new, params, stop_token_ids=[])
    stop = base[0][5]
    want = engine(folders["B"], "float32", cuda_graphs=False).generate(ps, new, params, stop_token_ids=[stop])
    eng = engine(folders["B"], "float32")
    got = eng.generate(ps, new, params, stop_token_ids=[stop])
    assert got == want
    assert eng.graph_replays > 0
    eng.cache.check()
    assert eng.cache.slots.held_count == 0
    if sp == "greedy":
        kw = {k: v for k, v in vars(params).items() if k != "seed"}
        assert want == [P.plain_generate(cfg, weights, p, n, stop_ids=[stop], **kw) for p, n in zip(ps, new)]


def test_a_kernel_fault_becomes_an_exception_and_leaves_the_cache_clean(folders):
    """Kernels that wait on barriers give up after a bounded time and set a flag on the device.  The flag
    travels to the host with every step; ``generate`` looks at it when it has a step's tokens, ``step``
    when it is called again, ``check_errors`` when asked.  The fault is made on the host here: the flag is
    written as a kernel would write it."""
    from mivi_v4_b200 import KernelError, SamplingParams
    from mivi_v4_b200.ops import kernels as K
    cfg, _ = plain_view(folders["F"])
    ps = prompts(cfg["vocab_size"], [5, 9, 3], seed=31)
    eng = engine(folders["F"], "bfloat16")
    assert len(eng.generate(ps, 4, SamplingParams.greedy(), stop_token_ids=[])[0]) == 4
    K._error_flag(eng.device).fill_(2)
    with pytest.raises(KernelError, match="MMA issuer"):
        eng.generate(ps, 6, SamplingParams.greedy(), stop_token_ids=[])
    eng.cache.check()
    assert eng.cache.slots.held_count == 0
    # the flag was cleared with the report: the engine works again
    assert len(eng.generate(ps, 4, SamplingParams.greedy(), stop_token_ids=[])[2]) == 4
    # the step function: the fault of one step is reported by check_errors once the host has waited,
    # or by the next step
    s = eng.open()
    K._error_flag(eng.device).fill_(3)
    lg = eng.step([(s, [1, 2, 3])], "last")
    lg.cpu()
    with pytest.raises(KernelError, match="epilogue"):
        eng.check_errors()
    eng.step([(s, [4])], "last").cpu()
    eng.check_errors()
    K._error_flag(eng.device).fill_(1)
    eng.step([(s, [5])], "last").cpu()
    with pytest.raises(KernelError, match="TMA producer"):
        eng.step([(s, [6])], "last")
    eng.close(s)
    eng.cache.check()
