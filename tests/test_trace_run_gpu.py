"""bin/trace_run as a user runs it: a subprocess fed steps on standard input.
The same requests are replayed whole, with the last 32 tokens one by one, and
in batches of unequal lengths whose shorter requests end earlier, one batch
after another through a cache that only just holds one batch; in 32-bit and in
bfloat16; all against the plain implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import assert_close, plain_logits, plain_noise, write_model
from tiny_configs import CONFIGS, LOUD_CONFIGS, prompts

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def replay(folder, dtype, steps, out_dir, max_tokens):
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out",
         str(out_dir), "--max-tokens", str(max_tokens)],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    return proc


def read(out_dir, step, vocab):
    return torch.from_numpy(np.fromfile(os.path.join(str(out_dir), f"{step}.f32"), dtype="<f4").reshape(-1, vocab).copy())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "BL"])
def test_replay_three_ways(name, dtype, tmp_path):
    cfg, seed = CONFIGS[name] if name in CONFIGS else LOUD_CONFIGS[name]
    V = cfg["vocab_size"]
    folder = write_model(tmp_path, cfg, seed, init="loud" if name in LOUD_CONFIGS else "baseline")
    reqs = {f"r{i}": p for i, p in enumerate(prompts(V, [40, 75, 33, 100, 64, 36], seed=7))}
    want = {k: plain_logits(folder, v) for k, v in reqs.items()}
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    # single rows and rows of several requests are compared: the largest of the requests' rounding noises
    noise = max(plain_noise(folder, v, tdt) for v in reqs.values())

    # 1. whole: each request alone, logits everywhere
    steps = [{"step": i, "entries": [{"id": k, "tokens": v, "want": list(range(len(v)))}], "end": [k]}
             for i, (k, v) in enumerate(reqs.items())]
    out = tmp_path / f"whole_{dtype}"
    replay(folder, dtype, steps, out, 128)
    for i, k in enumerate(reqs):
        assert_close(read(out, i, V), want[k], tdt, f"whole {k}", noise=noise)

    # 2. the last 32 tokens one by one
    steps, expect, n = [], [], 0
    for k, v in reqs.items():
        cut = len(v) - 32
        steps.append({"step": n, "entries": [{"id": k, "tokens": v[:cut], "want": [cut - 1]}], "end": []})
        expect.append((n, want[k][cut - 1:cut]))
        n += 1
        for j in range(cut, len(v)):
            steps.append({"step": n, "entries": [{"id": k, "tokens": [v[j]], "want": [0]}],
                          "end": [k] if j == len(v) - 1 else []})
            expect.append((n, want[k][j:j + 1]))
            n += 1
    out = tmp_path / f"last32_{dtype}"
    replay(folder, dtype, steps, out, 128)
    for s, w in expect:
        assert_close(read(out, s, V), w, tdt, f"last32 step {s}", noise=noise)

    # 3. batches of three with unequal lengths: prompts (all but the last 8 tokens, at least one) in one
    #    step, then one token each; shorter requests end earlier; the cache holds one batch only
    steps, expect, n = [], [], 0
    keys = list(reqs)
    for batch in (keys[:3], keys[3:]):
        cut = {k: max(1, len(reqs[k]) - 8 - 3 * i) for i, k in enumerate(batch)}
        steps.append({"step": n, "entries": [{"id": k, "tokens": reqs[k][:cut[k]], "want": [0, cut[k] - 1]}
                                             for k in batch], "end": []})
        expect.append((n, torch.cat([want[k][[0, cut[k] - 1]] for k in batch])))
        n += 1
        pos = dict(cut)
        live = list(batch)
        while live:
            ends = [k for k in live if pos[k] == len(reqs[k]) - 1]
            steps.append({"step": n, "entries": [{"id": k, "tokens": [reqs[k][pos[k]]], "want": [0]} for k in live],
                          "end": ends})
            expect.append((n, torch.cat([want[k][pos[k]:pos[k] + 1] for k in live])))
            n += 1
            for k in live:
                pos[k] += 1
            live = [k for k in live if k not in ends]
    out = tmp_path / f"batched_{dtype}"
    need = max(sum(-(-len(reqs[k]) // 64) * 64 for k in b) for b in (keys[:3], keys[3:]))
    replay(folder, dtype, steps, out, need)
    for s, w in expect:
        assert_close(read(out, s, V), w, tdt, f"batched step {s}", noise=noise)


def test_replay_with_nothing_wanted_and_empty_lines(tmp_path):
    cfg, seed = CONFIGS["A"]
    folder = write_model(tmp_path, cfg, seed)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": [1, 2, 3], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [4], "want": [0]}], "end": ["a"]}]
    out = tmp_path / "o"
    replay(folder, "float32", steps, out, 64)
    assert not os.path.exists(out / "0.f32")
    assert_close(read(out, 1, cfg["vocab_size"]), plain_logits(folder, [1, 2, 3, 4])[3:], torch.float32, "after silent step")
