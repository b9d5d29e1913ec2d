"""Run one kernel alone at given sizes, for timing and for profilers.

    python -m mivi_v4_b200.ops.probe gemm_small_m --m 8 --n 16384 --k 2048 [--swiglu]
    python -m mivi_v4_b200.ops.probe gemm_tc_swap --m 64 --n 6144 --k 2048
    python -m mivi_v4_b200.ops.probe gemm_tc --m 2048 --n 6144 --k 2048
    python -m mivi_v4_b200.ops.probe attention_decode --batch 8 --context 520
    python -m mivi_v4_b200.ops.probe attention_prefill --tokens 2048
    python -m mivi_v4_b200.ops.probe decode_step --batch 8 [--config config.json]

Weights are rotated through enough copies that every launch reads them from
HBM, not from L2.  Timing is by CUDA events around ``--reps`` launches that are
replayed from a CUDA graph (so the host's launch cost is not in the number);
the profiled region (cudaProfilerStart/Stop) is one more, plain launch.
``decode_step`` runs whole decode steps of a model with random weights (by
default the benchmark's configuration from bench.py) and prints, from the CUDA
activity records of one replayed step, how long each kind of kernel took.
"""
from __future__ import annotations

import argparse
import math

import torch

from . import kernels as K


def _timed(fn_list, reps):
    """Median-free simple timing: capture the launches in one graph, replay, divide."""
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for fn in fn_list:
            fn()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(reps):
        g.replay()
    t1.record()
    torch.cuda.synchronize()
    return t0.elapsed_time(t1) * 1e3 / (reps * len(fn_list))


def decode_step(a) -> int:
    import json
    import os
    import sys

    from torch.profiler import ProfilerActivity, profile

    from .. import Engine, random_model
    if a.config:
        with open(a.config) as f:
            cfg = json.load(f)
    else:
        sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
        import bench
        cfg = bench.BENCH_CONFIG
    B = a.batch
    model = random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0", on_device=True)
    eng = Engine(model, max_tokens=B * (a.prompt + 512), max_batch=B)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, model.vocab_size, (a.prompt,), generator=g).tolist() for _ in range(B)]
    slots = [eng.open() for _ in range(B)]
    eng.step(list(zip(slots, prompts)), None)
    for i in range(6):
        eng.step([(s, [i + 3]) for s in slots], "last", copy=False)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for i in range(3):
            eng.step([(s, [i + 30]) for s in slots], "last", copy=False)
        torch.cuda.synchronize()
    ev = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA
          and "memcpy" not in e.name.lower() and "memset" not in e.name.lower()]
    ev.sort(key=lambda e: e.time_range.start)
    n = len(ev) // 3
    last = ev[-n:]
    agg = {}
    for e in last:
        name = e.name.replace("(anonymous namespace)::", "").replace("void ", "").split("(")[0]
        t = agg.setdefault(name, [0.0, 0])
        t[0] += e.time_range.end - e.time_range.start
        t[1] += 1
    span = last[-1].time_range.end - last[0].time_range.start
    print(f"one decode step, batch {B}, {a.prompt + 8} cached tokens: {n} kernels, {span:.0f} us from first start to last end")
    for name, (t, c) in sorted(agg.items(), key=lambda kv: -kv[1][0]):
        print(f"  {t:8.1f} us  {100 * t / span:5.1f} %  {c:3d} x {t / c:6.1f} us  {name}")
    return 0


def _kernel_table(events, title):
    ev = [e for e in events if e.device_type == torch.autograd.DeviceType.CUDA
          and "memcpy" not in e.name.lower() and "memset" not in e.name.lower()]
    ev.sort(key=lambda e: e.time_range.start)
    agg = {}
    for e in ev:
        name = e.name.replace("(anonymous namespace)::", "").replace("void ", "").split("(")[0]
        t = agg.setdefault(name, [0.0, 0])
        t[0] += e.time_range.end - e.time_range.start
        t[1] += 1
    span = ev[-1].time_range.end - ev[0].time_range.start
    print(f"{title}: {len(ev)} kernels, {span:.0f} us from first start to last end")
    for name, (t, c) in sorted(agg.items(), key=lambda kv: -kv[1][0]):
        print(f"  {t:8.1f} us  {100 * t / span:5.1f} %  {c:3d} x {t / c:6.1f} us  {name}")


def prefill_step(a) -> int:
    import json
    import os
    import sys

    from torch.profiler import ProfilerActivity, profile

    from .. import Engine, random_model
    if a.config:
        with open(a.config) as f:
            cfg = json.load(f)
    else:
        sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
        import bench
        cfg = bench.BENCH_CONFIG
    T = a.tokens
    model = random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0", on_device=True)
    eng = Engine(model, max_tokens=2 * T + 128, max_batch=2, max_step_tokens=T)
    g = torch.Generator().manual_seed(0)
    for i in range(3):
        toks = torch.randint(0, model.vocab_size, (T,), generator=g).tolist()
        s = eng.open()
        if i == 2:
            torch.cuda.synchronize()
            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                eng.step([(s, toks)], "last", copy=False)
                torch.cuda.synchronize()
        else:
            eng.step([(s, toks)], "last", copy=False)
        eng.close(s)
    _kernel_table(prof.events(), f"prefill of one prompt of {T} tokens")
    return 0


def sample(a) -> int:
    """The sampling kernel alone on ``--batch`` rows of ``--vocab`` logits, by sampling mode; each mode is
    timed as ten launches replayed from a CUDA graph, as generation runs it."""
    dev = "cuda:0"
    B, V = a.batch, a.vocab
    logits = torch.randn(B, V, device=dev) * 2
    work = torch.empty(B, K.sample_scratch_width(V), device=dev)
    out = torch.empty(B, dtype=torch.int32, device=dev)
    ring = torch.randint(0, V, (B, K.RECENT_RING), dtype=torch.int32, device=dev)
    rows = torch.arange(B, dtype=torch.int32, device=dev)
    streams = torch.arange(B, dtype=torch.int32, device=dev)
    steps = torch.full((B,), 100, dtype=torch.int32, device=dev)
    modes = {"greedy": dict(temperature=0.0),
             "temperature": dict(temperature=0.7),
             "temperature, top_p": dict(temperature=0.7, top_p=0.9),
             "temperature, top_k": dict(temperature=0.2, top_k=40),
             "temperature, top_k, top_p": dict(temperature=0.2, top_k=40, top_p=0.9),
             "the reference's defaults (and a repetition penalty over the ring)":
                 dict(temperature=0.2, top_k=40, top_p=0.9, repetition_penalty=1.05, ring=ring, ring_rows=rows),
             "temperature, top_k 2000, top_p (one block a row)": dict(temperature=0.7, top_k=2000, top_p=0.9)}
    print(f"sampling, {B} rows of {V} logits")
    for name, kw in modes.items():
        run = lambda: K.sample(logits, work, out, seed=1, streams=streams, steps=steps, **kw)
        run()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(10):
                run()
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        print(f"  {e0.elapsed_time(e1) * 1000 / (10 * a.reps):7.1f} us  {name}")
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="mivi_v4_b200.ops.probe")
    ap.add_argument("kernel", choices=["gemm_small_m", "gemm_tc_swap", "gemm_tc", "attention_decode", "attention_prefill",
                                      "attention_prefill_tc", "attention_decode_tc", "sample",
                                       "decode_step", "prefill_step"])
    ap.add_argument("--vocab", type=int, default=65536)
    ap.add_argument("--config", default=None, help="config.json for decode_step (default: bench.py's)")
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--m", type=int, default=8)
    ap.add_argument("--n", type=int, default=16384)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--swiglu", action="store_true")
    ap.add_argument("--accumulate", action="store_true")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=520)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--reps", type=int, default=20)
    a = ap.parse_args(argv)
    dev = "cuda:0"
    torch.manual_seed(0)

    if a.kernel == "decode_step":
        return decode_step(a)
    if a.kernel == "prefill_step":
        return prefill_step(a)

    if a.kernel == "sample":
        return sample(a)

    if a.kernel.startswith("gemm"):
        fn = getattr(K, a.kernel)
        M, N, Kd = a.m, a.n, a.k
        copies = max(2, min(64, (1 << 30) // (N * Kd * 2)))           # about 1 GB of weights in rotation
        ws = [(torch.randn(N, Kd, device=dev) * 0.05).to(torch.bfloat16) for _ in range(copies)]
        x = torch.randn(M, Kd, device=dev).to(torch.bfloat16)
        if a.swiglu:
            out = torch.empty(M, N // 2, dtype=torch.bfloat16, device=dev)
            kw = dict(swiglu=True)
        elif a.accumulate:
            out = torch.zeros(M, N, device=dev)
            kw = dict(accumulate=True)
        else:
            out = torch.empty(M, N, device=dev)
            kw = {}
        fn(x, ws[0], out, **kw)                                        # first call: attributes, tensor maps
        us = _timed([lambda w=w: fn(x, w, out, **kw) for w in ws], a.reps)
        gbs = N * Kd * 2 / us / 1e3
        tfl = 2.0 * M * N * Kd / us / 1e6
        print(f"{a.kernel} M={M} N={N} K={Kd}: {us:.2f} us, weights at {gbs:.0f} GB/s, {tfl:.1f} TFLOP/s")
        torch.cuda.profiler.start()
        fn(x, ws[1], out, **kw)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        K.check_device_errors()
        return 0

    from ..engine.step import Workspace
    nh, nkv, hd, page = a.heads, a.kv_heads, a.head_dim, 64
    scale = 1.0 / math.sqrt(hd)

    def cache(lengths):
        blocks = [-(-n // page) for n in lengths]
        pool = (torch.randn(sum(blocks) + 1, 2, nkv, page, hd, device=dev)).to(torch.bfloat16)
        table = torch.zeros(len(lengths), max(blocks), dtype=torch.int32)
        nxt = 1
        for b, nb in enumerate(blocks):
            table[b, :nb] = torch.arange(nxt, nxt + nb, dtype=torch.int32)
            nxt += nb
        return pool, table.to(dev)

    def ints(v):
        return torch.tensor(v, dtype=torch.int32, device=dev)

    if a.kernel in ("attention_decode", "attention_decode_tc"):
        B = a.batch
        lengths = [a.context + i for i in range(B)]
        pool, table = cache(lengths)
        q = torch.randn(B, nh * hd, device=dev).to(torch.bfloat16)
        out = torch.empty_like(q)
        ws = Workspace(dev)
        seq_of, positions = ints(list(range(B))), ints([n - 1 for n in lengths])
        if a.kernel == "attention_decode_tc":
            run = lambda: K.attention_decode_tc(q, pool, table, positions, seq_of, out, nh, nkv, hd, scale, ws)
        else:
            run = lambda: K.attention_decode(q, pool, table, positions, seq_of, out, nh, nkv, hd, scale, 0, ws)
        run()
        us = _timed([run], a.reps)
        kv_bytes = sum(lengths) * nkv * hd * 2 * 2
        K.check_device_errors()
        print(f"{a.kernel} batch={B} context={a.context}: {us:.2f} us, cache at {kv_bytes / us / 1e3:.0f} GB/s")
    else:
        T = a.tokens
        pool, table = cache([T])
        q = torch.randn(T, nh * hd, device=dev).to(torch.bfloat16)
        out = torch.empty_like(q)
        cu, starts = ints([0, T]), ints([0])
        if a.kernel == "attention_prefill_tc":
            run = lambda: K.attention_prefill_tc(q, pool, table, cu, starts, out, 1, nh, nkv, hd, scale)
        else:
            run = lambda: K.attention_prefill(q, pool, table, cu, starts, out, 1, nh, nkv, hd, scale, 0)
        run()
        us = _timed([run], a.reps)
        K.check_device_errors()
        flops = 4.0 * nh * hd * T * (T + 1) / 2
        print(f"{a.kernel} tokens={T}: {us:.2f} us, {flops / us / 1e6:.1f} TFLOP/s")
    torch.cuda.profiler.start()
    run()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
