"""Measurements of a model on the device: decode steps, a prefill, generation end
to end, the stages of a step, and single kernels, each timed with CUDA events on the
launching stream after warm-up.  ``bench.py`` and the command line's ``bench`` verb
print what these functions return.

The reference's ``bench`` command times an isolated prefill and generation without its
first token on a synthetic prompt, and prints the stages of its forward pass beside the
totals (crates/mivi-cli/src/runners/bench.rs:65-148, 178-238).
"""
from __future__ import annotations

import math
import statistics
import time
from typing import Dict, List, Optional, Sequence

import torch

from .cache import KVNeed
from .ops import kernels as K


def model_numbers(model) -> dict:
    """Bytes and floating-point operations of the model's steps, from the model itself: the bytes
    of all its tensors (a decode step reads each once), the cache bytes a token and a sequence
    hold, the matrix-product operations a token costs in the layers and a row of logits in the
    head, and the attention operations of a prompt of T tokens."""
    elt = 2 if model.dtype == torch.bfloat16 else 4
    plan = model.cache_plan()
    kv_per_token = sum(g.n_layers * 2 * g.need.n_kv_heads * g.need.head_dim * elt
                       for g in plan.groups if isinstance(g.need, KVNeed))
    state_per_seq = sum(g.n_layers * torch.empty(0, dtype=g.need.dtype).element_size() * math.prod(g.need.shape)
                        for g in plan.groups if not isinstance(g.need, KVNeed))

    def matrices(part) -> int:
        n = sum(math.prod(spec.shape) for spec in part.param_specs().values() if spec.role == "matrix")
        return n + sum(matrices(sub) for sub in part.nested().values())
    per_token = sum(matrices(model.blocks[e.block]) for e in model.schedule)
    attn = [(b.mixer.nh, b.mixer.hd) for b in (model.blocks[e.block] for e in model.schedule)
            if hasattr(getattr(b, "mixer", None), "nh")]
    return dict(weight_bytes=model.weight_bytes(), kv_bytes_per_token=kv_per_token, state_bytes_per_seq=state_per_seq,
                gemm_flops_per_token=2 * per_token, head_flops_per_row=2 * model.vocab_size * model.hidden_size,
                attn_flops=lambda T: sum(4 * nh * hd * T * (T + 1) // 2 for nh, hd in attn))


def random_prompts(vocab: int, lengths: Sequence[int], seed: int) -> List[List[int]]:
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (int(n),), generator=g).tolist() for n in lengths]


def _engine(model, prompt_lens, new_tokens, **kw):
    from .engine import Engine
    room = sum(-(-(n + new_tokens) // 64) * 64 for n in prompt_lens)
    return Engine(model, max_tokens=room, max_batch=len(prompt_lens), **kw)


def decode_run(model, prompt_lens: Sequence[int], steps: int, warmup: int, seed: int = 0,
               room_each: Optional[int] = None) -> dict:
    """Device time of exactly ``steps`` decode steps of sequences that hold prompts of ``prompt_lens``
    tokens, greedy sampling on the device included, host token ids in.  Also times the unequal prefill
    step that fills the cache.  ``room_each``: cache room per sequence (default: what the run needs)."""
    from .engine import Engine
    B = len(prompt_lens)
    V = model.vocab_size
    total = warmup + steps
    if room_each is not None:
        eng = Engine(model, max_tokens=B * room_each, max_batch=B)
    else:
        eng = _engine(model, prompt_lens, total + 1)
    prompts = random_prompts(V, prompt_lens, seed)
    g = torch.Generator().manual_seed(seed + 1)
    feed = torch.randint(0, V, (total, B), generator=g).tolist()
    # the prefill once untimed (first launches, buffers), then timed on fresh slots
    slots = [eng.open() for _ in range(B)]
    eng.step(list(zip(slots, prompts)), None)
    for s in slots:
        eng.close(s)
    slots = [eng.open() for _ in range(B)]
    torch.cuda.synchronize()
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record()
    eng.step(list(zip(slots, prompts)), None)
    p1.record()
    work = torch.empty((B, K.sample_scratch_width(V)), dtype=torch.float32, device=model.device)
    out = torch.empty((B,), dtype=torch.int32, device=model.device)

    def one(i):
        logits = eng.step([(s, [feed[i][b]]) for b, s in enumerate(slots)], "last", copy=False)
        K.sample(logits, work, out, temperature=0.0)

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    launches0 = K.launch_count()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for i in range(warmup, total):
        one(i)
    t1.record()
    torch.cuda.synchronize()
    eng.check_errors()
    ms = t0.elapsed_time(t1) / steps
    cached_mean = sum(prompt_lens) / B + warmup + (steps - 1) / 2.0       # tokens a sequence holds, mean over the steps
    res = dict(ms_per_step=ms, launches=K.launch_count() - launches0, cached_tokens_mean=cached_mean,
               prefill_ms=p0.elapsed_time(p1), replays=eng.graph_replays, cache_bytes=eng.cache.bytes())
    for s in slots:
        eng.close(s)
    del eng
    torch.cuda.empty_cache()
    return res


def prefill_run(model, tokens: int, reps: int, warmup: int, seed: int = 2) -> float:
    """Median device time (ms) of one prompt of ``tokens`` tokens in one step, last logits wanted."""
    from .engine import Engine
    eng = Engine(model, max_tokens=2 * tokens + 128, max_batch=2, max_step_tokens=tokens)
    g = torch.Generator().manual_seed(seed)
    times = []
    for i in range(warmup + reps):
        toks = torch.randint(0, model.vocab_size, (tokens,), generator=g).tolist()
        s = eng.open()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        eng.step([(s, toks)], "last", copy=False)
        t1.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(t0.elapsed_time(t1))
        eng.close(s)
    eng.check_errors()
    del eng
    torch.cuda.empty_cache()
    return statistics.median(times)


def generate_run(model, prompt_lens: Sequence[int], new_tokens: int, warmup_tokens: int = 4, seed: int = 1) -> dict:
    """Through the public entry point: host token lists in, host token lists out, one host-to-device copy
    of the step's inputs and one device-to-host read of the sampled tokens every step.  Decoding is timed
    by the host's clock from the first emitted token to the return, as the reference times generation
    without its first token; the prefill from the call to the first token."""
    from .sampling import SamplingParams
    eng = _engine(model, prompt_lens, max(new_tokens, warmup_tokens) + 1)
    prompts = random_prompts(model.vocab_size, prompt_lens, seed)
    # the same lengths as the timed run: its decode steps then find their shapes recorded
    eng.generate(prompts, warmup_tokens, SamplingParams.greedy(), stop_token_ids=[])
    first: Dict[str, float] = {}
    h2d0 = [0]

    def on_token(i, tok):
        if "t" not in first:
            first["t"] = time.perf_counter()
            h2d0[0] = eng.h2d_bytes
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    t0 = time.perf_counter()
    out = eng.generate(prompts, new_tokens, SamplingParams.greedy(), stop_token_ids=[], on_token=on_token)
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    if not all(len(o) == new_tokens for o in out):
        raise RuntimeError("generation ended early")
    B = len(prompt_lens)
    steps = new_tokens - 1
    res = dict(decode_tokens_per_s=B * steps / (t1 - first["t"]), prefill_tokens_per_s=sum(prompt_lens) / (first["t"] - t0),
               # the step's integer arrays, and the sampled tokens' way to the next step
               h2d_bytes_per_step=(eng.h2d_bytes - h2d0[0]) / max(steps, 1), d2h_bytes_per_step=B * 4,
               peak_memory_bytes=torch.cuda.max_memory_allocated(), cache_bytes=eng.cache.bytes())
    del eng
    torch.cuda.empty_cache()
    return res


def stage_report(model, prompt_lens: Sequence[int], steps: int = 8, prefill: bool = False, seed: int = 3) -> dict:
    """Where the time of decode steps (or of the prefill step) goes: an engine with ``profile=True`` runs
    them launch by launch with every launch timed; see ``KernelProfile.report``."""
    from .engine import Engine
    B = len(prompt_lens)
    room = sum(-(-(n + steps + 8) // 64) * 64 for n in prompt_lens)
    eng = Engine(model, max_tokens=room, max_batch=B, profile=True, max_step_tokens=max(8192, max(prompt_lens)))
    prompts = random_prompts(model.vocab_size, prompt_lens, seed)
    slots = [eng.open() for _ in range(B)]
    eng.step(list(zip(slots, prompts)), "last", copy=False)           # compiles nothing new later
    if prefill:
        for s in slots:
            eng.close(s)
        slots = [eng.open() for _ in range(B)]
        eng.profile_report()
        eng.step(list(zip(slots, prompts)), "last", copy=False)
        return eng.profile_report()
    for i in range(3):
        eng.step([(s, [i + 1]) for s in slots], "last", copy=False)
    eng.profile_report()
    for i in range(steps):
        eng.step([(s, [i + 5]) for s in slots], "last", copy=False)
    return eng.profile_report()


def replayed_kernels(model, prompt_lens: Sequence[int], prefill: bool = False, seed: int = 3) -> dict:
    """Kernel by kernel, how long one decode step took while it was REPLAYED from its recording (or, with
    ``prefill``, the prefill step as the engine launches it): from the CUDA activity records of the step
    (torch.profiler), so the kernels overlap as they do in service and none is serialised by a profiler.
    {"span_us", "kernels", "rows": [{kernel, calls, us, share}]}."""
    from torch.profiler import ProfilerActivity, profile

    from .engine import Engine
    B = len(prompt_lens)
    room = sum(-(-(n + 24) // 64) * 64 for n in prompt_lens)
    eng = Engine(model, max_tokens=2 * room, max_batch=B, max_step_tokens=max(8192, max(prompt_lens)))
    prompts = random_prompts(model.vocab_size, prompt_lens, seed)
    slots = [eng.open() for _ in range(B)]
    eng.step(list(zip(slots, prompts)), "last", copy=False)
    n_steps = 1 if prefill else 3
    if prefill:
        for s in slots:
            eng.close(s)
        slots = [eng.open() for _ in range(B)]
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            eng.step(list(zip(slots, prompts)), "last", copy=False)
            torch.cuda.synchronize()
    else:
        for i in range(6):
            eng.step([(s, [i + 3]) for s in slots], "last", copy=False)
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for i in range(n_steps):
                eng.step([(s, [i + 30]) for s in slots], "last", copy=False)
            torch.cuda.synchronize()
    ev = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA
          and "memcpy" not in e.name.lower() and "memset" not in e.name.lower()]
    ev.sort(key=lambda e: e.time_range.start)
    n = len(ev) // n_steps
    last = ev[-n:]
    agg: Dict[str, list] = {}
    for e in last:
        name = e.name.replace("(anonymous namespace)::", "").replace("void ", "").split("(")[0]
        t = agg.setdefault(name, [0.0, 0])
        t[0] += e.time_range.end - e.time_range.start
        t[1] += 1
    span = last[-1].time_range.end - last[0].time_range.start
    rows = [dict(kernel=k, calls=c, us=t, share=t / span) for k, (t, c) in sorted(agg.items(), key=lambda kv: -kv[1][0])]
    return dict(span_us=span, kernels=n, rows=rows)


def print_replayed_kernels(rep: dict, title: str, file=None) -> None:
    print(f"{title}: {rep['kernels']} kernels, {rep['span_us']:.0f} us from the first one's start to the last one's end",
          file=file)
    for r in rep["rows"]:
        print(f"  {r['us']:8.1f} us  {100 * r['share']:5.1f} %  {r['calls']:3d} x {r['us'] / r['calls']:6.1f} us  {r['kernel']}",
              file=file)


def print_stage_report(rep: dict, title: str, peaks: Optional[dict] = None, file=None) -> None:
    steps = max(rep["steps"], 1)
    print(f"{title}: {rep['total_us'] / steps:.0f} us a step over {steps} step(s), launch by launch", file=file)
    print("  by stage:", file=file)
    for stage, us in sorted(rep["stages"].items(), key=lambda kv: -kv[1]):
        print(f"    {us / steps:9.1f} us  {100 * us / rep['total_us']:5.1f} %  {stage}", file=file)
    print("  by stage and kernel:", file=file)
    for r in rep["rows"]:
        rate = []
        if r["gb_per_s"]:
            rate.append(f"{r['gb_per_s']:7.0f} GB/s" + (f" ({r['gb_per_s'] / peaks['hbm_gbs']:.2f})" if peaks else ""))
        if r["tflops"] and r["tflops"] > 1.0:
            rate.append(f"{r['tflops']:7.1f} TFLOP/s" + (f" ({r['tflops'] / peaks['bf16_tflops']:.2f})" if peaks else ""))
        print(f"    {r['us'] / steps:9.1f} us  {100 * r['share']:5.1f} %  {r['calls'] // steps:3d} x {r['us'] / r['calls']:7.1f} us  "
              f"{r['stage']:22s} {r['kernel']:28s} {'  '.join(rate)}", file=file)


# ---- single kernels -----------------------------------------------------------------------------
def _replayed_us(calls, reps: int) -> float:
    """Mean device time (us) of the launches in ``calls``, recorded once into a CUDA graph and replayed
    (the host's launch cost is not in the number)."""
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for fn in calls:
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
    return t0.elapsed_time(t1) * 1e3 / (reps * len(calls))


def kernel_run(kernel: str, *, m: int = 8, n: int = 16384, k: int = 2048, swiglu: bool = False, accumulate: bool = False,
               batch: int = 8, context: int = 520, tokens: int = 2048, heads: int = 32, kv_heads: int = 8,
               head_dim: int = 64, vocab: int = 65536, reps: int = 20, mark: bool = True,
               pair: Optional[bool] = None) -> dict:
    """One kernel alone at given sizes.  Weights are rotated through enough copies that every launch
    reads them from HBM, not from L2.  After the timing, one more plain launch runs between
    cudaProfilerStart and cudaProfilerStop (``mark``), for a profiler that captures from there."""
    from .engine.step import Workspace
    dev = "cuda:0"
    torch.manual_seed(0)
    res: dict = dict(kernel=kernel)
    if kernel == "reference_matmul":
        # not a kernel of this library: torch.matmul (cuBLAS) on the same operands in the same harness, as the
        # yardstick for the products above; it is on no path of the library
        copies = max(2, min(64, (1 << 30) // (n * k * 2)))
        ws = [(torch.randn(n, k, device=dev) * 0.05).to(torch.bfloat16) for _ in range(copies)]
        x = torch.randn(m, k, device=dev).to(torch.bfloat16)
        out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        torch.matmul(x, ws[0].T, out=out)
        us = _replayed_us([lambda w=w: torch.matmul(x, w.T, out=out) for w in ws], reps)
        res.update(m=m, n=n, k=k, us=us, weights_gb_per_s=n * k * 2 / us / 1e3, tflops=2.0 * m * n * k / us / 1e6)
        return res
    if kernel.startswith("gemm"):
        fn = getattr(K, kernel)
        copies = max(2, min(64, (1 << 30) // (n * k * 2)))           # about 1 GB of weights in rotation
        ws = [(torch.randn(n, k, device=dev) * 0.05).to(torch.bfloat16) for _ in range(copies)]
        x = torch.randn(m, k, device=dev).to(torch.bfloat16)
        if swiglu:
            out, kw = torch.empty(m, n // 2, dtype=torch.bfloat16, device=dev), dict(swiglu=True)
        elif accumulate:
            out, kw = torch.zeros(m, n, device=dev), dict(accumulate=True)
        else:
            out, kw = torch.empty(m, n, device=dev), {}
        if kernel == "gemm_tc":
            kw["pair"] = pair
        fn(x, ws[0], out, **kw)                                        # first call: attributes, tensor maps
        us = _replayed_us([lambda w=w: fn(x, w, out, **kw) for w in ws], reps)
        res.update(m=m, n=n, k=k, us=us, weights_gb_per_s=n * k * 2 / us / 1e3, tflops=2.0 * m * n * k / us / 1e6)
        run = lambda: fn(x, ws[1], out, **kw)                          # noqa: E731
    elif kernel == "sample":
        logits = torch.randn(batch, vocab, device=dev) * 2
        work = torch.empty(batch, K.sample_scratch_width(vocab), device=dev)
        out = torch.empty(batch, dtype=torch.int32, device=dev)
        ring = torch.randint(0, vocab, (batch, K.RECENT_RING), dtype=torch.int32, device=dev)
        rows = torch.arange(batch, dtype=torch.int32, device=dev)
        steps = torch.full((batch,), 100, dtype=torch.int32, device=dev)
        modes = {"greedy": dict(temperature=0.0), "temperature": dict(temperature=0.7),
                 "temperature, top_p": dict(temperature=0.7, top_p=0.9),
                 "temperature, top_k": dict(temperature=0.2, top_k=40),
                 "temperature, top_k, top_p": dict(temperature=0.2, top_k=40, top_p=0.9),
                 "the reference's defaults (and a repetition penalty over the ring)":
                     dict(temperature=0.2, top_k=40, top_p=0.9, repetition_penalty=1.05, ring=ring, ring_rows=rows),
                 "temperature, top_k 2000, top_p (one block a row)": dict(temperature=0.7, top_k=2000, top_p=0.9)}
        res.update(batch=batch, vocab=vocab, modes={})
        for name, kw in modes.items():
            run = lambda kw=kw: K.sample(logits, work, out, seed=1, streams=rows, steps=steps, **kw)   # noqa: E731
            run()
            res["modes"][name] = _replayed_us([run] * 10, reps)
    else:
        nh, nkv, hd, page = heads, kv_heads, head_dim, 64
        scale = 1.0 / math.sqrt(hd)

        def cache(lengths):
            blocks = [-(-x // page) for x in lengths]
            pool = (torch.randn(sum(blocks) + 1, 2, nkv, page, hd, device=dev)).to(torch.bfloat16)
            table = torch.zeros(len(lengths), max(blocks), dtype=torch.int32)
            nxt = 1
            for b, nb in enumerate(blocks):
                table[b, :nb] = torch.arange(nxt, nxt + nb, dtype=torch.int32)
                nxt += nb
            return pool, table.to(dev)

        def ints(v):
            return torch.tensor(v, dtype=torch.int32, device=dev)
        if kernel in ("attention_decode", "attention_decode_tc"):
            lengths = [context + i for i in range(batch)]
            pool, table = cache(lengths)
            q = torch.randn(batch, nh * hd, device=dev).to(torch.bfloat16)
            out = torch.empty_like(q)
            ws = Workspace(dev)
            seq_of, positions = ints(list(range(batch))), ints([x - 1 for x in lengths])
            if kernel == "attention_decode_tc":
                run = lambda: K.attention_decode_tc(q, pool, table, positions, seq_of, out, nh, nkv, hd, scale, ws)  # noqa: E731
            else:
                run = lambda: K.attention_decode(q, pool, table, positions, seq_of, out, nh, nkv, hd, scale, 0, ws)  # noqa: E731
            run()
            us = _replayed_us([run], reps)
            res.update(batch=batch, context=context, us=us, cache_gb_per_s=sum(lengths) * nkv * hd * 2 * 2 / us / 1e3)
        elif kernel in ("attention_prefill", "attention_prefill_tc"):
            pool, table = cache([tokens])
            q = torch.randn(tokens, nh * hd, device=dev).to(torch.bfloat16)
            out = torch.empty_like(q)
            cu, starts = ints([0, tokens]), ints([0])
            if kernel == "attention_prefill_tc":
                run = lambda: K.attention_prefill_tc(q, pool, table, cu, starts, out, 1, nh, nkv, hd, scale)      # noqa: E731
            else:
                run = lambda: K.attention_prefill(q, pool, table, cu, starts, out, 1, nh, nkv, hd, scale, 0)      # noqa: E731
            run()
            us = _replayed_us([run], reps)
            res.update(tokens=tokens, us=us, tflops=4.0 * nh * hd * tokens * (tokens + 1) / 2 / us / 1e6)
        else:
            raise ValueError(f"unknown kernel {kernel!r}")
    K.check_device_errors()
    if mark:
        torch.cuda.profiler.start()
        run()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    return res


KERNELS = ("gemm_small_m", "gemm_tc_swap", "gemm_tc", "attention_decode", "attention_decode_tc", "attention_prefill",
           "attention_prefill_tc", "sample", "reference_matmul")
