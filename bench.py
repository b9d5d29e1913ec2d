#!/usr/bin/env python3
"""Decode and prefill throughput of the LFM2.5-1.2B-shaped model with random
weights on one B200, in the manner of the reference's ``bench`` command
(crates/mivi-cli/src/runners/bench.rs:65-148: a synthetic prompt, an isolated
prefill, then generation timed without its first token).

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers 16]
    python bench.py --workload unequal32 | long32k      (the two further workloads, one JSON line each)

One "step" is one decode step of the whole batch.  Prints ONE JSON line:
``value`` is decoded tokens per second timed on the device over exactly K
steps; ``e2e`` is the same through ``Engine.generate`` with host token lists in
and out; ``prefill`` is one 2,048-token prompt; ``roofline`` compares the bytes
a decode step must read (every weight once, the cache of the live sequences)
with the measured copy bandwidth; ``points`` holds decode at batch 1 and 64.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# layer sizes of the benchmark configuration (LFM2.5-1.2B shape)
BENCH_CONFIG = dict(
    architectures=["Lfm2ForCausalLM"], model_type="lfm2", hidden_size=2048, num_hidden_layers=16,
    num_attention_heads=32, num_key_value_heads=8, vocab_size=65536, block_ff_dim=12288,
    block_auto_adjust_ff_dim=True, block_multiple_of=256, block_ffn_dim_multiplier=1.0,
    layer_types=["conv", "conv", "full_attention", "conv", "conv", "full_attention", "conv", "conv",
                 "full_attention", "conv", "full_attention", "conv", "full_attention", "conv",
                 "full_attention", "conv"],
    rope_theta=1000000.0, norm_eps=1e-5, conv_L_cache=3, conv_bias=False, tie_embedding=True)
FULL_LAYERS = 16
CONTEXT = 4096
PROMPT = 512
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            out = dict(FALLBACK_PEAKS)

            def walk(node):
                for k, v in node.items():
                    if isinstance(v, dict):
                        walk(v)
                    elif k in out and isinstance(v, (int, float)) and v > 0:
                        out[k] = float(v)
            walk(d)
            return out, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class NvmlSampler(threading.Thread):
    """Reads the SM clock and the clock event reasons of the benchmark's GPU through NVML every 20 ms
    (reading only; nothing is set).  Any failure ends the thread quietly: nvidia-smi's samples remain."""
    REASONS = ((0x8, "hw_slowdown"), (0x40, "hw_thermal_slowdown"), (0x20, "sw_thermal_slowdown"), (0x4, "sw_power_cap"))

    def __init__(self, period: float = 0.02):
        super().__init__(daemon=True)
        self.period, self.stop_flag = period, threading.Event()
        self.sm, self.max_sm, self.reasons = [], None, set()
        self.uuid = None
        try:                                  # asked here, in the caller's thread: the sampling thread calls NVML only
            import torch
            self.uuid = "GPU-" + str(torch.cuda.get_device_properties(0).uuid)
        except Exception:  # noqa: BLE001
            pass

    def run(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            handle = None
            for form in ((self.uuid, self.uuid.encode()) if self.uuid else ()):
                try:                                      # the binding's versions differ in which form they take
                    handle = pynvml.nvmlDeviceGetHandleByUUID(form)
                    break
                except Exception:  # noqa: BLE001
                    continue
            if handle is None:
                handle = pynvml.nvmlDeviceGetHandleByIndex(0)
            self.max_sm = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            read_reasons = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
            while not self.stop_flag.is_set():
                self.sm.append(float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)))
                mask = int(read_reasons(handle))
                self.reasons.update(name for bit, name in self.REASONS if mask & bit)
                self.stop_flag.wait(self.period)
        except Exception:  # noqa: BLE001
            pass

    def stop(self):
        self.stop_flag.set()
        self.join(timeout=2)


class ClockSampler:
    """The GPU's clocks while the timed regions run: NVML in a thread of this process, and
    nvidia-smi in the background as the second source (it needs a second or two before its first line)."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __enter__(self):
        self.nvml = NvmlSampler()
        self.nvml.start()
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        self.nvml.stop()
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        self.file.flush()

    def summary(self):
        sm, mx, reasons = [], [], set()
        try:
            with open(self.file.name) as f:
                for line in f:
                    parts = [p.strip() for p in line.split(",")]
                    if len(parts) < 9:
                        continue
                    try:
                        sm.append(float(parts[1]))
                        mx.append(float(parts[2]))
                    except ValueError:
                        continue
                    for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                         parts[5:9]):
                        if val.lower().startswith("active"):
                            reasons.add(name)
            os.unlink(self.file.name)
        except OSError:
            pass
        source = "nvidia-smi"
        try:
            nvml_sm = [float(v) for v in list(self.nvml.sm)]
            if len(nvml_sm) > len(sm) and self.nvml.max_sm:
                # the denser record; what nvidia-smi saw of the reasons is kept too
                sm, mx, source = nvml_sm, [float(self.nvml.max_sm)], "nvml"
                reasons |= set(self.nvml.reasons)
        except Exception:  # noqa: BLE001
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": source}


def model_numbers(model, cfg):
    """Bytes and flops of the benchmark's steps, from the model itself."""
    c = model.config
    H, F, V, hd, nh, nkv = c.hidden_size, c.ff_dim, c.vocab_size, c.head_dim, c.num_attention_heads, c.num_key_value_heads
    n_attn, n_conv = len(c.attn_layer_ids), len(c.conv_layer_ids)
    per_tok_matrix = (n_conv * (3 * H * H + H * H) + n_attn * ((nh + 2 * nkv) * hd * H + nh * hd * H)
                      + c.num_hidden_layers * 3 * H * F)
    kv_bytes_per_token = n_attn * 2 * nkv * hd * 2
    return dict(weight_bytes=model.weight_bytes(), kv_bytes_per_token=kv_bytes_per_token,
                conv_state_bytes=n_conv * (c.conv_L_cache - 1) * H * 4,
                gemm_flops_per_token=2 * per_tok_matrix, head_flops_per_row=2 * V * H,
                attn_flops=lambda T: n_attn * 4 * nh * hd * T * (T + 1) // 2)


def time_decode(model, batch, steps, warmup, seed=0):
    """Device time of exactly ``steps`` decode steps of ``batch`` sequences that
    each hold a PROMPT-token prompt; greedy sampling on the device included."""
    import torch
    from mivi_v4_b200 import Engine
    from mivi_v4_b200.ops import kernels as K
    eng = Engine(model, max_tokens=batch * CONTEXT, max_batch=batch)
    g = torch.Generator().manual_seed(seed)
    V = model.vocab_size
    prompts = [torch.randint(0, V, (PROMPT,), generator=g).tolist() for _ in range(batch)]
    feed = torch.randint(0, V, (warmup + steps, batch), generator=g).tolist()
    slots = [eng.open() for _ in range(batch)]
    eng.step(list(zip(slots, prompts)), None)
    work = torch.empty((batch, V), dtype=torch.float32, device=model.device)
    out = torch.empty((batch,), dtype=torch.int32, device=model.device)

    def one(i):
        logits = eng.step([(s, [feed[i][b]]) for b, s in enumerate(slots)], "last", copy=False)
        K.sample(logits, work, out, temperature=0.0)

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    launches0 = K.launch_count()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for i in range(warmup, warmup + steps):
        one(i)
    t1.record()
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1) / steps
    launches = K.launch_count() - launches0
    ctx_mean = PROMPT + warmup + (steps - 1) / 2.0
    for s in slots:
        eng.close(s)
    del eng
    torch.cuda.empty_cache()
    return ms, launches, ctx_mean


def time_e2e(model, batch, steps, warmup, seed=1):
    """The same through the public entry point: host token lists in, host token
    lists out, one host->device copy of the step's inputs and one device->host
    read of the sampled tokens every step.  Timed from the first emitted token
    to the return, as the reference times decoding without its first token."""
    import torch
    from mivi_v4_b200 import Engine, SamplingParams
    eng = Engine(model, max_tokens=batch * CONTEXT, max_batch=batch)
    g = torch.Generator().manual_seed(seed)
    prompts = [torch.randint(0, model.vocab_size, (PROMPT,), generator=g).tolist() for _ in range(batch)]
    eng.generate(prompts, warmup + 1, SamplingParams.greedy(), stop_token_ids=[])
    first = {}
    h2d0 = None

    def on_token(i, tok):
        nonlocal h2d0
        if "t" not in first:
            first["t"] = time.perf_counter()
            h2d0 = eng.h2d_bytes
    torch.cuda.synchronize()
    out = eng.generate(prompts, steps + 1, SamplingParams.greedy(), stop_token_ids=[], on_token=on_token)
    torch.cuda.synchronize()
    dt = time.perf_counter() - first["t"]
    assert all(len(o) == steps + 1 for o in out)
    h2d = (eng.h2d_bytes - h2d0) / steps + 2 * batch * 4
    del eng
    torch.cuda.empty_cache()
    return batch * steps / dt, h2d, batch * 4


def time_prefill(model, reps, warmup, seed=2):
    import torch
    from mivi_v4_b200 import Engine
    eng = Engine(model, max_tokens=2 * PREFILL_TOKENS, max_batch=2, max_step_tokens=PREFILL_TOKENS)
    g = torch.Generator().manual_seed(seed)
    times = []
    for i in range(warmup + reps):
        toks = torch.randint(0, model.vocab_size, (PREFILL_TOKENS,), generator=g).tolist()
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
    del eng
    torch.cuda.empty_cache()
    return statistics.median(times)


def further_workload(which: str) -> int:
    """The two further workloads of the benchmark set, through ``Engine.generate``:
    ``unequal32``: LFM2-700M shape, 32 prompts of 64..2,048 tokens in one unequal prefill step, 256 new tokens;
    ``long32k``: LFM2-350M shape, 8 prompts of 32,768 tokens, 128 new tokens (keys and values only for the six
    attention layers, convolution state for the ten others).  Prefill is timed to the first token, decoding
    from the first token to the end."""
    import torch
    from mivi_v4_b200 import Engine, SamplingParams, random_model
    cfg = dict(BENCH_CONFIG)
    if which == "long32k":
        cfg.update(hidden_size=1024, num_attention_heads=16, num_key_value_heads=8, block_ff_dim=6656)
        lens, new = [32768] * 8, 128
    else:
        cfg.update(hidden_size=1536, num_attention_heads=24, num_key_value_heads=8, block_ff_dim=10240)
        g = torch.Generator().manual_seed(0)
        lens, new = torch.randint(64, 2049, (32,), generator=g).tolist(), 256
    model = random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0", on_device=True)
    eng = Engine(model, max_tokens=sum(-(-(n + new) // 64) * 64 for n in lens), max_batch=len(lens))
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, model.vocab_size, (n,), generator=g).tolist() for n in lens]
    eng.generate([p[:64] for p in prompts[:2]], 4, SamplingParams.greedy(), stop_token_ids=[])       # warm-up
    first = {}
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    out = eng.generate(prompts, new, SamplingParams.greedy(), stop_token_ids=[],
                       on_token=lambda i, t: first.setdefault("t", time.perf_counter()))
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    assert all(len(o) == new for o in out)
    c = model.config
    print(json.dumps({
        "workload": which, "impl": "ours", "dtype": "bf16", "data": "synthetic (uniform random token ids, random weights)",
        "prompt_tokens": sum(lens), "prefill_tokens_per_s": sum(lens) / (first["t"] - t0),
        "decode_tokens_per_s": len(lens) * (new - 1) / (t1 - first["t"]), "new_tokens_each": new,
        "peak_memory_gib": torch.cuda.max_memory_allocated() / 2 ** 30, "cache_gib": eng.cache.bytes() / 2 ** 30,
        "config": {"hidden": c.hidden_size, "heads": c.num_attention_heads, "kv_heads": c.num_key_value_heads,
                   "ff": c.ff_dim, "layers": c.num_hidden_layers, "vocab": c.vocab_size, "batch": len(lens),
                   "longest_prompt": max(lens), "shortest_prompt": min(lens)}}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=FULL_LAYERS,
                    help="run the first LAYERS layers of the 16 (sizes unchanged); both numbers go into config")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 and 64 and the end-to-end run")
    ap.add_argument("--workload", default=None, choices=["unequal32", "long32k"],
                    help="run one of the two further workloads instead of the default benchmark")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust workspace (no setup.py/pyproject.toml: pip reports 'not "
                          "installable'), and this image has no cargo/rustc and no network"}))
        return 0
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        print(json.dumps({"error": "this library runs on one GPU; bench.py measures --gpus 1 only",
                          "n_gpus": args.gpus}))
        return 2
    warmup = max(3, args.warmup)
    if args.workload:
        return further_workload(args.workload)

    import torch
    from mivi_v4_b200 import random_model
    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device"}))
        return 1
    cfg = dict(BENCH_CONFIG)
    if args.layers != FULL_LAYERS:
        cfg["layer_types"] = cfg["layer_types"][:args.layers]
        cfg["num_hidden_layers"] = args.layers
    model = random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0", on_device=True)
    nums = model_numbers(model, cfg)
    pk, pk_src = peaks()

    # the clocks are sampled over all the timed regions of this run (the K decode steps alone are
    # shorter than one sampling period)
    with ClockSampler() as clk:
        ms, launches, ctx_mean = time_decode(model, args.batch, args.steps, warmup)
        value = args.batch * 1000.0 / ms
        step_bytes = nums["weight_bytes"] + args.batch * (ctx_mean * nums["kv_bytes_per_token"] + nums["conv_state_bytes"])
        achieved = step_bytes / (ms * 1e-3) / 1e9

        pre_ms = time_prefill(model, reps=5, warmup=3)
        pre_flops = (PREFILL_TOKENS * nums["gemm_flops_per_token"] + nums["head_flops_per_row"]
                     + nums["attn_flops"](PREFILL_TOKENS))
        prefill = {"value": PREFILL_TOKENS / (pre_ms * 1e-3), "tokens": PREFILL_TOKENS, "ms": pre_ms,
                   "frac": pre_flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12)}

        points, e2e = {}, None
        if not args.no_points:
            for b in (1, 64):
                pms, _, _ = time_decode(model, b, max(8, args.steps // 2), warmup)
                points[f"decode_b{b}"] = b * 1000.0 / pms
            e, h2d, d2h = time_e2e(model, args.batch, args.steps, warmup)
            e2e = {"value": e, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}
    clocks = clk.summary()

    c = model.config
    line = {
        "metric": "decode tokens/s, LFM2.5-1.2B shape, bf16, random weights", "value": value, "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic (uniform random token ids, random weights)",
        "impl": "ours",
        "config": {
            "model": "LFM2.5-1.2B shape", "layers": args.layers, "layers_full": FULL_LAYERS,
            "attention_layers": len(c.attn_layer_ids), "hidden": c.hidden_size, "heads": c.num_attention_heads,
            "kv_heads": c.num_key_value_heads, "head_dim": c.head_dim, "ff": c.ff_dim, "vocab": c.vocab_size,
            "conv_width": c.conv_L_cache, "tied": c.tie_embedding, "global_batch": args.batch,
            "seq_len": CONTEXT, "prompt_len": PROMPT, "parallelism": "single GPU",
            "l2": "inputs larger than L2 (a step reads %.2f GB of weights)" % (nums["weight_bytes"] / 1e9),
            "peaks": pk_src,
        },
        "clocks": clocks,
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"]},
        "points": points,
    }
    if e2e is not None:
        line["e2e"] = e2e
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
