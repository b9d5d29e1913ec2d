#!/usr/bin/env python3
"""Decode and prefill throughput of the LFM2.5-1.2B-shaped model with random
weights on one B200, in the manner of the reference's ``bench`` command
(crates/mivi-cli/src/runners/bench.rs:65-148: a synthetic prompt, an isolated
prefill, then generation timed without its first token).

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers 16]
    python bench.py --workload unequal32 | long32k      (the two further workloads, the same line for each)
    python bench.py --stages decode|prefill [--batch B] (where a step's time goes, by stage and kernel)
    python bench.py --kernel NAME [--m .. --n .. --k ..] (one kernel alone, for timing and for profilers)

One "step" is one decode step of the whole batch.  Prints ONE JSON line:
``value`` is decoded tokens per second timed on the device over exactly K
steps; ``e2e`` is the same through ``Engine.generate`` with host token lists in
and out; ``prefill`` is one 2,048-token prompt (the workloads: their own unequal
prompts in one step); ``roofline`` compares the bytes a decode step must read
(every weight once, the cache of the live sequences) with the measured copy
bandwidth; ``points`` holds decode at batch 1, 64 and 256 with their own fractions, and the prefill of
512 tokens (tokens a second).
The timing itself is the library's (``mivi_v4_b200/measure.py``); this file adds
the benchmark's configurations, the clocks and the line.
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


WORKLOADS = {
    # LFM2-700M shape: 32 prompts of 64..2,048 tokens in one unequal prefill step, 256 decode steps
    "unequal32": dict(sizes=dict(hidden_size=1536, num_attention_heads=24, num_key_value_heads=8, block_ff_dim=10240),
                      model="LFM2-700M shape", new=256),
    # LFM2-350M shape: 8 prompts of 32,768 tokens, 128 decode steps (keys and values only for the six
    # attention layers, convolution state for the ten others)
    "long32k": dict(sizes=dict(hidden_size=1024, num_attention_heads=16, num_key_value_heads=8, block_ff_dim=6656),
                    model="LFM2-350M shape", new=128),
}


def workload_lengths(which: str):
    import torch
    if which == "long32k":
        return [32768] * 8
    g = torch.Generator().manual_seed(0)
    return torch.randint(64, 2049, (32,), generator=g).tolist()


def flat_config(model, name, layers, layers_full, batch, prompt_note, context, pk_src, weight_bytes):
    """Every size of the run, flat (at most 20 keys)."""
    c = model.config
    return {
        "model": name, "layers": layers, "layers_full": layers_full, "attention_layers": len(c.attn_layer_ids),
        "hidden": c.hidden_size, "heads": c.num_attention_heads, "kv_heads": c.num_key_value_heads,
        "head_dim": c.head_dim, "ff": c.ff_dim, "vocab": c.vocab_size, "conv_width": c.conv_L_cache,
        "tied": c.tie_embedding, "global_batch": batch, "seq_len": context, "prompt_len": prompt_note,
        "parallelism": "single GPU",
        "l2": "inputs larger than L2 (a step reads %.2f GB of weights)" % (weight_bytes / 1e9), "peaks": pk_src,
    }


def decode_point(nums, res, batch, pk):
    """tokens/s, bytes a step, GB/s and the fraction of the copy bandwidth of a timed decode run."""
    step_bytes = nums["weight_bytes"] + batch * (res["cached_tokens_mean"] * nums["kv_bytes_per_token"]
                                                 + nums["state_bytes_per_seq"])
    gbs = step_bytes / (res["ms_per_step"] * 1e-3) / 1e9
    return dict(value=batch * 1000.0 / res["ms_per_step"], ms_per_step=res["ms_per_step"], bytes_per_step=step_bytes,
                gb_per_s=gbs, frac=gbs / pk["hbm_gbs"])


def run_workload(which: str, steps_arg, warmup: int) -> int:
    """One of the two further workloads, reported like the default run: decode steps timed on the device
    (``value``, ``ms_per_step``, ``roofline``), the unequal prefill step of all prompts (``prefill``), the
    same through ``Engine.generate`` (``e2e``), the clocks, every size."""
    import torch
    from mivi_v4_b200 import measure, random_model
    w = WORKLOADS[which]
    cfg = dict(BENCH_CONFIG)
    cfg.update(w["sizes"])
    lens = workload_lengths(which)
    B, new = len(lens), w["new"]
    steps = new - warmup if steps_arg is None else steps_arg
    model = random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0", on_device=True)
    nums = measure.model_numbers(model)
    pk, pk_src = peaks()
    with ClockSampler() as clk:
        res = measure.decode_run(model, lens, steps, warmup)
        e = measure.generate_run(model, lens, new)
    clocks = clk.summary()
    point = decode_point(nums, res, B, pk)
    T = sum(lens)
    pre_flops = T * nums["gemm_flops_per_token"] + sum(nums["attn_flops"](n) for n in lens)    # no logits wanted
    pre_tflops = pre_flops / (res["prefill_ms"] * 1e-3) / 1e12
    print(json.dumps({
        "metric": f"decode tokens/s, {w['model']}, bf16, random weights ({which})", "workload": which,
        "value": point["value"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (uniform random token ids, random weights)", "impl": "ours",
        "config": flat_config(model, w["model"], FULL_LAYERS, FULL_LAYERS, B,
                              f"{min(lens)}..{max(lens)} (sum {T})", max(lens) + new, pk_src, nums["weight_bytes"]),
        "clocks": clocks, "gpu_launches": res["launches"],
        "prefill": {"value": T / (res["prefill_ms"] * 1e-3), "tokens": T, "ms": res["prefill_ms"], "tflops": pre_tflops,
                    "frac": pre_tflops / pk["bf16_tflops"], "frac_of_sustained": pre_tflops / pk["bf16_tflops_sustained"]},
        "roofline": {"bound": "hbm", "bytes_per_step": point["bytes_per_step"], "achieved": point["gb_per_s"],
                     "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": point["frac"]},
        "e2e": {"value": e["decode_tokens_per_s"], "unit": "tokens/s", "prefill_tokens_per_s": e["prefill_tokens_per_s"],
                "h2d_bytes_per_step": e["h2d_bytes_per_step"], "d2h_bytes_per_step": e["d2h_bytes_per_step"]},
        "peak_memory_gib": e["peak_memory_bytes"] / 2 ** 30, "cache_gib": e["cache_bytes"] / 2 ** 30}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None, help="timed decode steps (default 64; a workload: all of its own)")
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=FULL_LAYERS,
                    help="run the first LAYERS layers of the 16 (sizes unchanged); both numbers go into config")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip the further points and the end-to-end run")
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS),
                    help="run one of the two further workloads instead of the default benchmark")
    ap.add_argument("--stages", default=None, choices=["decode", "prefill"],
                    help="print where the time of a decode step (of --batch sequences) or of the prefill goes")
    ap.add_argument("--prompt-len", type=int, default=PROMPT,
                    help="with --stages decode: tokens that each sequence holds before the profiled steps")
    ap.add_argument("--replayed", action="store_true",
                    help="with --stages: the kernels of the step as replayed from its recording (activity records), "
                         "instead of launch by launch with stages")
    ap.add_argument("--kernel", default=None, help="time one kernel alone (see --m/--n/--k, --context, --tokens)")
    for name, default in (("m", 8), ("n", 16384), ("k", 2048), ("context", 520), ("tokens", PREFILL_TOKENS),
                          ("heads", 32), ("kv-heads", 8), ("head-dim", 64), ("vocab", 65536), ("reps", 20)):
        ap.add_argument("--" + name, type=int, default=default)
    ap.add_argument("--pair", default=None, choices=["0", "1"],
                    help="--kernel gemm_tc: 1 the kernel of two multiprocessors a tile, 0 the one-multiprocessor kernels")
    ap.add_argument("--swiglu", action="store_true")
    ap.add_argument("--accumulate", action="store_true")
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

    import torch
    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device"}))
        return 1
    from mivi_v4_b200 import measure, random_model
    if args.kernel:
        if args.kernel not in measure.KERNELS:
            print(json.dumps({"error": f"unknown kernel {args.kernel!r}", "known": list(measure.KERNELS)}))
            return 2
        print(json.dumps(measure.kernel_run(
            args.kernel, m=args.m, n=args.n, k=args.k, swiglu=args.swiglu, accumulate=args.accumulate, batch=args.batch,
            context=args.context, tokens=args.tokens, heads=args.heads, kv_heads=args.kv_heads, head_dim=args.head_dim,
            vocab=args.vocab, reps=args.reps, pair=None if args.pair is None else args.pair == "1")))
        return 0
    if args.workload:
        return run_workload(args.workload, args.steps, warmup)

    steps = 64 if args.steps is None else args.steps
    cfg = dict(BENCH_CONFIG)
    if args.layers != FULL_LAYERS:
        cfg["layer_types"] = cfg["layer_types"][:args.layers]
        cfg["num_hidden_layers"] = args.layers
    model = random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0", on_device=True)
    nums = measure.model_numbers(model)
    pk, pk_src = peaks()
    if args.stages:
        lens = [args.tokens] if args.stages == "prefill" else [args.prompt_len] * args.batch
        if args.replayed:
            rep = measure.replayed_kernels(model, lens, prefill=args.stages == "prefill")
            measure.print_replayed_kernels(rep, f"{args.stages} step as the engine runs it, {len(lens)} sequence(s) of "
                                                f"{lens[0]} tokens, LFM2.5-1.2B shape")
            return 0
        rep = measure.stage_report(model, lens, prefill=args.stages == "prefill")
        measure.print_stage_report(rep, f"{args.stages} step, {len(lens)} sequence(s) of {lens[0]} tokens, LFM2.5-1.2B shape", pk)
        return 0

    # the clocks are sampled over all the timed regions of this run (the K decode steps alone are
    # shorter than one sampling period)
    with ClockSampler() as clk:
        res = measure.decode_run(model, [PROMPT] * args.batch, steps, warmup, room_each=CONTEXT)
        main_point = decode_point(nums, res, args.batch, pk)

        pre_ms = measure.prefill_run(model, PREFILL_TOKENS, reps=5, warmup=3)
        pre_flops = (PREFILL_TOKENS * nums["gemm_flops_per_token"] + nums["head_flops_per_row"]
                     + nums["attn_flops"](PREFILL_TOKENS))
        pre_tflops = pre_flops / (pre_ms * 1e-3) / 1e12
        prefill = {"value": PREFILL_TOKENS / (pre_ms * 1e-3), "tokens": PREFILL_TOKENS, "ms": pre_ms,
                   "tflops": pre_tflops, "frac": pre_tflops / pk["bf16_tflops"],
                   # frac is against the burst figure (one step, timed alone); the library product under the
                   # power cap of a long run settles lower, for comparison:
                   "frac_of_sustained": pre_tflops / pk["bf16_tflops_sustained"]}

        points, e2e = {}, None
        if not args.no_points:
            for b in (1, 64, 256):
                # enough steps that the first one's enqueue (the GPU idles meanwhile) does not weigh
                r = measure.decode_run(model, [PROMPT] * b, max(32, steps), warmup, room_each=CONTEXT)
                pt = decode_point(nums, r, b, pk)
                points[f"decode_b{b}"] = pt["value"]
                points[f"decode_b{b}_ms"] = pt["ms_per_step"]
                points[f"decode_b{b}_frac"] = pt["frac"]
            # a prompt of a quarter of the headline's length, where the step's launches weigh more
            points["prefill_512"] = 512 / (measure.prefill_run(model, 512, reps=5, warmup=3) * 1e-3)
            # at least 256 steps: generation's ends (the prefill before the first token, the last step, which
            # has no successor enqueued behind it) then weigh as little as they do in service
            e = measure.generate_run(model, [PROMPT] * args.batch, max(steps, 256) + 1, warmup_tokens=warmup + 1)
            e2e = {"value": e["decode_tokens_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": e["h2d_bytes_per_step"],
                   "d2h_bytes_per_step": e["d2h_bytes_per_step"]}
    clocks = clk.summary()

    line = {
        "metric": "decode tokens/s, LFM2.5-1.2B shape, bf16, random weights", "value": main_point["value"],
        "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": res["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (uniform random token ids, random weights)", "impl": "ours",
        "config": flat_config(model, "LFM2.5-1.2B shape", args.layers, FULL_LAYERS, args.batch, PROMPT, CONTEXT, pk_src,
                              nums["weight_bytes"]),
        "clocks": clocks,
        "gpu_launches": res["launches"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "bytes_per_step": main_point["bytes_per_step"], "achieved": main_point["gb_per_s"],
                     "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": main_point["frac"]},
        "points": points,
    }
    if e2e is not None:
        line["e2e"] = e2e
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
