"""Command line in the manner of the reference's ``mivi`` binary
(crates/mivi-cli/src/commands.rs:21-139): the same verbs where they make sense
for a token-id library (generate in place of chat, info, doctor, bench) and
the same option names and meanings where the reference has them:

    -m/--model  -t/--temp  -p/--top-p  -k/--top-k  --min-p  -r/--rep-penalty
    --seed  -n/--max-tokens  -c/--ctx-size

with the chat command's defaults (commands.rs:86-99: temp 0.2, top-p 0.9,
top-k 40, min-p 0.05, repetition penalty 1.1, 512 tokens).  The library has no
tokenizer, so prompts are token ids.  ``random`` is the random-weights mode: it
writes a model folder from a configuration and a seed.

    python -m mivi_v4_b200 generate -m DIR --prompt-ids 1,2,3 --prompt-ids 4,5 -n 16 -t 0
    python -m mivi_v4_b200 info -m DIR
    python -m mivi_v4_b200 random --config cfg.json --seed 0 --out DIR
    python -m mivi_v4_b200 doctor
    python -m mivi_v4_b200 bench -m DIR | --config cfg.json [--bench-prompt-tokens 2048] [--batch 8] [--profile]
    python -m mivi_v4_b200 replay --model DIR --dtype bfloat16 --out DIR --max-tokens N < steps.jsonl
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import List


def _ids(text: str) -> List[int]:
    try:
        return [int(t) for t in text.replace(",", " ").split()]
    except ValueError:
        raise argparse.ArgumentTypeError(f"not a list of token ids: {text!r}") from None


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="mivi_v4_b200", description="LFM2 / LFM2.5 generation on one B200")
    sub = ap.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="generate token ids for prompts of token ids")
    g.add_argument("-m", "--model", required=True, help="folder with config.json and model.safetensors")
    g.add_argument("--prompt-ids", type=_ids, action="append", default=[],
                   help='one prompt as token ids, e.g. "1,2,3"; may be repeated')
    g.add_argument("--prompts-file", help="file with one prompt per line (token ids), or a JSON list of lists")
    g.add_argument("-t", "--temp", type=float, default=0.2, help="temperature; 0 is greedy")
    g.add_argument("-p", "--top-p", type=float, default=0.9)
    g.add_argument("-k", "--top-k", type=int, default=40)
    g.add_argument("--min-p", type=float, default=0.05)
    g.add_argument("-r", "--rep-penalty", type=float, default=1.1)
    g.add_argument("--presence-penalty", type=float, default=0.0)
    g.add_argument("--frequency-penalty", type=float, default=0.0)
    g.add_argument("--seed", type=int, default=None)
    g.add_argument("-n", "--max-tokens", type=int, default=512, help="most new tokens per prompt")
    g.add_argument("-c", "--ctx-size", type=int, default=None, help="most tokens of one sequence (default: from the model, else 16384)")
    g.add_argument("--stop-ids", type=_ids, default=None, help="token ids that end a sequence (default: the model's eos)")
    g.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    g.add_argument("--max-batch", type=int, default=64, help="most sequences that run together")
    g.add_argument("--json", action="store_true", help="print one JSON object instead of lines of ids")

    i = sub.add_parser("info", help="configuration and tensor table of a model folder")
    i.add_argument("-m", "--model", required=True)

    r = sub.add_parser("random", help="write a model folder with random weights")
    r.add_argument("--config", required=True, help="config.json to build from")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--out", required=True)
    r.add_argument("--store-dtype", default="bfloat16", choices=["bfloat16", "float32"])
    r.add_argument("--init", default="baseline", choices=["baseline", "loud"],
                   help="baseline: N(0, 0.02) matrices; loud: standard deviation 1/sqrt(columns)")

    sub.add_parser("doctor", help="GPU, compiler and kernel-library report")

    rp = sub.add_parser("replay", help="feed given token ids step by step and write logits (bin/trace_run)")
    rp.add_argument("--model", required=True)
    rp.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    rp.add_argument("--out", required=True)
    rp.add_argument("--max-tokens", type=int, required=True)

    b = sub.add_parser("bench", help="prefill and decode throughput of a model folder")
    b.add_argument("-m", "--model", default=None, help="model folder")
    b.add_argument("--config", default=None, help="config.json: measure a model of these sizes with random weights")
    b.add_argument("--bench-prompt-tokens", type=int, default=2048, help="tokens of the timed prefill")
    b.add_argument("--prompt-tokens", type=int, default=512, help="cached tokens of each decoding sequence")
    b.add_argument("--batch", type=int, default=8, help="sequences that decode together")
    b.add_argument("--steps", type=int, default=64, help="timed decode steps")
    b.add_argument("--profile", action="store_true", help="also print where a step's time goes, by stage and kernel")
    b.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    return ap


def cmd_generate(a) -> int:
    from . import Engine, SamplingParams, load_model
    prompts = list(a.prompt_ids)
    if a.prompts_file:
        text = open(a.prompts_file).read().strip()
        prompts += json.loads(text) if text.startswith("[") else [_ids(line) for line in text.splitlines() if line.strip()]
    if not prompts:
        print("generate: no prompts (use --prompt-ids or --prompts-file)", file=sys.stderr)
        return 2
    model = load_model(a.model, a.dtype, "cuda:0")
    ctx = a.ctx_size or model.spec.max_positions or 16384
    model.spec.max_positions = ctx
    longest = max(len(p) for p in prompts) + a.max_tokens
    batch = min(a.max_batch, len(prompts))
    eng = Engine(model, max_tokens=batch * (min(ctx, longest) + 64), max_batch=batch)
    sp = SamplingParams(temperature=a.temp, top_p=a.top_p, top_k=a.top_k, min_p=a.min_p,
                        repetition_penalty=a.rep_penalty, presence_penalty=a.presence_penalty,
                        frequency_penalty=a.frequency_penalty, seed=a.seed)
    t0 = time.perf_counter()
    reqs = eng.generate(prompts, a.max_tokens, sp, stop_token_ids=a.stop_ids, return_requests=True)
    dt = time.perf_counter() - t0
    n_new = sum(len(r.output) for r in reqs)
    if a.json:
        print(json.dumps({"outputs": [r.output for r in reqs], "finish": [r.finish_reason for r in reqs],
                          "seconds": dt, "new_tokens": n_new}))
    else:
        for r in reqs:
            print(" ".join(str(t) for t in r.output))
        print(f"[{n_new} tokens in {dt:.2f} s, {n_new / dt:.1f} tok/s]", file=sys.stderr)
    return 0


def cmd_info(a) -> int:
    from .config import read_config_json
    from .engine.model import describe_config
    from .weights import read_model_headers
    cfg = read_config_json(a.model)
    config, spec = describe_config(cfg)
    print(f"architecture: {cfg['architectures'][0]}")
    for k, v in config.to_dict().items():
        print(f"  {k}: {v}")
    for k in ("head_dim", "kv_dim", "ff_dim", "attn_layer_ids", "conv_layer_ids"):
        if hasattr(config, k):
            print(f"  ({k}: {getattr(config, k)})")
    entries = read_model_headers(a.model)
    total = 0
    print(f"tensors: {len(entries)}")
    for name, e in entries.items():
        n = 1
        for s in e.shape:
            n *= s
        total += n
        print(f"  {name:56s} {e.dtype:5s} {list(e.shape)}")
    print(f"parameters: {total:,}")
    return 0


def cmd_random(a) -> int:
    from . import write_random_model
    with open(a.config) as f:
        cfg = json.load(f)
    print(write_random_model(a.out, cfg, a.seed, a.store_dtype, a.init))
    return 0


def cmd_doctor(a) -> int:
    import torch
    from .ops.build import LIBRARIES, build_dir, find_nvcc, library_path
    import os
    print(f"torch {torch.__version__}, CUDA available: {torch.cuda.is_available()}")
    if torch.cuda.is_available():
        p = torch.cuda.get_device_properties(0)
        print(f"GPU 0: {p.name}, sm_{p.major}{p.minor}, {p.multi_processor_count} SMs, {p.total_memory / 2**30:.1f} GiB")
        if (p.major, p.minor) != (10, 0):
            print("  warning: the kernels are compiled for sm_100a only")
    try:
        print(f"nvcc: {find_nvcc()}")
    except Exception as e:  # noqa: BLE001
        print(f"nvcc: NOT FOUND ({e})")
    print(f"build folder: {build_dir()}")
    for name in LIBRARIES:
        path = library_path(name)
        print(f"  {name}: {'built' if os.path.isfile(path) else 'not built yet'} ({os.path.basename(path)})")
    return 0


def cmd_bench(a) -> int:
    """Prefill and decode throughput of a model folder (or of random weights for a config.json), and with
    ``--profile`` where the time of a decode step and of the prefill goes, stage by stage, as the
    reference's bench prints its forward profile (crates/mivi-cli/src/runners/bench.rs:178-238)."""
    from . import load_model, measure, random_model
    if a.model is not None:
        model = load_model(a.model, a.dtype, "cuda:0")
    elif a.config is not None:
        with open(a.config) as f:
            model = random_model(json.load(f), seed=0, dtype=a.dtype, device="cuda:0", on_device=True)
    else:
        print("bench: give a model folder (-m) or a config.json for random weights (--config)", file=sys.stderr)
        return 2
    T, B = a.bench_prompt_tokens, a.batch
    nums = measure.model_numbers(model)
    pre_ms = measure.prefill_run(model, T, reps=3, warmup=2)
    dec = measure.decode_run(model, [a.prompt_tokens] * B, a.steps, warmup=4)
    gen = measure.generate_run(model, [a.prompt_tokens] * B, a.steps + 1)
    step_bytes = nums["weight_bytes"] + B * (dec["cached_tokens_mean"] * nums["kv_bytes_per_token"]
                                             + nums["state_bytes_per_seq"])
    pre_flops = T * nums["gemm_flops_per_token"] + nums["head_flops_per_row"] + nums["attn_flops"](T)
    print(json.dumps({
        "prompt_tokens": T, "prefill_tok_s": T / (pre_ms * 1e-3), "prefill_ms": pre_ms,
        "prefill_tflops": pre_flops / (pre_ms * 1e-3) / 1e12, "batch": B, "decode_tok_s": B * 1e3 / dec["ms_per_step"],
        "decode_ms_per_step": dec["ms_per_step"], "decode_bytes_per_step": step_bytes,
        "decode_gb_per_s": step_bytes / (dec["ms_per_step"] * 1e-3) / 1e9,
        "generate_tok_s": gen["decode_tokens_per_s"], "kernels_per_step": dec["launches"] / a.steps}))
    if a.profile:
        measure.print_stage_report(measure.stage_report(model, [a.prompt_tokens] * B),
                                   f"decode step, {B} sequence(s) of {a.prompt_tokens} cached tokens")
        measure.print_stage_report(measure.stage_report(model, [T], prefill=True), f"prefill of {T} tokens")
    return 0


def cmd_replay(a) -> int:
    from .replay import main as replay_main
    return replay_main(["--model", a.model, "--dtype", a.dtype, "--out", a.out, "--max-tokens", str(a.max_tokens)])


def main(argv=None) -> int:
    a = build_parser().parse_args(argv)
    if a.command in ("generate", "bench", "replay"):
        import torch
        if not torch.cuda.is_available():
            print(f"{a.command}: no CUDA device; this library runs on a GPU only (there is no CPU path)",
                  file=sys.stderr)
            return 2
    try:
        return {"replay": cmd_replay, "generate": cmd_generate, "info": cmd_info, "random": cmd_random,
                "doctor": cmd_doctor, "bench": cmd_bench}[a.command](a)
    except Exception as e:            # the library's own errors as one line, anything else as it is
        if type(e).__name__ in ("ConfigError", "WeightsError", "SafetensorsError", "StepError", "CacheError",
                                "GenerationError", "KernelError", "BuildError") and not os.environ.get("MIVI_TRACEBACK"):
            print(f"mivi {a.command}: {type(e).__name__}: {e}", file=sys.stderr)
            return 1
        if not isinstance(e, BrokenPipeError):
            raise
        # the reader of our output went away (``| head``): nothing more to say, and no traceback
        try:
            sys.stdout = open(os.devnull, "w")
        except OSError:
            pass
        return 0
