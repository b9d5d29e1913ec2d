"""Trace replay: feeds given token ids through a model step by step and writes
logits.  It samples nothing, and it has no forward pass, cache or loader of its
own: it drives the library's model, step function, cache and kernels, the ones
that generation uses.  ``bin/trace_run`` and the command line's ``replay`` verb
both end here.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps come on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries``: for each request its next tokens and the places among them whose
logits are wanted.  ``end``: requests that are finished after this step; what
they hold goes back to the cache.  For a step in which something is wanted,
DIR/<step>.f32 gets the logits at the wanted places, in the order of the
entries and of ``want``, as little-endian float32 [wanted, vocab].  After every
step a line ``done <step>`` is printed and flushed.  Exit status 0 when the
input ends.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Optional, Sequence


def main(argv: Optional[Sequence[str]] = None, stdin=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens that live requests hold at any time, each request rounded up to 64")
    args = ap.parse_args(argv)

    import torch
    from . import Engine, load_model

    if not torch.cuda.is_available():
        print("trace_run: no CUDA device; this library runs on a GPU only", file=sys.stderr)
        return 2
    os.makedirs(args.out, exist_ok=True)
    model = load_model(args.model, args.dtype, "cuda:0")
    engine = Engine(model, max_tokens=max(64, args.max_tokens), page_size=64)
    slots = {}
    for line in (sys.stdin if stdin is None else stdin):
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        items, want = [], []
        for e in rec.get("entries", []):
            rid = e["id"]
            if rid not in slots:
                slots[rid] = engine.open()
            items.append((slots[rid], e["tokens"]))
            want.append(e.get("want", []))
        if items:
            logits = engine.step(items, want, copy=False)
            if logits is not None:
                arr = logits.detach().to("cpu", torch.float32).contiguous().numpy().astype("<f4", copy=False)
                arr.tofile(os.path.join(args.out, f"{step}.f32"))
            else:
                torch.cuda.synchronize()
            engine.check_errors()                 # the host has waited for the step: a kernel's fault shows now
        for rid in rec.get("end", []):
            if rid in slots:
                engine.close(slots.pop(rid))
        print(f"done {step}", flush=True)
    return 0
