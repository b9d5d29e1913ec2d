"""Shared by the tests: model folders in temporary directories, the plain
implementation's view of a folder, and the comparison rules."""
import json
import os

import torch
from safetensors.torch import load_file       # an independent reader: cross-checks the library's writer

import plain_lfm2 as P

# Tolerances.  float32: the engine and the plain implementation (float64) differ
# by summation order only.  bfloat16: weights are exact in both, activations
# between kernels are rounded to bfloat16 (2^-9 relative) a few times per layer.
TOL = {torch.float32: dict(atol=2e-5, rtol=2e-5), torch.bfloat16: dict(atol=2.5e-2, rtol=2.5e-2)}


def write_model(tmpdir, cfg, seed, store="bfloat16"):
    from mivi_v4_b200 import write_random_model
    d = os.path.join(str(tmpdir), f"model_s{seed}_{store}")
    if not os.path.isdir(d):
        write_random_model(d, cfg, seed, store)
    return d


def plain_view(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    weights = load_file(os.path.join(model_dir, "model.safetensors"))
    return cfg, weights


def plain_logits(model_dir, tokens):
    cfg, weights = plain_view(model_dir)
    return P.plain_forward(cfg, weights, tokens, dtype=torch.float64)


def assert_close(got, want, dtype, what=""):
    got = got.detach().double().cpu()
    want = want.detach().double().cpu()
    assert got.shape == want.shape, (what, got.shape, want.shape)
    tol = TOL[dtype]
    # logits of these models are O(1) or smaller; the absolute term carries the bfloat16 case
    err = (got - want).abs()
    bound = tol["atol"] * max(1.0, want.abs().max().item()) + tol["rtol"] * want.abs()
    bad = err > bound
    if bad.any():
        idx = bad.nonzero()[0].tolist()
        raise AssertionError(f"{what}: {int(bad.sum())} of {bad.numel()} values differ; first at {idx}: "
                             f"got {got[tuple(idx)].item():.6g}, want {want[tuple(idx)].item():.6g}; "
                             f"max error {err.max().item():.3g}")
