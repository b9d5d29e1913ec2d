"""Shared by the tests: model folders in temporary directories, the plain
implementation's view of a folder, and the comparison rules."""
import json
import os
from collections import OrderedDict

import torch
from safetensors.torch import load_file       # an independent reader: cross-checks the library's writer

import plain_lfm2 as P

# Tolerances.  float32: the engine and the plain implementation (float64) differ
# by summation order only.  bfloat16 without a measured noise (kernels and parts
# alone): weights are exact in both, activations between kernels are rounded to
# bfloat16 (2^-9 relative) a few times per layer.
TOL = {torch.float32: dict(atol=2e-5, rtol=2e-5), torch.bfloat16: dict(atol=2.5e-2, rtol=2.5e-2)}

# bfloat16 at engine level: the error is held against the rounding noise that the plain
# implementation itself shows when it rounds its activations where a bfloat16 run stores them
# (``plain_noise``).  Each row's error (root mean square over the vocabulary) may be
# RMS_FACTOR times that noise, a single logit MAX_FACTOR times (among 10^5..10^7 values of a
# bell-shaped error the largest lies 4.5 to 5.5 deviations out; the engine rounds at slightly
# other places than the estimate, hence the margin).  A fault that these tests are after (a
# wrong slot, position, page or tap) moves logits by as much as a whole part contributes,
# tens to hundreds of times the noise when every part is loud.
RMS_FACTOR, MAX_FACTOR = 4.0, 16.0


def write_model(tmpdir, cfg, seed, store="bfloat16", init="baseline", store_overrides=None, tag=""):
    from mivi_v4_b200 import write_random_model
    d = os.path.join(str(tmpdir), f"model_s{seed}_{store}_{init}{tag}")
    if not os.path.isdir(d):
        write_random_model(d, cfg, seed, store, init, store_overrides)
    return d


def plain_view(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    weights = load_file(os.path.join(model_dir, "model.safetensors"))
    return cfg, weights


_views = {}


def plain_view64(model_dir):
    """The folder's configuration and its weights widened to float64 once (exact)."""
    if model_dir not in _views:
        cfg, weights = plain_view(model_dir)
        _views[model_dir] = (cfg, {k: v.to(torch.float64) for k, v in weights.items()})
    return _views[model_dir]


def forget_view(model_dir):
    _views.pop(model_dir, None)
    for k in [k for k in _memo if k[0] == model_dir]:
        del _memo[k]


_memo = OrderedDict()
_MEMO_BYTES = 1 << 30


def _remember(key, make):
    if key in _memo:
        _memo.move_to_end(key)
        return _memo[key]
    val = make()
    _memo[key] = val
    size = lambda v: v.numel() * v.element_size() if isinstance(v, torch.Tensor) else 8   # noqa: E731
    while sum(size(v) for v in _memo.values()) > _MEMO_BYTES and len(_memo) > 1:
        _memo.popitem(last=False)
    return val


def plain_logits(model_dir, tokens):
    """float64 logits [T, V] of the whole sequence by the plain implementation."""
    cfg, weights = plain_view64(model_dir)
    return _remember((model_dir, tuple(tokens), "logits"),
                     lambda: P.plain_forward(cfg, weights, list(tokens), dtype=torch.float64))


def plain_noise(model_dir, tokens, dtype):
    """How far a run in ``dtype`` may lie from the float64 logits by rounding alone: the root mean
    square, over all logits of the sequence, of the plain implementation's own difference when it
    rounds what such a run stores between kernels (bfloat16), or works in float32 throughout."""
    def make():
        cfg, weights = plain_view64(model_dir)
        want = plain_logits(model_dir, tokens)
        if dtype == torch.bfloat16:
            sim = P.plain_forward(cfg, weights, list(tokens), dtype=torch.float64, rnd=P.round_to(torch.bfloat16))
        else:
            sim = P.plain_forward(cfg, {k: v.float() for k, v in weights.items()}, list(tokens),
                                  dtype=torch.float32).double()
        return float((sim - want).pow(2).mean().sqrt())
    return _remember((model_dir, tuple(tokens), "noise", str(dtype)), make)


def noise_verdict(got, want, noise):
    """None if ``got`` lies within the noise rule of ``want``, else what breaks it."""
    got = got.detach().double().cpu()
    want = want.detach().double().cpu()
    if got.shape != want.shape:
        return f"shapes {tuple(got.shape)} and {tuple(want.shape)}"
    if not torch.isfinite(got).all():
        return "values that are not finite"
    err = (got - want).abs()
    row_rms = err.pow(2).mean(dim=-1).sqrt()
    worst_row = int(row_rms.argmax())
    if row_rms[worst_row].item() > RMS_FACTOR * noise:
        return (f"row {worst_row} is off by {row_rms[worst_row].item():.3g} rms = "
                f"{row_rms[worst_row].item() / noise:.1f} x the rounding noise {noise:.3g} "
                f"(allowed {RMS_FACTOR:g} x); first row beyond: {int((row_rms > RMS_FACTOR * noise).nonzero()[0])}")
    if err.max().item() > MAX_FACTOR * noise:
        idx = (err == err.max()).nonzero()[0].tolist()
        return (f"value {idx} is off by {err.max().item():.3g} = {err.max().item() / noise:.1f} x the rounding "
                f"noise {noise:.3g} (allowed {MAX_FACTOR:g} x): got {got[tuple(idx)].item():.6g}, "
                f"want {want[tuple(idx)].item():.6g}")
    return None


def assert_close(got, want, dtype, what="", noise=None):
    """``noise``: the rounding noise of this comparison (``plain_noise``); given for bfloat16, the
    noise rule above replaces the flat tolerance."""
    if noise is not None and dtype == torch.bfloat16:
        verdict = noise_verdict(got, want, noise)
        if verdict is not None:
            raise AssertionError(f"{what}: {verdict}")
        return
    got = got.detach().double().cpu()
    want = want.detach().double().cpu()
    assert got.shape == want.shape, (what, got.shape, want.shape)
    tol = TOL[dtype]
    # logits of these models are O(1) or smaller; the absolute term carries the bfloat16 case
    err = (got - want).abs()
    bound = tol["atol"] * max(1.0, want.abs().max().item()) + tol["rtol"] * want.abs()
    bad = ~(err <= bound)
    if bad.any():
        idx = bad.nonzero()[0].tolist()
        raise AssertionError(f"{what}: {int(bad.sum())} of {bad.numel()} values differ; first at {idx}: "
                             f"got {got[tuple(idx)].item():.6g}, want {want[tuple(idx)].item():.6g}; "
                             f"max error {err.max().item():.3g}")


def would_fail(got, want, dtype, noise=None):
    try:
        assert_close(got, want, dtype, "", noise)
    except AssertionError:
        return True
    return False


def mutated_logits(model_dir, tokens, name, change=lambda w: torch.zeros_like(w)):
    """The plain logits of the folder's model with the tensor ``name`` changed."""
    cfg, weights = plain_view64(model_dir)
    mutated = dict(weights)
    mutated[name] = change(weights[name])
    return P.plain_forward(cfg, mutated, list(tokens), dtype=torch.float64)


def plain_cache(model_dir, tokens, dtype=None):
    """What a cache holds after ``tokens`` by the plain implementation ({"kv": ..., "state": ...}, float64),
    and with ``dtype`` the rounding noise of each of the two (root mean square) in a run of that dtype."""
    cfg, weights = plain_view64(model_dir)
    want = P.plain_forward(cfg, weights, list(tokens), dtype=torch.float64, return_cache=True)
    if dtype is None:
        return want
    if dtype == torch.bfloat16:
        sim = P.plain_forward(cfg, weights, list(tokens), dtype=torch.float64, rnd=P.round_to(torch.bfloat16),
                              return_cache=True)
    else:
        sim = P.plain_forward(cfg, {k: v.float() for k, v in weights.items()}, list(tokens), dtype=torch.float32,
                              return_cache=True)
    noise = {k: float((sim[k].double() - want[k]).pow(2).mean().sqrt()) for k in want if want[k] is not None}
    return want, noise


def check_cache(engine, slot, model_dir, tokens, dtype, what=""):
    """The keys, values and fixed-size state that ``slot`` holds after ``tokens`` against the plain
    implementation's: float32 to 2e-5 of the largest value; bfloat16 by the noise rule, each key, value or
    state row against the rounding noise of its kind (which includes the cache's own storage rounding)."""
    from mivi_v4_b200.cache import KVNeed
    want, noise = _remember((model_dir, tuple(tokens), "cache", str(dtype)),
                            lambda: plain_cache(model_dir, tokens, dtype))
    for g, got in engine.cache.dump_slot(slot).items():
        got = got.double().cpu()
        kind = "kv" if isinstance(engine.cache.plan.groups[g].need, KVNeed) else "state"
        ref = want[kind]
        assert got.shape == ref.shape, (what, kind, got.shape, ref.shape)
        if got.numel() == 0:
            continue
        if dtype == torch.float32:
            assert (got - ref).abs().max().item() <= 2e-5 * ref.abs().max().item(), (what, kind)
        else:
            verdict = noise_verdict(got.reshape(-1, got.shape[-1]), ref.reshape(-1, ref.shape[-1]), noise[kind])
            assert verdict is None, (what, kind, verdict)
