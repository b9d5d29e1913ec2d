"""The tolerance of the engine-level comparisons can fail: statements about the comparison rules
themselves, checked with the plain implementation alone (no GPU)."""
import pytest
import torch

from helpers import mutated_logits, plain_logits, plain_noise, would_fail
from tiny_configs import all_folders, config_of, prompts

DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return all_folders(tmp_path_factory.mktemp("models"))


@pytest.mark.parametrize("name,dtype", [(n, d) for n in ["A", "B", "AL", "BL", "FL"] for d in DTYPES
                                        if not (n in ("A", "B") and d == torch.bfloat16)])
def test_a_fault_in_any_one_part_would_show(folders, name, dtype):
    """The comparisons above can fail: the plain logits of the same model with ONE tensor of ONE layer
    zeroed (a convolution's out_proj, an attention's out_proj, a feed-forward's w2) or a convolution's taps
    reversed lie outside the tolerance in use, for every layer.  (The two quiet configurations are
    held to this in float32 only: in bfloat16 their convolutions move the logits by four to nine
    times the rounding noise, too close to the rule's own factor to be a statement; the loud
    sets are there for that.)"""
    cfg = config_of(name)
    toks = prompts(cfg["vocab_size"], [40], seed=21)[0]
    want = plain_logits(folders[name], toks)
    noise = plain_noise(folders[name], toks, dtype)
    assert not would_fail(want, want, dtype, noise)
    for i, kind in enumerate(cfg["layer_types"]):
        pre = f"model.layers.{i}."
        names = [pre + "feed_forward.w2.weight",
                 pre + ("conv.out_proj.weight" if kind == "conv" else "self_attn.out_proj.weight")]
        for n in names:
            assert would_fail(mutated_logits(folders[name], toks, n), want, dtype, noise), (name, n)
        if kind == "conv" and cfg["conv_L_cache"] > 1:
            flipped = mutated_logits(folders[name], toks, pre + "conv.conv.weight", lambda w: w.flip(-1))
            assert would_fail(flipped, want, dtype, noise), (name, i, "taps reversed")
