"""Configuration, registry and weight loading (CPU)."""
import copy
import json
import os

import pytest
import torch

from tiny_configs import TINY_A, TINY_B

from mivi_v4_b200 import ConfigError, Lfm2Config, WeightsError, known_architectures, write_random_model
from mivi_v4_b200.config import architecture_for
from mivi_v4_b200.engine import expected_tensors, load_model
from mivi_v4_b200.weights import SafetensorsError, read_header, read_model_headers, read_tensor, write_file


def test_config_fields_and_derived_sizes():
    a, b = Lfm2Config.from_dict(TINY_A), Lfm2Config.from_dict(TINY_B)
    assert (a.head_dim, a.kv_dim, a.ff_dim, a.attn_layer_ids, a.conv_layer_ids) == (16, 32, 192, [1, 3], [0, 2])
    assert (b.head_dim, b.kv_dim, b.ff_dim, b.attn_layer_ids) == (32, 32, 256, [0, 3, 5])
    assert b.conv_bias and not b.tie_embedding and b.conv_L_cache == 4 and b.norm_eps == 1e-6
    assert a.rope_style == "interleaved"


@pytest.mark.parametrize("block_ff,want", [(12288, 8192), (10240, 6912), (6656, 4608)])
def test_ff_dim_auto_adjust(block_ff, want):
    cfg = dict(TINY_A, block_ff_dim=block_ff, block_auto_adjust_ff_dim=True, block_multiple_of=256,
               block_ffn_dim_multiplier=1.0)
    assert Lfm2Config.from_dict(cfg).ff_dim == want


def test_config_defaults_follow_the_reference():
    minimal = {k: TINY_A[k] for k in ("hidden_size", "num_hidden_layers", "num_attention_heads",
                                      "num_key_value_heads", "vocab_size", "block_ff_dim", "layer_types")}
    c = Lfm2Config.from_dict(minimal)
    assert (c.rope_theta, c.norm_eps, c.conv_L_cache, c.conv_bias, c.tie_embedding) == (1e6, 1e-5, 3, False, True)
    assert Lfm2Config.from_dict(dict(minimal, tie_word_embeddings=False)).tie_embedding is False


@pytest.mark.parametrize("patch,needle", [
    (dict(hidden_size=None), "hidden_size"),
    (dict(num_attention_heads=5), "multiple of num_attention_heads"),
    (dict(num_key_value_heads=3), "multiple of"),
    (dict(layer_types=["conv"]), "layer_types has 1"),
    (dict(layer_types=["conv", "mamba", "conv", "conv"]), "known kinds"),
    (dict(hidden_size="64"), "must be an integer"),
    (dict(conv_bias="yes"), "true or false"),
    (dict(rope_style="spiral"), "rope_style"),
    (dict(norm_eps=0.0), "norm_eps"),
    (dict(hidden_size=60, num_attention_heads=4, num_key_value_heads=2), "even"),
])
def test_config_errors_name_the_fault(patch, needle):
    cfg = dict(TINY_A)
    for k, v in patch.items():
        if v is None:
            cfg.pop(k)
        else:
            cfg[k] = v
    with pytest.raises(ConfigError) as e:
        Lfm2Config.from_dict(cfg)
    assert needle in str(e.value)


def test_registry():
    assert "Lfm2ForCausalLM" in known_architectures()
    assert architecture_for(TINY_A).name == "Lfm2ForCausalLM"
    with pytest.raises(ConfigError) as e:
        architecture_for(dict(TINY_A, architectures=["GptForCausalLM"]))
    assert "Lfm2ForCausalLM" in str(e.value)
    with pytest.raises(ConfigError):
        architecture_for({k: v for k, v in TINY_A.items() if k != "architectures"})


def test_name_table():
    names = expected_tensors(TINY_B)
    assert names["model.layers.1.conv.conv.weight"].shape == (96, 1, 4)
    assert names["model.layers.1.conv.in_proj.bias"].shape == (288,)
    assert names["model.layers.0.self_attn.k_proj.weight"].shape == (32, 96)
    assert names["model.layers.0.self_attn.q_layernorm.weight"].shape == (32,)
    assert names["model.layers.0.feed_forward.w1.weight"].shape == (256, 96)
    assert names["lm_head.weight"].shape == (384, 96)
    assert "lm_head.weight" not in expected_tensors(TINY_A)
    assert "model.layers.0.conv.in_proj.bias" not in expected_tensors(TINY_A)


def test_random_folder_round_trip(tmp_path):
    d = write_random_model(str(tmp_path / "m"), TINY_B, seed=1)
    d2 = write_random_model(str(tmp_path / "m2"), TINY_B, seed=1)
    h = read_model_headers(d)
    assert set(h) == set(expected_tensors(TINY_B))
    assert all(e.dtype == "BF16" for e in h.values())
    for name in ("model.embed_tokens.weight", "model.layers.1.conv.conv.weight"):
        assert torch.equal(read_tensor(h[name]), read_tensor(read_model_headers(d2)[name]))
    from safetensors.torch import load_file
    theirs = load_file(os.path.join(d, "model.safetensors"))
    assert torch.equal(theirs["lm_head.weight"], read_tensor(h["lm_head.weight"]))
    w = read_tensor(h["model.layers.1.operator_norm.weight"]).float()
    assert abs(w.mean() - 1.0) < 0.1 and 0.03 < w.std() < 0.2
    assert 0.1 < read_tensor(h["model.layers.1.conv.conv.weight"]).float().std() < 0.3
    assert json.load(open(os.path.join(d, "config.json")))["architectures"] == ["Lfm2ForCausalLM"]


def test_dtypes_kept(tmp_path):
    """bfloat16 stays bfloat16; a tensor stored in 32-bit stays so; vectors are read in 32-bit."""
    d = write_random_model(str(tmp_path / "m"), TINY_A, seed=0)
    path = os.path.join(d, "model.safetensors")
    from safetensors.torch import load_file
    t = load_file(path)
    t["model.layers.0.conv.in_proj.weight"] = t["model.layers.0.conv.in_proj.weight"].float()
    write_file(path, t)
    m = load_model(d, "bfloat16", "cpu")
    conv = m.blocks[0].mixer
    assert conv.w_in.dtype == torch.float32 and conv.w_out.dtype == torch.bfloat16
    assert conv.taps.dtype == torch.float32 and conv.taps.shape == (64, 3)
    assert m.embedding.weight.dtype == torch.bfloat16
    m32 = load_model(d, "float32", "cpu")
    assert m32.blocks[0].mixer.w_out.dtype == torch.float32 and m32.embedding.weight.dtype == torch.float32


def test_one_error_lists_every_fault(tmp_path):
    d = write_random_model(str(tmp_path / "m"), TINY_A, seed=0)
    path = os.path.join(d, "model.safetensors")
    from safetensors.torch import load_file
    t = load_file(path)
    del t["model.layers.1.self_attn.q_layernorm.weight"]
    del t["model.embedding_norm.weight"]
    t["model.layers.9.extra.weight"] = torch.zeros(3)
    t["model.layers.0.conv.conv.weight"] = torch.zeros(64, 3, dtype=torch.bfloat16)
    t["model.layers.0.ffn_norm.weight"] = torch.zeros(64, dtype=torch.int32)
    write_file(path, t)
    with pytest.raises(WeightsError) as e:
        load_model(d, "bfloat16", "cpu")
    err = e.value
    assert sorted(err.missing) == ["model.embedding_norm.weight", "model.layers.1.self_attn.q_layernorm.weight"]
    assert err.unexpected == ["model.layers.9.extra.weight"]
    assert err.wrong_shape == [("model.layers.0.conv.conv.weight", (64, 3), (64, 1, 3))]
    assert err.wrong_dtype == [("model.layers.0.ffn_norm.weight", "I32")]
    msg = str(err)
    for needle in ("missing (2)", "unexpected (1)", "wrong shape (1)", "[64, 3], expected [64, 1, 3]"):
        assert needle in msg


def test_tied_checkpoint_may_carry_the_head(tmp_path):
    d = write_random_model(str(tmp_path / "m"), TINY_A, seed=0)
    path = os.path.join(d, "model.safetensors")
    from safetensors.torch import load_file
    t = load_file(path)
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    write_file(path, t)
    load_model(d, "bfloat16", "cpu")


def test_corrupt_containers(tmp_path):
    p = str(tmp_path / "x.safetensors")
    open(p, "wb").write(b"\x05\x00")
    with pytest.raises(SafetensorsError):
        read_header(p)
    open(p, "wb").write((10 ** 12).to_bytes(8, "little") + b"{}")
    with pytest.raises(SafetensorsError):
        read_header(p)
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    open(p, "wb").write(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 8)      # data shorter than claimed
    with pytest.raises(SafetensorsError):
        read_header(p)
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [3], "data_offsets": [0, 16]}}).encode()
    open(p, "wb").write(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 16)     # size and shape disagree
    with pytest.raises(SafetensorsError):
        read_header(p)


def test_folder_without_weights(tmp_path):
    json.dump(TINY_A, open(str(tmp_path / "config.json"), "w"))
    with pytest.raises(WeightsError) as e:
        load_model(str(tmp_path), "bfloat16", "cpu")
    assert "model.safetensors" in str(e.value) and len(e.value.missing) == len(expected_tensors(TINY_A))


def test_sharded_folder(tmp_path):
    d = write_random_model(str(tmp_path / "m"), TINY_A, seed=0)
    from safetensors.torch import load_file
    t = load_file(os.path.join(d, "model.safetensors"))
    os.remove(os.path.join(d, "model.safetensors"))
    names = sorted(t)
    half = len(names) // 2
    write_file(os.path.join(d, "model-00001-of-00002.safetensors"), {n: t[n] for n in names[:half]})
    write_file(os.path.join(d, "model-00002-of-00002.safetensors"), {n: t[n] for n in names[half:]})
    wm = {n: "model-00001-of-00002.safetensors" for n in names[:half]}
    wm.update({n: "model-00002-of-00002.safetensors" for n in names[half:]})
    json.dump({"weight_map": wm}, open(os.path.join(d, "model.safetensors.index.json"), "w"))
    m = load_model(d, "float32", "cpu")
    assert torch.equal(m.embedding.weight, t["model.embed_tokens.weight"].float())


def test_missing_shard_is_a_weights_error(tmp_path):
    d = write_random_model(str(tmp_path / "m"), TINY_A, seed=0)
    os.rename(os.path.join(d, "model.safetensors"), os.path.join(d, "model-00001-of-00002.safetensors"))
    names = list(read_header(os.path.join(d, "model-00001-of-00002.safetensors")))
    wm = {n: "model-00001-of-00002.safetensors" for n in names[:-1]}
    wm[names[-1]] = "model-00002-of-00002.safetensors"
    json.dump({"weight_map": wm}, open(os.path.join(d, "model.safetensors.index.json"), "w"))
    with pytest.raises(WeightsError, match="model-00002-of-00002.safetensors"):
        load_model(d, "float32", "cpu")


def test_loud_init_and_storage_overrides(tmp_path):
    """``init="loud"``: matrices with standard deviation 1/sqrt(columns); ``store_overrides`` keeps single
    tensors in another dtype, which the loader then leaves in 32-bit in a bfloat16 run."""
    over = {"model.layers.0.feed_forward.w2.weight": "float32"}
    d = write_random_model(str(tmp_path / "m"), TINY_A, seed=3, init="loud", store_overrides=over)
    entries = read_model_headers(d)
    assert entries["model.layers.0.feed_forward.w2.weight"].dtype == "F32"
    assert entries["model.layers.0.feed_forward.w1.weight"].dtype == "BF16"
    m = load_model(d, "bfloat16", "cpu")
    ffn = m.blocks[0].ffn
    assert ffn.w2.dtype == torch.float32 and ffn.w13.dtype == torch.bfloat16
    w = m.blocks[0].mixer.w_in.float()
    assert abs(w.std().item() * TINY_A["hidden_size"] ** 0.5 - 1.0) < 0.1
    with pytest.raises(ValueError, match="does not have"):
        write_random_model(str(tmp_path / "n"), TINY_A, seed=3, store_overrides={"nope": "float32"})
    with pytest.raises(ValueError, match="init"):
        write_random_model(str(tmp_path / "n"), TINY_A, seed=3, init="quiet")


def test_weight_order_hints_follow_the_recorded_order():
    """The order of a step's products is noted once; replayed in that order each product learns its
    successor's weights (the last one the first's), capped in size; any other order ends the hints."""
    import torch
    from mivi_v4_b200.ops import linear as L
    ws = [torch.zeros(n, 64, dtype=torch.bfloat16) for n in (4, 100000, 8, 2)]
    with L.recording() as order:
        for w in ws:
            assert L._order.next_after(w) is None
    assert L._order is None and len(order.seen) == 4
    with L.looking_ahead(order):
        got = [L._order.next_after(w) for w in ws]
    assert got[0] == (ws[1].data_ptr(), min(100000 * 128, L._AHEAD_BYTES))
    assert got[1] == (ws[2].data_ptr(), 8 * 128)
    assert got[3] == (ws[0].data_ptr(), 4 * 128)              # the next step begins with the first again
    with L.looking_ahead(order):
        assert L._order.next_after(ws[0]) is not None
        assert L._order.next_after(ws[2]) is None             # not the recorded successor
        assert L._order.next_after(ws[3]) is None             # and nothing after it
    with L.looking_ahead(order, {ws[1].data_ptr(): 100000 * 128, ws[2].data_ptr(): 8}):
        got = [L._order.next_after(w) for w in ws]            # only memory that is known to last, whole tensors
    assert got[0] is not None and got[1] is None and got[2] is None and got[3] is None
    with L.looking_ahead(order):                              # a step with more products than recorded
        for w in ws:
            L._order.next_after(w)
        assert L._order.next_after(ws[0]) is None
