#!/usr/bin/env python3
"""Compare tests/plain_lfm2.py once with the reference's own Python oracle.

Usage:  python tests/golden/make_golden.py /path/to/aswin402-mivi-v4

It imports ``reference/reference_engine.py`` of the reference checkout
(standard library only, runs on the CPU) and
1. rebuilds the weights of the reference's fixture with its own generators
   (training/export/generate_fixture.py:20-38, 73-97), runs the oracle on the
   tokens [1, 5, 12, 3] and checks that it reproduces the reference's checked-in
   tests/fixtures/oracle_output.json, then runs the plain implementation on the
   same weights;
2. builds a second tiny model with closed-form weights (no random generator,
   so the test can rebuild it bit for bit) and runs both on a longer sequence.
The oracle's logits are written to tests/golden/oracle_golden.json, which is
committed; tests/test_plain.py compares the plain implementation with that
file without needing the reference.

What the oracle cannot anchor (reference_engine.py has no per-head q/k norm,
a convolution width fixed at 3, eps fixed at 1e-5, no biases, no tied head,
interleaved rotation only) rests on the formulas cited in plain_lfm2.py.

One difference between the oracle and the Rust engine shows here.  The
oracle's apply_rope (reference_engine.py:66-81) is handed the whole q and k
vectors and loops ``for i in range(0, head_dim, 2)``, so it rotates only the
FIRST head of q and of k; the Rust engine rotates every head
(crates/mivi-core/src/rope.rs:211-231, called with n_heads and n_kv_heads at
crates/mivi-model/src/transformer.rs:99-105), and its own test passes only
because of its 0.05 tolerance (tests/oracle_comparison_test.rs:57-75).  The
plain implementation follows the Rust engine.  So the cases with more than one
head are compared with the rotation limited to the first head
(``first_head_only``), which reproduces the oracle to 1e-15, and one case with
a single head is compared as it stands.
"""
import json
import math
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import plain_lfm2  # noqa: E402
from plain_lfm2 import plain_forward  # noqa: E402

_full_rope = plain_lfm2.plain_rope


def first_head_only(v, positions, theta, style="interleaved"):
    """The oracle's rotation: head 0 only (see the header)."""
    out = v.clone()
    out[:, :1] = _full_rope(v[:, :1], positions, theta, style)
    return out


def closed_form_matrix(rows, cols, phase, scale=0.08):
    return [[scale * math.sin(1.7 * r + 0.61 * c + phase) + 0.5 * scale * math.cos(0.37 * r * c + phase)
             for c in range(cols)] for r in range(rows)]


def closed_form_vector(n, phase, base=1.0, scale=0.1):
    return [base + scale * math.sin(0.9 * i + phase) for i in range(n)]


def second_model(n_heads=4, n_kv_heads=2):
    hd = 32 // n_heads
    cfg = dict(dim=32, hidden_dim=48, n_layers=3, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=hd,
               kv_dim=hd * n_kv_heads, vocab_size=40, block_types=["ssm", "attention", "ssm"],
               rope_base=10000.0)
    H, F, V, kvd = 32, 48, 40, hd * n_kv_heads
    w = {"token_embd.weight": closed_form_matrix(V, H, 0.1, 0.5),
         "output.weight": closed_form_matrix(V, H, 0.2, 0.3),
         "output_norm.weight": closed_form_vector(H, 0.3)}
    ph = 1.0
    for l, kind in enumerate(cfg["block_types"]):
        def nxt():
            nonlocal ph
            ph += 0.77
            return ph
        if kind == "ssm":
            w[f"blk.{l}.ssm_norm.weight"] = closed_form_vector(H, nxt())
            w[f"blk.{l}.shortconv.in_proj.weight"] = closed_form_matrix(3 * H, H, nxt(), 0.3)
            w[f"blk.{l}.shortconv.conv.weight"] = closed_form_vector(3 * H, nxt(), 0.3, 0.4)
            w[f"blk.{l}.shortconv.out_proj.weight"] = closed_form_matrix(H, H, nxt(), 0.3)
        else:
            w[f"blk.{l}.attn_norm.weight"] = closed_form_vector(H, nxt())
            w[f"blk.{l}.attn_q.weight"] = closed_form_matrix(H, H, nxt(), 0.4)
            w[f"blk.{l}.attn_k.weight"] = closed_form_matrix(kvd, H, nxt(), 0.4)
            w[f"blk.{l}.attn_v.weight"] = closed_form_matrix(kvd, H, nxt(), 0.4)
            w[f"blk.{l}.attn_output.weight"] = closed_form_matrix(H, H, nxt(), 0.3)
        w[f"blk.{l}.ffn_norm.weight"] = closed_form_vector(H, nxt())
        w[f"blk.{l}.ffn_gate.weight"] = closed_form_matrix(F, H, nxt(), 0.3)
        w[f"blk.{l}.ffn_up.weight"] = closed_form_matrix(F, H, nxt(), 0.3)
        w[f"blk.{l}.ffn_down.weight"] = closed_form_matrix(H, F, nxt(), 0.3)
    return cfg, w, [3, 17, 0, 39, 8, 8, 21, 5, 30, 12, 1]


def to_checkpoint(cfg, w):
    """The oracle's names and sizes -> config.json keys and checkpoint tensor names."""
    kinds = {"ssm": "conv", "attention": "full_attention"}
    hf_cfg = dict(hidden_size=cfg["dim"], num_hidden_layers=cfg["n_layers"],
                  num_attention_heads=cfg["n_heads"], num_key_value_heads=cfg["n_kv_heads"],
                  vocab_size=cfg["vocab_size"], rope_theta=cfg["rope_base"], norm_eps=1e-5,
                  conv_L_cache=3, conv_bias=False, block_ff_dim=cfg["hidden_dim"],
                  block_auto_adjust_ff_dim=False, tie_embedding=False, rope_style="interleaved",
                  layer_types=[kinds[k] for k in cfg["block_types"]])
    t = lambda x: torch.tensor(x, dtype=torch.float64)
    H = cfg["dim"]
    out = {"model.embed_tokens.weight": t(w["token_embd.weight"]),
           "lm_head.weight": t(w["output.weight"]),
           "model.embedding_norm.weight": t(w["output_norm.weight"])}
    for l, kind in enumerate(cfg["block_types"]):
        p = f"model.layers.{l}."
        if kind == "ssm":
            out[p + "operator_norm.weight"] = t(w[f"blk.{l}.ssm_norm.weight"])
            out[p + "conv.in_proj.weight"] = t(w[f"blk.{l}.shortconv.in_proj.weight"])
            out[p + "conv.conv.weight"] = t(w[f"blk.{l}.shortconv.conv.weight"]).reshape(H, 1, 3)
            out[p + "conv.out_proj.weight"] = t(w[f"blk.{l}.shortconv.out_proj.weight"])
        else:
            out[p + "operator_norm.weight"] = t(w[f"blk.{l}.attn_norm.weight"])
            out[p + "self_attn.q_proj.weight"] = t(w[f"blk.{l}.attn_q.weight"])
            out[p + "self_attn.k_proj.weight"] = t(w[f"blk.{l}.attn_k.weight"])
            out[p + "self_attn.v_proj.weight"] = t(w[f"blk.{l}.attn_v.weight"])
            out[p + "self_attn.out_proj.weight"] = t(w[f"blk.{l}.attn_output.weight"])
        out[p + "ffn_norm.weight"] = t(w[f"blk.{l}.ffn_norm.weight"])
        out[p + "feed_forward.w1.weight"] = t(w[f"blk.{l}.ffn_gate.weight"])
        out[p + "feed_forward.w3.weight"] = t(w[f"blk.{l}.ffn_up.weight"])
        out[p + "feed_forward.w2.weight"] = t(w[f"blk.{l}.ffn_down.weight"])
    return hf_cfg, out


def main():
    ref_root = sys.argv[1]
    sys.path.insert(0, ref_root)
    from reference.reference_engine import LFMConfig, ReferenceEngine
    import importlib.util
    spec = importlib.util.spec_from_file_location(
        "generate_fixture", os.path.join(ref_root, "training/export/generate_fixture.py"))
    # the fixture script imports its GGUF writer at module level; only its two
    # generator functions are needed, so load it with that import satisfied.
    fx = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(fx)
    gm, gv = fx.generate_deterministic_matrix, fx.generate_deterministic_vector

    # 1. the reference's own fixture
    dim, hid, kvd, V = 64, 128, 32, 64
    cfg1 = dict(dim=dim, hidden_dim=hid, n_layers=2, n_heads=2, n_kv_heads=1, head_dim=32, kv_dim=kvd,
                vocab_size=V, block_types=["ssm", "attention"], rope_base=1_000_000.0)
    w1 = {"token_embd.weight": gm(V, dim, 0.15), "output.weight": gm(V, dim, 0.25),
          "output_norm.weight": gv(dim, 1.0),
          "blk.0.ssm_norm.weight": gv(dim, 1.0),
          "blk.0.shortconv.in_proj.weight": gm(3 * dim, dim, 0.3),
          "blk.0.shortconv.conv.weight": gv(3 * dim, 0.25),
          "blk.0.shortconv.out_proj.weight": gm(dim, dim, 0.4),
          "blk.0.ffn_norm.weight": gv(dim, 1.0), "blk.0.ffn_gate.weight": gm(hid, dim, 0.5),
          "blk.0.ffn_up.weight": gm(hid, dim, 0.6), "blk.0.ffn_down.weight": gm(dim, hid, 0.7),
          "blk.1.attn_norm.weight": gv(dim, 1.0), "blk.1.attn_q.weight": gm(dim, dim, 0.8),
          "blk.1.attn_k.weight": gm(kvd, dim, 0.9), "blk.1.attn_v.weight": gm(kvd, dim, 1.1),
          "blk.1.attn_output.weight": gm(dim, dim, 1.2), "blk.1.ffn_norm.weight": gv(dim, 1.0),
          "blk.1.ffn_gate.weight": gm(hid, dim, 1.3), "blk.1.ffn_up.weight": gm(hid, dim, 1.4),
          "blk.1.ffn_down.weight": gm(dim, hid, 1.5)}
    toks1 = [1, 5, 12, 3]
    golden = {}
    cases = {"fixture": (cfg1, w1, toks1), "closed_form": second_model(),
             "closed_form_one_head": second_model(1, 1)}
    for tag, (cfg, w, toks) in cases.items():
        eng = ReferenceEngine(LFMConfig(name=tag, max_seq_len=512, **cfg), w)
        oracle = [eng.forward_token(t, p)["logits"] for p, t in enumerate(toks)]
        hf_cfg, ck = to_checkpoint(cfg, w)
        quirk = cfg["n_heads"] > 1
        plain_lfm2.plain_rope = first_head_only if quirk else _full_rope
        plain = plain_forward(hf_cfg, ck, toks, dtype=torch.float64)
        plain_lfm2.plain_rope = _full_rope
        diff = (plain - torch.tensor(oracle, dtype=torch.float64)).abs().max().item()
        print(f"{tag}: max |plain - oracle| = {diff:.3e} over {len(toks)} positions")
        assert diff < 1e-12, diff
        golden[tag] = {"tokens": toks, "oracle_logits": oracle, "max_abs_diff_plain_vs_oracle": diff,
                       "rotation": "first_head_only" if quirk else "all_heads"}
        if tag == "fixture":
            with open(os.path.join(ref_root, "tests/fixtures/oracle_output.json")) as f:
                committed = json.load(f)
            for row, lg in zip(committed, oracle):
                assert row["top_token"] == max(range(len(lg)), key=lambda i: lg[i])
                assert max(abs(a - b) for a, b in zip(row["logits_sample"], lg[:8])) == 0.0
            print("fixture: oracle reproduces the reference's tests/fixtures/oracle_output.json exactly")
            golden[tag]["reference_fixture"] = committed
    with open(os.path.join(HERE, "oracle_golden.json"), "w") as f:
        json.dump(golden, f)
    print("wrote", os.path.join(HERE, "oracle_golden.json"))


if __name__ == "__main__":
    main()
