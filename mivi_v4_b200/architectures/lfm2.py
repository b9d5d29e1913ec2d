"""The LFM2 / LFM2.5 hybrid decoder described in parts: which part sits in
which layer, with which sizes, under which tensor names.

Layers are pre-norm residual blocks; the mixer of layer i is the gated short
convolution where ``layer_types[i]`` is "conv" and grouped-query attention
where it is "full_attention"; every layer has a SwiGLU feed-forward; a final
norm and a tied or untied head follow.  The reference decides the kind of a
layer by the tensors present (crates/mivi-model/src/loader.rs:157-174) and
names them blk.i.* (loader.rs:264-342, 359-415); the checkpoint names used
here are the model folder's:

  model.embed_tokens.weight                          [V, H]
  model.layers.i.operator_norm.weight                [H]
  model.layers.i.conv.{in_proj,out_proj}.weight      [3H, H], [H, H]
  model.layers.i.conv.conv.weight                    [H, 1, k]
  model.layers.i.conv.{in_proj,conv,out_proj}.bias   with conv_bias
  model.layers.i.self_attn.{q,k,v}_proj.weight       [nh*hd, H], [nkv*hd, H] x 2
  model.layers.i.self_attn.out_proj.weight           [H, nh*hd]
  model.layers.i.self_attn.{q,k}_layernorm.weight    [hd]
  model.layers.i.ffn_norm.weight                     [H]
  model.layers.i.feed_forward.{w1,w3,w2}.weight      [F, H], [F, H], [H, F]
  model.embedding_norm.weight                        [H]
  lm_head.weight                                     [V, H], untied only
"""
from __future__ import annotations

from ..config.lfm2 import Lfm2Config
from ..config.registry import register_architecture
from ..parts.spec import ModelSpec, PartSpec, ScheduleEntry

NAME = "Lfm2ForCausalLM"


def describe(cfg: Lfm2Config) -> ModelSpec:
    H = cfg.hidden_size
    blocks = []
    for i, kind in enumerate(cfg.layer_types):
        pre = f"model.layers.{i}."
        if kind == "conv":
            mixer = PartSpec("short_conv", dict(hidden=H, kernel=cfg.conv_L_cache, bias=cfg.conv_bias),
                             prefix=pre + "conv.")
        else:
            rope = PartSpec("rope", dict(head_dim=cfg.head_dim, theta=cfg.rope_theta, style=cfg.rope_style))
            mixer = PartSpec("gqa", dict(hidden=H, n_heads=cfg.num_attention_heads,
                                         n_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim,
                                         qk_norm_eps=cfg.norm_eps),
                             prefix=pre + "self_attn.", parts={"position": rope})
        blocks.append(PartSpec("prenorm", prefix=pre, parts={
            "mixer_norm": PartSpec("rmsnorm", dict(dim=H, eps=cfg.norm_eps), prefix=pre + "operator_norm."),
            "mixer": mixer,
            "ffn_norm": PartSpec("rmsnorm", dict(dim=H, eps=cfg.norm_eps), prefix=pre + "ffn_norm."),
            "ffn": PartSpec("swiglu", dict(hidden=H, ff=cfg.ff_dim), prefix=pre + "feed_forward."),
        }))
    stops = () if cfg.eos_token_id is None else (cfg.eos_token_id,)
    return ModelSpec(
        hidden_size=H, vocab_size=cfg.vocab_size,
        embedding=PartSpec("table", dict(vocab=cfg.vocab_size, hidden=H), prefix="model.embed_tokens."),
        blocks=blocks,
        schedule=[ScheduleEntry(i) for i in range(cfg.num_hidden_layers)],
        final_norm=PartSpec("rmsnorm", dict(dim=H, eps=cfg.norm_eps), prefix="model.embedding_norm."),
        head=PartSpec("linear", dict(vocab=cfg.vocab_size, hidden=H, tied=cfg.tie_embedding), prefix="lm_head."),
        # a tied checkpoint may still carry a copy of the table under the head's name
        ignorable=("lm_head.weight",) if cfg.tie_embedding else (),
        stop_token_ids=stops, max_positions=cfg.max_position_embeddings,
    )


register_architecture(NAME, Lfm2Config.from_dict, describe, replace=True)
