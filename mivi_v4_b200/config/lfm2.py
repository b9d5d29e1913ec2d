"""Typed configuration of the LFM2 / LFM2.5 hybrid decoder, read from the
architecture's own config.json keys.

The reference keeps the same hyper-parameters in ``ModelConfig``
(crates/mivi-model/src/config.rs:67-83) with the checks of ``validate``
(config.rs:87-120) and fills them from its model file's metadata
(crates/mivi-model/src/loader.rs:44-177).  Here they come from config.json;
defaults are the reference's where it has them (rope base 1e6, eps 1e-5,
convolution width 3: config.rs:5-13,155).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, fields
from typing import Any, List, Optional

from .errors import ConfigError

LAYER_KINDS = ("conv", "full_attention")
ROPE_STYLES = ("interleaved", "half_split")

_REQUIRED = (
    "hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
    "vocab_size", "block_ff_dim", "layer_types",
)


def _as_int(key: str, v: Any) -> int:
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
        raise ConfigError(f"config key {key!r} must be an integer, got {v!r}")
    return int(v)


def _as_float(key: str, v: Any) -> float:
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config key {key!r} must be a number, got {v!r}")
    return float(v)


def _as_bool(key: str, v: Any) -> bool:
    if not isinstance(v, bool):
        raise ConfigError(f"config key {key!r} must be true or false, got {v!r}")
    return v


@dataclass
class Lfm2Config:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    vocab_size: int
    block_ff_dim: int
    layer_types: List[str]
    rope_theta: float = 1_000_000.0
    norm_eps: float = 1e-5
    conv_L_cache: int = 3
    conv_bias: bool = False
    block_auto_adjust_ff_dim: bool = False
    block_multiple_of: int = 256
    block_ffn_dim_multiplier: Optional[float] = 1.0
    tie_embedding: bool = True
    # how the rotation pairs the elements of a head: the reference pairs
    # (2i, 2i+1) (crates/mivi-core/src/rope.rs:219-229)
    rope_style: str = "interleaved"
    max_position_embeddings: Optional[int] = None
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    pad_token_id: Optional[int] = None
    architectures: List[str] = field(default_factory=lambda: ["Lfm2ForCausalLM"])
    model_type: str = "lfm2"

    # ---- derived sizes -------------------------------------------------
    @property
    def head_dim(self) -> int:
        """hidden_size / num_attention_heads (crates/mivi-model/src/loader.rs:150-154)."""
        return self.hidden_size // self.num_attention_heads

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def ff_dim(self) -> int:
        """Width of the SwiGLU feed-forward from the block_* keys: block_ff_dim
        as it stands, or, with block_auto_adjust_ff_dim, int(2*block_ff_dim/3)
        times block_ffn_dim_multiplier rounded up to block_multiple_of."""
        ff = self.block_ff_dim
        if self.block_auto_adjust_ff_dim:
            ff = int(2 * ff / 3)
            if self.block_ffn_dim_multiplier is not None:
                ff = int(self.block_ffn_dim_multiplier * ff)
            m = self.block_multiple_of
            ff = m * ((ff + m - 1) // m)
        return ff

    @property
    def attn_layer_ids(self) -> List[int]:
        return [i for i, t in enumerate(self.layer_types) if t == "full_attention"]

    @property
    def conv_layer_ids(self) -> List[int]:
        return [i for i, t in enumerate(self.layer_types) if t == "conv"]

    # ---- checks ----------------------------------------------------------
    def validate(self) -> "Lfm2Config":
        for k in ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                  "vocab_size", "block_ff_dim", "conv_L_cache", "block_multiple_of"):
            if getattr(self, k) < 1:
                raise ConfigError(f"config key {k!r} must be at least 1, got {getattr(self, k)}")
        if self.hidden_size % self.num_attention_heads:
            raise ConfigError(
                f"hidden_size {self.hidden_size} is not a multiple of num_attention_heads "
                f"{self.num_attention_heads}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"head size {self.head_dim} must be even for the rotary encoding")
        if len(self.layer_types) != self.num_hidden_layers:
            raise ConfigError(
                f"layer_types has {len(self.layer_types)} entries, num_hidden_layers is "
                f"{self.num_hidden_layers}")
        for i, t in enumerate(self.layer_types):
            if t not in LAYER_KINDS:
                raise ConfigError(f"layer_types[{i}] = {t!r}; known kinds: {', '.join(LAYER_KINDS)}")
        if self.rope_style not in ROPE_STYLES:
            raise ConfigError(f"rope_style {self.rope_style!r}; known: {', '.join(ROPE_STYLES)}")
        if not (self.norm_eps > 0):
            raise ConfigError(f"norm_eps must be positive, got {self.norm_eps}")
        if not (self.rope_theta > 0):
            raise ConfigError(f"rope_theta must be positive, got {self.rope_theta}")
        if self.ff_dim < 1:
            raise ConfigError(f"feed-forward width works out to {self.ff_dim}")
        return self

    # ---- reading and writing ----------------------------------------------
    @classmethod
    def from_dict(cls, d: dict) -> "Lfm2Config":
        for k in _REQUIRED:
            if k not in d:
                raise ConfigError(f"config.json lacks the required key {k!r}")
        kw: dict = {}
        for k in ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                  "vocab_size", "block_ff_dim", "conv_L_cache", "block_multiple_of"):
            if k in d:
                kw[k] = _as_int(k, d[k])
        for k in ("rope_theta", "norm_eps"):
            if k in d:
                kw[k] = _as_float(k, d[k])
        for k in ("conv_bias", "block_auto_adjust_ff_dim"):
            if k in d:
                kw[k] = _as_bool(k, d[k])
        if "block_ffn_dim_multiplier" in d:
            v = d["block_ffn_dim_multiplier"]
            kw["block_ffn_dim_multiplier"] = None if v is None else _as_float("block_ffn_dim_multiplier", v)
        if "tie_embedding" in d:
            kw["tie_embedding"] = _as_bool("tie_embedding", d["tie_embedding"])
        elif "tie_word_embeddings" in d:
            kw["tie_embedding"] = _as_bool("tie_word_embeddings", d["tie_word_embeddings"])
        lt = d["layer_types"]
        if not isinstance(lt, (list, tuple)) or not all(isinstance(t, str) for t in lt):
            raise ConfigError("config key 'layer_types' must be a list of strings")
        kw["layer_types"] = list(lt)
        if "rope_style" in d:
            kw["rope_style"] = str(d["rope_style"])
        for k in ("max_position_embeddings", "bos_token_id", "eos_token_id", "pad_token_id"):
            if d.get(k) is not None:
                kw[k] = _as_int(k, d[k])
        if isinstance(d.get("architectures"), list) and d["architectures"]:
            kw["architectures"] = [str(a) for a in d["architectures"]]
        if "model_type" in d:
            kw["model_type"] = str(d["model_type"])
        return cls(**kw).validate()

    def to_dict(self) -> dict:
        return {f.name: getattr(self, f.name) for f in fields(self)}


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in {model_dir!r}")
    try:
        with open(path) as f:
            d = json.load(f)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: expected a JSON object")
    return d
