"""Typed configuration of the Llama-3 family, read from the architecture's config.json keys.

The keys are the ones the reference engine reads (engine/model.py:28-48): hidden_size,
intermediate_size, num_hidden_layers, num_attention_heads, num_key_value_heads, head_dim
(default hidden_size // num_attention_heads), vocab_size, rms_norm_eps, rope_theta,
rope_scaling, tie_word_embeddings, eos_token_id and max_position_embeddings.  The reference
fills a missing key with None and fails later; here a missing key is an error at once, and
options the reference silently ignores but that would change the result (attention_bias,
mlp_bias, a hidden_act other than silu) are refused.
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field

from .errors import ConfigError
from .specs import (CacheNeed, FeedForwardSpec, LayerCall, LayerSpec, MixerSpec, ModelSpec,
                    NormSpec, PositionSpec)


_REQUIRED = ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
             "vocab_size", "rms_norm_eps", "max_position_embeddings")


@dataclass
class LlamaConfig:
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: dict | None
    tie_word_embeddings: bool
    eos_token_id: int | list | None
    max_position_embeddings: int
    architectures: list = field(default_factory=lambda: ["LlamaForCausalLM"])

    # ---- reading -------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, c: dict) -> "LlamaConfig":
        c = dict(c)
        missing = [k for k in _REQUIRED if c.get(k) is None]
        if missing:
            raise ConfigError(f"config.json lacks required key(s): {', '.join(missing)}")
        # newer exporters nest the rotary constants under "rope_parameters"
        rp = c.get("rope_parameters") or {}
        if c.get("rope_theta") is None:
            if rp.get("rope_theta") is None:
                raise ConfigError("config.json lacks required key(s): rope_theta")
            c["rope_theta"] = rp["rope_theta"]
        if c.get("rope_scaling") is None and rp.get("rope_type", "default") != "default":
            c["rope_scaling"] = {k: v for k, v in rp.items() if k != "rope_theta"}
        if c.get("attention_bias") or c.get("mlp_bias"):
            raise ConfigError("attention_bias / mlp_bias = true is not supported (no bias terms)")
        act = c.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act {act!r} is not supported (only 'silu')")
        heads = int(c["num_attention_heads"])
        cfg = cls(
            hidden_size=int(c["hidden_size"]),
            intermediate_size=int(c["intermediate_size"]),
            num_hidden_layers=int(c["num_hidden_layers"]),
            num_attention_heads=heads,
            num_key_value_heads=int(c.get("num_key_value_heads") or heads),
            head_dim=int(c.get("head_dim") or int(c["hidden_size"]) // heads),
            vocab_size=int(c["vocab_size"]),
            rms_norm_eps=float(c["rms_norm_eps"]),
            rope_theta=float(c["rope_theta"]),
            rope_scaling=dict(c["rope_scaling"]) if c.get("rope_scaling") else None,
            tie_word_embeddings=bool(c.get("tie_word_embeddings", False)),
            eos_token_id=c.get("eos_token_id"),
            max_position_embeddings=int(c["max_position_embeddings"]),
            architectures=list(c.get("architectures") or ["LlamaForCausalLM"]),
        )
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "LlamaConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path, encoding="utf-8") as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> dict:
        d = asdict(self)
        d["model_type"] = "llama"
        d["hidden_act"] = "silu"
        return d

    # ---- checks --------------------------------------------------------------------------
    def validate(self) -> None:
        for name in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                     "num_key_value_heads", "head_dim", "vocab_size", "max_position_embeddings"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                              f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 16 or self.head_dim > 256:
            raise ConfigError(f"head_dim {self.head_dim} is not supported: the attention kernels take "
                              f"multiples of 16 up to 256")
        if not self.rms_norm_eps > 0:
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")
        rs = self.rope_scaling
        if rs:
            kind = rs.get("rope_type", rs.get("type"))
            if kind == "llama3":
                lacking = [k for k in ("factor", "low_freq_factor", "high_freq_factor",
                                       "original_max_position_embeddings") if k not in rs]
                if lacking:
                    raise ConfigError(f"rope_scaling (llama3) lacks {', '.join(lacking)}")
                if rs["high_freq_factor"] == rs["low_freq_factor"]:
                    raise ConfigError("rope_scaling: high_freq_factor equals low_freq_factor")
            elif kind not in (None, "default"):
                raise ConfigError(f"rope_scaling type {kind!r} is not supported (only 'llama3')")

    # ---- derived -------------------------------------------------------------------------
    @property
    def eos_ids(self) -> tuple:
        e = self.eos_token_id
        if e is None:
            return ()
        return tuple(e) if isinstance(e, (list, tuple)) else (int(e),)

    def kv_bytes_per_token(self, itemsize: int = 2) -> int:
        """Bytes of keys and values one token occupies over all layers (engine/model.py:50-51)."""
        return 2 * self.num_hidden_layers * self.num_key_value_heads * self.head_dim * itemsize

    def model_spec(self) -> ModelSpec:
        """Llama as data: L identical pre-norm blocks of GQA attention and a SwiGLU feed-forward."""
        rs = self.rope_scaling or {}
        kind = rs.get("rope_type", rs.get("type"))
        scaling = tuple(sorted(rs.items())) if kind == "llama3" else ()
        pos = PositionSpec(kind="rope", head_dim=self.head_dim, rotary_dim=self.head_dim,
                           theta=self.rope_theta, scaling=scaling,
                           max_position=self.max_position_embeddings)
        mixer = MixerSpec(kind="attention", width=self.hidden_size, heads=self.num_attention_heads,
                          kv_heads=self.num_key_value_heads, head_dim=self.head_dim, window=0,
                          softmax_scale=0.0, position=pos)
        ff = FeedForwardSpec(kind="swiglu", width=self.hidden_size, inner=self.intermediate_size,
                             activation="silu")
        norm = NormSpec(kind="rmsnorm", width=self.hidden_size, eps=self.rms_norm_eps)
        layer = LayerSpec.of("prenorm", mixer_norm=norm, mixer=mixer, feed_forward_norm=norm, feed_forward=ff)
        n = self.num_hidden_layers
        return ModelSpec(width=self.hidden_size, vocab=self.vocab_size,
                         layers=tuple(layer for _ in range(n)),
                         order=tuple(LayerCall(layer=i, cache=i, write=True) for i in range(n)),
                         final_norm=norm, tie_embeddings=self.tie_word_embeddings,
                         max_position=self.max_position_embeddings, eos_token_ids=self.eos_ids)
