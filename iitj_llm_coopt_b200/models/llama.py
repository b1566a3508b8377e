"""Llama-3 family: 'LlamaForCausalLM' in the registry.

Checkpoint tensor names as the reference reads them (engine/model.py:104-117):
model.embed_tokens.weight, model.norm.weight, lm_head.weight (untied models only),
model.layers.{i}.input_layernorm.weight, .post_attention_layernorm.weight,
.self_attn.{q,k,v,o}_proj.weight, .mlp.{gate,up,down}_proj.weight.
"""
from __future__ import annotations

import re

from ..config.llama import LlamaConfig
from ..config.registry import register_architecture
from .base import Architecture

_LAYER = re.compile(r"^layers\.(\d+)\.(.+)$")

_IN_LAYER = {
    ("mixer_norm.weight", None): "input_layernorm.weight",
    ("feed_forward_norm.weight", None): "post_attention_layernorm.weight",
    ("mixer.qkv", "q"): "self_attn.q_proj.weight",
    ("mixer.qkv", "k"): "self_attn.k_proj.weight",
    ("mixer.qkv", "v"): "self_attn.v_proj.weight",
    ("mixer.o", None): "self_attn.o_proj.weight",
    ("feed_forward.gate_up", "gate"): "mlp.gate_proj.weight",
    ("feed_forward.gate_up", "up"): "mlp.up_proj.weight",
    ("feed_forward.down", None): "mlp.down_proj.weight",
}
_TOP = {
    "embedding.weight": "model.embed_tokens.weight",
    "final_norm.weight": "model.norm.weight",
    "lm_head.weight": "lm_head.weight",
}


class LlamaForCausalLM(Architecture):
    name = "LlamaForCausalLM"
    config_class = LlamaConfig
    ignored_tensors = ("*.rotary_emb.inv_freq",)

    def checkpoint_name(self, path: str, piece: str | None) -> str:
        if path in _TOP and piece is None:
            return _TOP[path]
        m = _LAYER.match(path)
        if m and (m.group(2), piece) in _IN_LAYER:
            return f"model.layers.{m.group(1)}." + _IN_LAYER[(m.group(2), piece)]
        raise KeyError(f"LlamaForCausalLM has no checkpoint tensor for parameter {path!r} piece {piece!r}")

    def is_ignored(self, tensor_name: str, config) -> bool:
        # a tied model may still carry a copy of the head; the embedding is used (engine/model.py:106)
        if tensor_name == "lm_head.weight" and config.tie_word_embeddings:
            return True
        return super().is_ignored(tensor_name, config)


register_architecture(LlamaForCausalLM())
