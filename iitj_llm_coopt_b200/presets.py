"""Named model shapes: the config.json of a model folder, as data, for runs with random weights.

Each entry holds exactly the keys a config.json of that model would hold; nothing in the engine reads a size
from here (the typed configuration is built from the dict as it would be from a file).  The benchmark, the
command line (`--shape NAME --random-seed S` in place of `--model DIR`) and the tests use them.
"""
from __future__ import annotations

import copy

_LLAMA3_SCALING = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                   "original_max_position_embeddings": 8192}

LLAMA_3_1_8B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 4096, "intermediate_size": 14336, "num_hidden_layers": 32,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 128256,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "rope_scaling": dict(_LLAMA3_SCALING),
    "tie_word_embeddings": False, "max_position_embeddings": 131072, "eos_token_id": 128001,
}
LLAMA_3_2_3B = dict(LLAMA_3_1_8B, hidden_size=3072, intermediate_size=8192, num_hidden_layers=28, num_attention_heads=24,
                    head_dim=128, tie_word_embeddings=True, rope_scaling=dict(_LLAMA3_SCALING, factor=32.0))
LLAMA_3_2_1B = dict(LLAMA_3_2_3B, hidden_size=2048, num_hidden_layers=16, num_attention_heads=32, head_dim=64)

# the two tiny test shapes (they differ in every size and option)
TINY_A = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 64, "intermediate_size": 176, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "vocab_size": 256, "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "rope_scaling": None,
    "tie_word_embeddings": False, "max_position_embeddings": 256, "eos_token_id": 0,
}
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 96, "intermediate_size": 256, "num_hidden_layers": 3,
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32,
    "vocab_size": 320, "rms_norm_eps": 1e-6, "rope_theta": 500000.0,
    "rope_scaling": dict(_LLAMA3_SCALING, original_max_position_embeddings=64),
    "tie_word_embeddings": True, "max_position_embeddings": 512, "eos_token_id": [1, 2],
}
# a small shape for trying a benchmark out in seconds
TOY = dict(LLAMA_3_1_8B, hidden_size=512, intermediate_size=1408, num_hidden_layers=2, num_attention_heads=8,
           num_key_value_heads=2, head_dim=64, vocab_size=4096)

# name -> (label used in reports, config.json dict)
SHAPES = {
    "8b": ("llama-3.1-8b-shape-random", LLAMA_3_1_8B),
    "3b": ("llama-3.2-3b-shape-random", LLAMA_3_2_3B),
    "1b": ("llama-3.2-1b-shape-random", LLAMA_3_2_1B),
    "tinyA": ("llama-tiny-a-shape-random", TINY_A),
    "tinyB": ("llama-tiny-b-shape-random", TINY_B),
    "toy": ("llama-toy-shape-random", TOY),
}


def shape_config(name: str) -> dict:
    """A fresh copy of the config.json dict of shape `name`."""
    if name not in SHAPES:
        raise KeyError(f"shape {name!r} is not known; known: {', '.join(sorted(SHAPES))}")
    return copy.deepcopy(SHAPES[name][1])
