"""The tiny test configurations: two Llamas that differ in every size and option."""

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
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
    "tie_word_embeddings": True, "max_position_embeddings": 512, "eos_token_id": [1, 2],
}

# A third shape for the tensor-core paths: head_dim 64 and 128 heads are what the bfloat16
# attention kernels specialise on; widths that are no power of two.
TINY_C = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 192, "intermediate_size": 320, "num_hidden_layers": 2,
    "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 64,
    "vocab_size": 500, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 128},
    "tie_word_embeddings": False, "max_position_embeddings": 1024, "eos_token_id": 3,
}

TINY_D = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 256, "intermediate_size": 384, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 1, "head_dim": 128,
    "vocab_size": 384, "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "rope_scaling": None,
    "tie_word_embeddings": True, "max_position_embeddings": 2048, "eos_token_id": 3,
}

# Awkward sizes: a width and an inner size that are no multiple of 4 or 8, a prime vocabulary, plain multi-head
# attention (no grouping), query width different from the model width, one layer.
TINY_E = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 100, "intermediate_size": 90, "num_hidden_layers": 1,
    "num_attention_heads": 5, "num_key_value_heads": 5, "head_dim": 16,
    "vocab_size": 131, "rms_norm_eps": 2e-5, "rope_theta": 1000.0, "rope_scaling": None,
    "tie_word_embeddings": True, "max_position_embeddings": 300, "eos_token_id": 7,
}

CONFIGS = {"A": (TINY_A, 0, 16), "B": (TINY_B, 1, 8), "C": (TINY_C, 5, 16), "D": (TINY_D, 6, 16), "E": (TINY_E, 7, 4)}  # config, seed, page size
