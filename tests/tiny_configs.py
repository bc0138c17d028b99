"""Tiny Llama configurations for tests: config.json dicts that differ in every size and option."""

# 2 layers, head_dim = hidden / heads, tied embeddings, plain RoPE.
TINY_A = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "vocab_size": 256, "hidden_size": 64, "intermediate_size": 192, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "max_position_embeddings": 128,
    "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "tie_word_embeddings": True,
}

# 3 layers, explicit head_dim (heads * head_dim != hidden), 3:1 groups, llama3 RoPE scaling, untied head.
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "vocab_size": 384, "hidden_size": 96, "intermediate_size": 160, "num_hidden_layers": 3,
    "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 32, "max_position_embeddings": 256,
    "rms_norm_eps": 1e-6, "rope_theta": 500000.0, "tie_word_embeddings": False,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 32},
}

# 1 KV head, head_dim 48, a vocabulary that is no multiple of 8, partial rotary, linear scaling and the
# four multipliers the reference reads for every model_type.
TINY_C = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "vocab_size": 499, "hidden_size": 80, "intermediate_size": 112, "num_hidden_layers": 2,
    "num_attention_heads": 5, "num_key_value_heads": 1, "head_dim": 48, "max_position_embeddings": 512,
    "rms_norm_eps": 3e-5, "rope_theta": 25000.0, "tie_word_embeddings": True,
    "partial_rotary_factor": 0.5,
    "rope_scaling": {"type": "linear", "factor": 2.0},
    "embedding_multiplier": 3.0, "residual_multiplier": 0.5, "attention_multiplier": 0.2, "logits_scaling": 4.0,
}

# Sizes that defeat every vector path: a width and an inner width that are no multiple of 8, an odd vocabulary,
# one KV head for five heads, 4 layers, nothing optional given.
TINY_D = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "vocab_size": 301, "hidden_size": 100, "intermediate_size": 172, "num_hidden_layers": 4,
    "num_attention_heads": 5, "num_key_value_heads": 1, "head_dim": 16, "max_position_embeddings": 300,
    "rms_norm_eps": 1e-5,
}

# The head sizes that the tcgen05 prompt attention takes: 64 with 2:1 groups and llama3 scaling ...
TINY_E = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "vocab_size": 320, "hidden_size": 128, "intermediate_size": 208, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "max_position_embeddings": 512,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "tie_word_embeddings": True,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
}

# ... and 128 with three heads on one KV head, untied.
TINY_F = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "vocab_size": 272, "hidden_size": 72, "intermediate_size": 136, "num_hidden_layers": 2,
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 128, "max_position_embeddings": 512,
    "rms_norm_eps": 2e-6, "rope_theta": 10000.0, "tie_word_embeddings": False,
}

# Seven heads with a KV head each (no grouping), three layers, and the biases of all four attention projections,
# which the architecture takes when the file carries them (see OPTIONAL_TENSORS).
TINY_G = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "vocab_size": 333, "hidden_size": 112, "intermediate_size": 184, "num_hidden_layers": 3,
    "num_attention_heads": 7, "num_key_value_heads": 7, "max_position_embeddings": 256,
    "rms_norm_eps": 4e-6, "rope_theta": 1000000.0, "tie_word_embeddings": False,
}

# name -> (config, weight seed)
TINY = {"a": (TINY_A, 0), "b": (TINY_B, 2), "c": (TINY_C, 9), "d": (TINY_D, 4), "e": (TINY_E, 6), "f": (TINY_F, 8),
        "g": (TINY_G, 10)}

# name -> file names of tensors that the model folder carries although the configuration does not ask for them
OPTIONAL_TENSORS = {
    "g": [f"model.layers.{l}.self_attn.{p}_proj.bias" for l in range(TINY_G["num_hidden_layers"]) for p in "qkvo"],
}
