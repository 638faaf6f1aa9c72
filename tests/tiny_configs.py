"""Tiny Qwen3 configurations for the tests.  A and B differ in every size and option: layers,
width, head counts and group size, head size, feed-forward width, vocabulary, rope base, eps,
tied or separate head.  C adds what A and B do not have: windowed layers, a layer that runs
twice and a run that reads another run's cache."""

TINY_A = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 64,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 160,
    "vocab_size": 512, "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 256, "hidden_act": "silu",
}
TINY_B = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 3, "hidden_size": 96,
    "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 32, "intermediate_size": 224,
    "vocab_size": 1000, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    "max_position_embeddings": 512, "hidden_act": "silu",
}
TINY_C = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 3, "hidden_size": 80,
    "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 48, "intermediate_size": 136,
    "vocab_size": 777, "rope_theta": 50000.0, "rms_norm_eps": 3e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 384, "hidden_act": "silu",
    "use_sliding_window": True, "sliding_window": 21,
    "layer_types": ["full_attention", "sliding_attention", "full_attention"],
    "layer_order": [0, 1, 2, 1, [2, 2]],
}

# D: head size 64 with pages of 16, which the tcgen05 attention kernel serves
TINY_D = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 128,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 192,
    "vocab_size": 600, "rope_theta": 300000.0, "rms_norm_eps": 2e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 640, "hidden_act": "silu",
}

# E: odd sizes everywhere (no vector loads, products that only the library takes), one query head per key head
TINY_E = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 119,
    "num_attention_heads": 5, "num_key_value_heads": 5, "head_dim": 80, "intermediate_size": 99,
    "vocab_size": 1131, "rope_theta": 777.0, "rms_norm_eps": 3e-4, "tie_word_embeddings": True,
    "max_position_embeddings": 320, "hidden_act": "silu",
}
