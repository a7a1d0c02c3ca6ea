"""Tiny Qwen3 configurations for tests.  A and B differ in every size and
option: layer count, hidden size (B's is no multiple of 64), head counts and
group (2 vs 6), head_dim (16 vs 32, with heads*head_dim != hidden in B),
intermediate size, vocabulary (B's is no multiple of 8), rope_theta, the norms'
eps, tied vs untied head, and the window (none vs sliding on some layers in C).
"""

TINY_A = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 192, "vocab_size": 512, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 256,
    "hidden_act": "silu", "attention_bias": False, "rope_scaling": None,
    "use_sliding_window": False, "sliding_window": None,
}

TINY_B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 6, "num_key_value_heads": 1,
    "head_dim": 32, "intermediate_size": 320, "vocab_size": 1000, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 512,
    "hidden_act": "silu", "attention_bias": False, "rope_scaling": None,
    "use_sliding_window": False, "sliding_window": None,
}

# sliding layers (1 and 3) beside full ones, a window that is no multiple of the
# page size, head_dim 48, group 3, a long context
TINY_C = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 4, "hidden_size": 80, "num_attention_heads": 3, "num_key_value_heads": 1,
    "head_dim": 48, "intermediate_size": 136, "vocab_size": 777, "rope_theta": 50000.0,
    "rms_norm_eps": 3e-6, "tie_word_embeddings": False, "max_position_embeddings": 2048,
    "hidden_act": "silu", "attention_bias": False, "rope_scaling": None,
    "use_sliding_window": True, "sliding_window": 37,
    "layer_types": ["full_attention", "sliding_attention", "full_attention", "sliding_attention"],
}

# widths that are no multiple of 8 (hidden 100, intermediate 100, vocabulary 333):
# no 16-byte unit fits their bfloat16 rows, so the tensor-core products hand over
# to the library product and nothing may assume they ran; five heads, no grouping
TINY_D = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 100, "num_attention_heads": 5, "num_key_value_heads": 5,
    "head_dim": 16, "intermediate_size": 100, "vocab_size": 333, "rope_theta": 7777.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 512,
    "hidden_act": "silu", "attention_bias": False, "rope_scaling": None,
    "use_sliding_window": False, "sliding_window": None,
}

ALL = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}
