"""Tiny Qwen3 configurations of the tests; they differ in every size and option.

A and B are the two tiny configurations of the build's baseline description (A: tied head,
group of 2, derived head size; B: one kv head for six query heads, a head size that is not
hidden / heads, sizes that are no power of two, untied head).  C adds what A and B lack: a
sliding window on some layers only, three kv heads, a head size of 48.
"""

from __future__ import annotations

TINY_A = {
    "architectures": ["Qwen3ForCausalLM"],
    "model_type": "qwen3",
    "vocab_size": 256,
    "hidden_size": 64,
    "intermediate_size": 128,
    "num_hidden_layers": 2,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "head_dim": 16,
    "max_position_embeddings": 128,
    "rms_norm_eps": 1e-6,
    "rope_theta": 10000.0,
    "tie_word_embeddings": True,
    "attention_bias": False,
    "hidden_act": "silu",
    "sliding_window": None,
    "use_sliding_window": False,
    "torch_dtype": "float32",
}

TINY_B = {
    "architectures": ["Qwen3ForCausalLM"],
    "model_type": "qwen3",
    "vocab_size": 384,
    "hidden_size": 96,
    "intermediate_size": 160,
    "num_hidden_layers": 3,
    "num_attention_heads": 6,
    "num_key_value_heads": 1,
    "head_dim": 32,
    "max_position_embeddings": 256,
    "rms_norm_eps": 1e-5,
    "rope_theta": 1000000.0,
    "tie_word_embeddings": False,
    "attention_bias": False,
    "hidden_act": "silu",
    "sliding_window": None,
    "use_sliding_window": False,
    "torch_dtype": "float32",
}

TINY_C = {
    "architectures": ["Qwen3ForCausalLM"],
    "model_type": "qwen3",
    "vocab_size": 331,
    "hidden_size": 80,
    "intermediate_size": 208,
    "num_hidden_layers": 4,
    "num_attention_heads": 6,
    "num_key_value_heads": 3,
    "head_dim": 48,
    "max_position_embeddings": 512,
    "rms_norm_eps": 3e-6,
    "rope_theta": 50000.0,
    "tie_word_embeddings": False,
    "attention_bias": False,
    "hidden_act": "silu",
    "sliding_window": 40,
    "use_sliding_window": True,
    "max_window_layers": 2,
    "layer_types": ["full_attention", "sliding_attention", "full_attention", "sliding_attention"],
    "torch_dtype": "float32",
}

SEEDS = {"A": 0, "B": 1, "C": 2}
PAGE_SIZES = {"A": 16, "B": 8, "C": 16}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C}
