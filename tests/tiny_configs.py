"""The tiny configurations of the tests.  They differ in every size and option:
layer count, width, head counts and group size, head size, feed-forward width,
vocabulary, rotary base, norm epsilon, tied or untied head, context length, and
window (none; none; a window on some layers)."""
from __future__ import annotations

import torch

TINY_A = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 64,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 128,
    "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 128, "hidden_act": "silu",
}
TINY_B = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 3, "hidden_size": 96,
    "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 32, "intermediate_size": 160,
    "vocab_size": 320, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    "max_position_embeddings": 256, "hidden_act": "silu",
}
# group of 3, head size 48 (a multiple of 16 that is no power of two), width 80,
# a window of 24 keys on layers 1 and 3, long enough context for far keys
TINY_C = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 4, "hidden_size": 80,
    "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 48, "intermediate_size": 112,
    "vocab_size": 304, "rope_theta": 50000.0, "rms_norm_eps": 3e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 1024, "hidden_act": "silu", "sliding_window": 24,
    "layer_types": ["full_attention", "sliding_attention", "full_attention", "sliding_attention"],
}
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C}


def plain_sizes(cfg) -> dict:
    """The plain implementation's size dict for a typed Qwen3 configuration."""
    return {"num_layers": cfg.num_hidden_layers, "num_heads": cfg.num_attention_heads,
            "num_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "eps": cfg.rms_norm_eps,
            "rope_theta": cfg.rope_theta, "tied": cfg.tie_word_embeddings,
            "windows": list(cfg.layer_windows)}
