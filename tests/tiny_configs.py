"""The two tiny Qwen3 configurations that the tests run on, and a few variants.

They differ in every size and option: layers, width, head counts and groups,
head_dim (B: q width != hidden), intermediate size, vocabulary (B: odd), rope
base, norm eps, tied or untied head, maximum position and cache page size.
"""

from __future__ import annotations

TINY_A = {
    "architectures": ["Qwen3ForCausalLM"],
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 192, "vocab_size": 256, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 256,
}
TINY_A_INIT = {"seed": 0, "std": 0.02, "norm_std": 0.1}
TINY_A_PAGE = 16

TINY_B = {
    "architectures": ["Qwen3ForCausalLM"],
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 6, "num_key_value_heads": 1,
    "head_dim": 32, "intermediate_size": 160, "vocab_size": 317,
    "rope_parameters": {"rope_theta": 1000000.0, "rope_type": "default"},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 512,
}
TINY_B_INIT = {"seed": 1, "std": 0.05, "norm_std": 0.1}
TINY_B_PAGE = 8

# A third shape for the window: layer 0 sees everything, layers 1.. only the last 24 positions.
TINY_W = {
    "architectures": ["Qwen3ForCausalLM"],
    "num_hidden_layers": 3, "hidden_size": 80, "num_attention_heads": 5, "num_key_value_heads": 5,
    "head_dim": 48, "intermediate_size": 112, "vocab_size": 199, "rope_theta": 50000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 384,
    "use_sliding_window": True, "sliding_window": 24, "max_window_layers": 1,
}
TINY_W_INIT = {"seed": 2, "std": 0.04, "norm_std": 0.1}
TINY_W_PAGE = 16

# Head sizes that the tensor-core attention kernels take (64 and 128), with small and large groups.
TINY_C = {
    "architectures": ["Qwen3ForCausalLM"],
    "num_hidden_layers": 2, "hidden_size": 96, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 64, "intermediate_size": 144, "vocab_size": 211, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 512,
}
TINY_C_INIT = {"seed": 3, "std": 0.05, "norm_std": 0.1}
TINY_C_PAGE = 16

TINY_D = {
    "architectures": ["Qwen3ForCausalLM"],
    "num_hidden_layers": 2, "hidden_size": 160, "num_attention_heads": 8, "num_key_value_heads": 1,
    "head_dim": 128, "intermediate_size": 208, "vocab_size": 300, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 512,
    "use_sliding_window": True, "sliding_window": 40, "max_window_layers": 1,
}
TINY_D_INIT = {"seed": 4, "std": 0.04, "norm_std": 0.1}
TINY_D_PAGE = 32

# Sizes off every fast path: a width and an intermediate size that are no multiple of 8, a head
# size (80) that only the general attention kernel takes, a group of 5, an odd vocabulary.
TINY_O = {
    "architectures": ["Qwen3ForCausalLM"],
    "num_hidden_layers": 2, "hidden_size": 100, "num_attention_heads": 5, "num_key_value_heads": 1,
    "head_dim": 80, "intermediate_size": 150, "vocab_size": 333, "rope_theta": 20000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 320,
}
TINY_O_INIT = {"seed": 5, "std": 0.05, "norm_std": 0.1}
TINY_O_PAGE = 16

# A head size of 256 (the kernels' limit) and more query heads per key/value head (24) than the
# tensor-core decode kernel packs into one tile.
TINY_H = {
    "architectures": ["Qwen3ForCausalLM"],
    "num_hidden_layers": 1, "hidden_size": 128, "num_attention_heads": 24, "num_key_value_heads": 1,
    "head_dim": 256, "intermediate_size": 64, "vocab_size": 128, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 256,
}
TINY_H_INIT = {"seed": 6, "std": 0.03, "norm_std": 0.1}
TINY_H_PAGE = 16

ALL = {
    "A": (TINY_A, TINY_A_INIT, TINY_A_PAGE),
    "B": (TINY_B, TINY_B_INIT, TINY_B_PAGE),
    "W": (TINY_W, TINY_W_INIT, TINY_W_PAGE),
    "C": (TINY_C, TINY_C_INIT, TINY_C_PAGE),
    "D": (TINY_D, TINY_D_INIT, TINY_D_PAGE),
    "O": (TINY_O, TINY_O_INIT, TINY_O_PAGE),
    "H": (TINY_H, TINY_H_INIT, TINY_H_PAGE),
}

# The layer sizes of Qwen3-8B (hidden 4096, 32 query / 8 key-value heads of 128, intermediate 12288)
# with two layers and a small vocabulary: the shapes the serving kernels are tuned for.
LAYER_8B = {
    "architectures": ["Qwen3ForCausalLM"],
    "num_hidden_layers": 2, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "intermediate_size": 12288, "vocab_size": 2048, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 4096,
}

# The layer sizes of Qwen3-14B and Qwen3-32B with one layer and a small vocabulary: a width of
# 5120 (no power of two), groups of 5 and of 8 query heads, intermediate sizes 17408 and 25600.
LAYER_14B = {
    "architectures": ["Qwen3ForCausalLM"],
    "num_hidden_layers": 1, "hidden_size": 5120, "num_attention_heads": 40, "num_key_value_heads": 8,
    "head_dim": 128, "intermediate_size": 17408, "vocab_size": 1000, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 4096,
}
LAYER_32B = {
    "architectures": ["Qwen3ForCausalLM"],
    "num_hidden_layers": 1, "hidden_size": 5120, "num_attention_heads": 64, "num_key_value_heads": 8,
    "head_dim": 128, "intermediate_size": 25600, "vocab_size": 1000, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 4096,
}
