"""Tiny Qwen3-dense configurations for the tests (config.json dicts) and the
random-weight recipe of each.  A and B differ in every size and option; C adds
a sliding window on its later layers, a qkv bias and a head size of 48."""

from __future__ import annotations

TINY_A = {
    "architectures": ["Qwen3ForCausalLM"],
    "num_hidden_layers": 2,
    "hidden_size": 64,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "head_dim": 16,
    "intermediate_size": 128,
    "vocab_size": 256,
    "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6,
    "attention_bias": False,
    "tie_word_embeddings": True,
    "use_sliding_window": False,
    "max_position_embeddings": 128,
    "torch_dtype": "float32",
}
TINY_A_INIT = dict(seed=0, std=0.02, norm_std=0.05)
TINY_A_PAGE = 4

TINY_B = {
    "architectures": ["Qwen3ForCausalLM"],
    "num_hidden_layers": 3,
    "hidden_size": 80,
    "num_attention_heads": 9,
    "num_key_value_heads": 3,
    "head_dim": 32,
    "intermediate_size": 176,
    "vocab_size": 331,
    "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-5,
    "attention_bias": False,
    "tie_word_embeddings": False,
    "use_sliding_window": False,
    "max_position_embeddings": 256,
    "torch_dtype": "float32",
}
TINY_B_INIT = dict(seed=2, std=0.03, norm_std=0.1)
TINY_B_PAGE = 16

TINY_C = {
    "architectures": ["Qwen3ForCausalLM"],
    "num_hidden_layers": 4,
    "hidden_size": 72,
    "num_attention_heads": 6,
    "num_key_value_heads": 1,
    "head_dim": 48,
    "intermediate_size": 200,
    "vocab_size": 509,
    "rope_theta": 50000.0,
    "rms_norm_eps": 3e-6,
    "attention_bias": True,
    "tie_word_embeddings": False,
    "use_sliding_window": True,
    "sliding_window": 24,
    "max_window_layers": 2,
    "max_position_embeddings": 512,
    "torch_dtype": "float32",
}
TINY_C_INIT = dict(seed=7, std=0.05, norm_std=0.2)
TINY_C_PAGE = 16

# D and E have the head sizes the bfloat16 tensor-core attention kernels take (64 and 128), so that the
# engine's choice of kernel is exercised end to end; E also has a sliding window on its last layer.
TINY_D = {
    "architectures": ["Qwen3ForCausalLM"],
    "num_hidden_layers": 2,
    "hidden_size": 192,
    "num_attention_heads": 6,
    "num_key_value_heads": 2,
    "head_dim": 64,
    "intermediate_size": 320,
    "vocab_size": 777,
    "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6,
    "attention_bias": False,
    "tie_word_embeddings": True,
    "use_sliding_window": False,
    "max_position_embeddings": 512,
    "torch_dtype": "float32",
}
TINY_D_INIT = dict(seed=11, std=0.04, norm_std=0.1)
TINY_D_PAGE = 16

TINY_E = {
    "architectures": ["Qwen3ForCausalLM"],
    "num_hidden_layers": 3,
    "hidden_size": 160,
    "num_attention_heads": 4,
    "num_key_value_heads": 4,
    "head_dim": 128,
    "intermediate_size": 256,
    "vocab_size": 1031,
    "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6,
    "attention_bias": False,
    "tie_word_embeddings": False,
    "use_sliding_window": True,
    "sliding_window": 40,
    "max_window_layers": 2,
    "max_position_embeddings": 512,
    "torch_dtype": "float32",
}
TINY_E_INIT = dict(seed=13, std=0.04, norm_std=0.1)
TINY_E_PAGE = 16

ALL = {
    "A": (TINY_A, TINY_A_INIT, TINY_A_PAGE),
    "B": (TINY_B, TINY_B_INIT, TINY_B_PAGE),
    "C": (TINY_C, TINY_C_INIT, TINY_C_PAGE),
    "D": (TINY_D, TINY_D_INIT, TINY_D_PAGE),
    "E": (TINY_E, TINY_E_INIT, TINY_E_PAGE),
}
