"""Tiny Qwen3 configurations of the tests; they differ in every size and option."""
import copy

# 2 layers, head size 16, group 2, tied head, theta 1e4, eps 1e-6, no window; cache pages of 4
TINY_A = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 64,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 128,
    "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 128, "torch_dtype": "float32",
}
A_SEED, A_STD, A_PAGE = 0, 0.02, 4

# 3 layers, head size 32 (q width 256 != hidden 96), group 4, untied head, vocabulary 500, theta 1e6,
# eps 1e-5; cache pages of 8
TINY_B = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 3, "hidden_size": 96,
    "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 32, "intermediate_size": 160,
    "vocab_size": 500, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    "max_position_embeddings": 256, "torch_dtype": "float32",
}
B_SEED, B_STD, B_PAGE = 1, 0.05, 8

# 4 layers, head size 48 (no power of two), 6 heads in 3 groups of 2, hidden 80, vocabulary 301,
# layers 1..3 read a window of 24 keys (layer 0 all keys): two cache groups; pages of 16
TINY_C = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 4, "hidden_size": 80,
    "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 48, "intermediate_size": 208,
    "vocab_size": 301, "rope_theta": 50000.0, "rms_norm_eps": 3e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 512, "torch_dtype": "float32",
    "use_sliding_window": True, "sliding_window": 24, "max_window_layers": 1,
}
C_SEED, C_STD, C_PAGE = 2, 0.04, 16

# head size 64: the tensor-core attention kernels of the bfloat16 path; layer 1 reads a window of 40 keys
TINY_D = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 128,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 192,
    "vocab_size": 333, "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 1024, "torch_dtype": "float32",
    "use_sliding_window": True, "sliding_window": 40, "max_window_layers": 1,
}
D_SEED, D_STD, D_PAGE = 3, 0.03, 16

# head size 128, one kv head for 8 q heads, pages of 32
TINY_E = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 96,
    "num_attention_heads": 8, "num_key_value_heads": 1, "head_dim": 128, "intermediate_size": 128,
    "vocab_size": 260, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    "max_position_embeddings": 1024, "torch_dtype": "float32",
}
E_SEED, E_STD, E_PAGE = 4, 0.03, 32

ALL = {
    "A": (TINY_A, A_SEED, A_STD, A_PAGE),
    "B": (TINY_B, B_SEED, B_STD, B_PAGE),
    "C": (TINY_C, C_SEED, C_STD, C_PAGE),
    "D": (TINY_D, D_SEED, D_STD, D_PAGE),
    "E": (TINY_E, E_SEED, E_STD, E_PAGE),
}


def get(name):
    cfg, seed, std, page = ALL[name]
    return copy.deepcopy(cfg), seed, std, page
