"""The tiny configurations that the tests use: they differ in every size and option."""

TINY_A = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 128, "vocab_size": 256, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 256,
    "use_sliding_window": False, "sliding_window": None, "max_window_layers": 2,
    "hidden_act": "silu", "eos_token_id": None, "torch_dtype": "bfloat16",
}
TINY_A_PAGE = 16

TINY_B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 3, "hidden_size": 192, "num_attention_heads": 6, "num_key_value_heads": 1,
    "head_dim": 32, "intermediate_size": 320, "vocab_size": 503, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 512,
    "use_sliding_window": False, "sliding_window": None, "max_window_layers": 3,
    "hidden_act": "silu", "eos_token_id": None, "torch_dtype": "bfloat16",
}
TINY_B_PAGE = 8

# B with a window of 24 keys on its last two layers: two cache groups, pages returned while a
# request is still running. head_dim 48 here (a step of 16 that is no power of two).
TINY_W = dict(TINY_B, num_hidden_layers=3, hidden_size=144, num_attention_heads=3, num_key_value_heads=3,
              head_dim=48, intermediate_size=200, vocab_size=311, use_sliding_window=True,
              sliding_window=24, max_window_layers=1, rms_norm_eps=3e-6, rope_theta=50000.0)
TINY_W_PAGE = 8

# Heads of 64 and a prompt of a few hundred tokens reach the kernels that the large models run on: tcgen05
# GEMMs (also on pairs of SMs), tcgen05 prefill attention, TMA decode attention.
TINY_C = dict(TINY_A, num_hidden_layers=2, hidden_size=256, num_attention_heads=4, num_key_value_heads=2,
              head_dim=64, intermediate_size=640, vocab_size=1000, rope_theta=1000000.0, tie_word_embeddings=False,
              max_position_embeddings=1024)
TINY_C_PAGE = 16

ALL = {"A": (TINY_A, TINY_A_PAGE), "B": (TINY_B, TINY_B_PAGE), "W": (TINY_W, TINY_W_PAGE), "C": (TINY_C, TINY_C_PAGE)}
