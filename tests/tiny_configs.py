"""Tiny configurations of the architecture used by the tests. They differ in every size and option:
layers, width, head counts and groups, head size, intermediate size (200 and 176 are no multiples
of 64), vocabulary, rope base and sections, the norms' eps, tied/untied head, and the window."""

ARCH = "Qwen2VLForConditionalGeneration"

TINY_A = {
    "architectures": [ARCH], "model_type": "qwen2_vl",
    "hidden_size": 64, "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 128, "vocab_size": 512, "rms_norm_eps": 1e-6,
    "rope_theta": 10000.0, "rope_scaling": {"type": "mrope", "mrope_section": [2, 3, 3]},
    "tie_word_embeddings": True, "hidden_act": "silu", "use_sliding_window": False,
    "image_token_id": 500, "vision_start_token_id": 499,
}
TINY_A_INIT = {"seed": 0, "std": 0.02, "norm_noise": 0.1}

TINY_B = {
    "architectures": [ARCH], "model_type": "qwen2_vl",
    "hidden_size": 96, "num_hidden_layers": 3, "num_attention_heads": 3, "num_key_value_heads": 1,
    "head_dim": 32, "intermediate_size": 200, "vocab_size": 1000, "rms_norm_eps": 1e-5,
    "rope_theta": 1000000.0, "rope_scaling": {"type": "mrope", "mrope_section": [4, 6, 6]},
    "tie_word_embeddings": False, "hidden_act": "silu", "use_sliding_window": False,
    "image_token_id": 990, "vision_start_token_id": 989,
}
TINY_B_INIT = {"seed": 1, "std": 0.02, "norm_noise": 0.0}

# Windowed variant: layer 0 sees all keys, layers 1..3 the last 20; head size 48, 6 heads in 3 groups.
TINY_C = {
    "architectures": [ARCH], "model_type": "qwen2_vl",
    "hidden_size": 80, "num_hidden_layers": 4, "num_attention_heads": 6, "num_key_value_heads": 3,
    "head_dim": 48, "intermediate_size": 176, "vocab_size": 777, "rms_norm_eps": 3e-6,
    "rope_theta": 50000.0, "rope_scaling": {"type": "mrope", "mrope_section": [10, 7, 7]},
    "tie_word_embeddings": True, "hidden_act": "silu",
    "use_sliding_window": True, "sliding_window": 20, "max_window_layers": 1,
}
TINY_C_INIT = {"seed": 5, "std": 0.05, "norm_noise": 0.05}

# Sizes that the decode step's weight-streaming kernels take (width and intermediate size multiples of 128) and the
# streaming decode attention (head size 64): the fast kernels of serving inside the engine, at a size a CPU can check.
TINY_D = {
    "architectures": [ARCH], "model_type": "qwen2_vl",
    "hidden_size": 256, "num_hidden_layers": 2, "num_attention_heads": 6, "num_key_value_heads": 2,
    "head_dim": 64, "intermediate_size": 384, "vocab_size": 640, "rms_norm_eps": 1e-6,
    "rope_theta": 10000.0, "rope_scaling": {"type": "mrope", "mrope_section": [8, 12, 12]},
    "tie_word_embeddings": False, "hidden_act": "silu", "use_sliding_window": False,
}
TINY_D_INIT = {"seed": 9, "std": 0.03, "norm_noise": 0.1}

ALL = {"tiny_a": (TINY_A, TINY_A_INIT), "tiny_b": (TINY_B, TINY_B_INIT), "tiny_c": (TINY_C, TINY_C_INIT),
       "tiny_d": (TINY_D, TINY_D_INIT)}
