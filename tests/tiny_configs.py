"""Two tiny Qwen2 configurations that differ in every size and option."""

TINY_A = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 176, "vocab_size": 512, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "use_sliding_window": False,
    "max_position_embeddings": 256, "hidden_act": "silu",
}

TINY_B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1,
    "head_dim": 32, "intermediate_size": 256, "vocab_size": 1000, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "use_sliding_window": True,
    "sliding_window": 48, "max_window_layers": 1, "max_position_embeddings": 512, "hidden_act": "silu",
}

# a third shape for kernels: wider heads, group 7, sizes that are no power of two
TINY_C = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 224, "num_attention_heads": 7, "num_key_value_heads": 1,
    "head_dim": 48, "intermediate_size": 400, "vocab_size": 777, "rope_theta": 50000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "use_sliding_window": False,
    "max_position_embeddings": 1024, "hidden_act": "silu",
}

# Two shapes with the head sizes real checkpoints have (64 and 128), stored in bf16: a bfloat16 engine
# runs them through the kernels serving uses (tensor-core products, TMA-fed decode attention,
# tcgen05 prompt attention, the native launcher of the built-in block).
TINY_D = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 3, "hidden_size": 128, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 64, "intermediate_size": 320, "vocab_size": 408, "rope_theta": 20000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "use_sliding_window": True,
    "sliding_window": 48, "max_window_layers": 1, "max_position_embeddings": 512, "hidden_act": "silu",
}

TINY_E = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 256, "num_attention_heads": 2, "num_key_value_heads": 1,
    "head_dim": 128, "intermediate_size": 616, "vocab_size": 650, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "use_sliding_window": False,
    "max_position_embeddings": 1024, "hidden_act": "silu",
}

NORM_STD = {"A": 0.0, "B": 0.1, "C": 0.1, "D": 0.1, "E": 0.05}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E}
# how the test folders of a configuration are stored
STORE = {"A": "float32", "B": "float32", "C": "float32", "D": "bfloat16", "E": "bfloat16"}


def write_model(tmpdir, name, seed=1234, dtype="float32"):
    """Write a random model folder for configuration ``name`` and return its path."""
    import os
    from infero_b200.loading import write_random_model_dir
    d = os.path.join(str(tmpdir), f"tiny_{name}_{dtype}")
    if not os.path.exists(os.path.join(d, "model.safetensors")):
        write_random_model_dir(d, CONFIGS[name], seed=seed, dtype=dtype, std=0.02, norm_std=NORM_STD[name])
    return d
