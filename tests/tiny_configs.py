"""The two tiny Qwen2 configurations the tests run on.  They differ in every size and
option: layers, width, head counts and group size, head size, intermediate size (B's is
no multiple of 64), vocabulary, rope_theta, rms_norm_eps, tied or untied output matrix,
page size and initial scale of the weights."""

TINY_A = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 256, "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "max_position_embeddings": 1024,
    "tie_word_embeddings": True, "use_sliding_window": False, "hidden_act": "silu",
    "initializer_range": 0.02, "eos_token_id": 255,
}

TINY_B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 384, "hidden_size": 96, "intermediate_size": 200, "num_hidden_layers": 3,
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-5, "max_position_embeddings": 2048,
    "tie_word_embeddings": False, "use_sliding_window": False, "hidden_act": "silu",
    "initializer_range": 0.05,
}

# Sizes the kernels' fast paths do not take: a head size that is no multiple of 16 (bfloat16 attention falls to the
# exact kernel, the rotation to the two-values-at-a-time kernel), an intermediate size that is no multiple of 8
# (gate and up rows are not interleaved), a hidden size that is no multiple of 16, pages of 4 tokens.
TINY_C = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 131, "hidden_size": 72, "intermediate_size": 100, "num_hidden_layers": 2,
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 24,
    "rope_theta": 50000.0, "rms_norm_eps": 1e-5, "max_position_embeddings": 512,
    "tie_word_embeddings": True, "use_sliding_window": False, "hidden_act": "silu",
    "initializer_range": 0.06,
}

PAGE_SIZE = {"A": 16, "B": 8, "C": 4}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C}
SEEDS = {"A": 1234, "B": 4321, "C": 77}
