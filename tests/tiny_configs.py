"""Tiny Qwen2-MoE configurations for the tests.  A and B are the two named by the build's
baseline description; they differ in every size and option.  C adds what A and B leave
out: a sliding window on some layers (said layer by layer), a sparse step of two, sizes that are no power of
two anywhere, a head size of 48, more query heads per group."""

import random

TINY_A = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "num_hidden_layers": 2, "hidden_size": 256, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 512,
    "num_experts": 8, "num_experts_per_tok": 2, "moe_intermediate_size": 128,
    "shared_expert_intermediate_size": 256, "norm_topk_prob": False,
    "decoder_sparse_step": 1, "mlp_only_layers": [], "vocab_size": 1024,
    "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "use_sliding_window": False, "sliding_window": 4096, "max_window_layers": 2,
    "hidden_act": "silu", "qkv_bias": True,
}

TINY_B = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "num_hidden_layers": 3, "hidden_size": 512, "num_attention_heads": 4,
    "num_key_value_heads": 1, "head_dim": 128, "intermediate_size": 768,
    "num_experts": 16, "num_experts_per_tok": 4, "moe_intermediate_size": 96,
    "shared_expert_intermediate_size": 384, "norm_topk_prob": True,
    "decoder_sparse_step": 1, "mlp_only_layers": [1], "vocab_size": 2003,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
    "use_sliding_window": False, "sliding_window": 4096, "max_window_layers": 3,
    "hidden_act": "silu", "qkv_bias": True,
}

TINY_C = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "num_hidden_layers": 4, "hidden_size": 200, "num_attention_heads": 6,
    "num_key_value_heads": 2, "head_dim": 48, "intermediate_size": 232,
    "num_experts": 6, "num_experts_per_tok": 3, "moe_intermediate_size": 72,
    "shared_expert_intermediate_size": 104, "norm_topk_prob": True,
    "decoder_sparse_step": 2, "mlp_only_layers": [], "vocab_size": 777,
    "rope_theta": 50000.0, "rms_norm_eps": 3e-6, "tie_word_embeddings": False,
    "use_sliding_window": True, "sliding_window": 40,
    "layer_types": ["full_attention", "sliding_attention", "sliding_attention", "full_attention"],
    "hidden_act": "silu", "qkv_bias": True,
}

# Awkward on purpose: a width and inner sizes that are not multiples of 8 (so the 16-byte-row
# kernels must step aside for the general ones), a single kv head for five query heads, one
# expert per token, a dense first layer, a tiny vocabulary, no `head_dim` key (derived), no bias.
TINY_D = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "num_hidden_layers": 2, "hidden_size": 100, "num_attention_heads": 5,
    "num_key_value_heads": 1, "head_dim": 32, "intermediate_size": 76,
    "num_experts": 4, "num_experts_per_tok": 1, "moe_intermediate_size": 36,
    "shared_expert_intermediate_size": 52, "norm_topk_prob": False,
    "decoder_sparse_step": 1, "mlp_only_layers": [0], "vocab_size": 131,
    "rope_theta": 777.0, "rms_norm_eps": 1e-4, "tie_word_embeddings": True,
    "use_sliding_window": False, "qkv_bias": False, "hidden_act": "silu",
}

CONFIGS = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 2), "D": (TINY_D, 3)}


def random_tokens(n: int, vocab: int, seed: int):
    r = random.Random(seed)
    return [r.randrange(vocab) for _ in range(n)]
