"""Qwen2-MoE (``Qwen2MoeForCausalLM``): configuration -> plan of parts.

The reference lists ``qwen2_moe`` as supported (README.md:28-30; ``is_moe`` in
src/models/config.cpp:36) and names tensors as in src/models/model.hip:487-512, 530-532,
559, 576, 586-587, 619.  The q/k/v biases, per-expert tensors
``mlp.experts.{e}.{gate,up,down}_proj.weight``, ``mlp.shared_expert.*`` and
``mlp.shared_expert_gate.weight`` are this architecture's own.
"""

from __future__ import annotations

from ..config.model_config import LayerCall, LayerSpec, ModelPlan, PartSpec, Qwen2MoeConfig
from ..registry import register_architecture

_NAMES = (("norm1", "input_layernorm"), ("mixer", "self_attn"),
          ("norm2", "post_attention_layernorm"), ("feed_forward", "mlp"))


def build_plan(cfg: Qwen2MoeConfig) -> ModelPlan:
    norm = PartSpec.make("rms_norm", size=cfg.hidden_size, eps=cfg.rms_norm_eps)
    position = PartSpec.make("rotary_half_split", head_dim=cfg.head_dim, theta=cfg.rope_theta)
    layers = []
    for l in range(cfg.num_hidden_layers):
        mixer = PartSpec.make(
            "paged_gqa_attention", hidden_size=cfg.hidden_size,
            num_heads=cfg.num_attention_heads, num_kv_heads=cfg.num_key_value_heads,
            head_dim=cfg.head_dim, qkv_bias=cfg.qkv_bias, position=position,
            window=cfg.layer_window(l))
        if cfg.layer_is_sparse(l):
            ffn = PartSpec.make(
                "sparse_moe_swiglu", hidden_size=cfg.hidden_size, num_experts=cfg.num_experts,
                top_k=cfg.num_experts_per_tok, norm_topk_prob=cfg.norm_topk_prob,
                moe_intermediate_size=cfg.moe_intermediate_size,
                shared_intermediate_size=cfg.shared_expert_intermediate_size)
        else:
            ffn = PartSpec.make("dense_swiglu", hidden_size=cfg.hidden_size,
                                intermediate_size=cfg.intermediate_size)
        layers.append(LayerSpec("pre_norm", norm, mixer, ffn,
                                prefix=f"model.layers.{l}.", names=_NAMES))
    order = tuple(LayerCall(l, l, True) for l in range(cfg.num_hidden_layers))
    return ModelPlan(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
                     layers=tuple(layers), order=order, final_norm=norm,
                     tie_word_embeddings=cfg.tie_word_embeddings)


register_architecture(Qwen2MoeConfig.ARCHITECTURE, Qwen2MoeConfig.from_dict, build_plan)
