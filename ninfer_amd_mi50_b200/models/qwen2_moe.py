"""Qwen2-MoE (``Qwen2MoeForCausalLM``): its config.json keys, and configuration -> plan of parts.

The reference parses HuggingFace ``config.json`` in ``ModelConfig::parse``
(src/models/config.cpp:10-58): required integers ``vocab_size``, ``hidden_size``,
``num_hidden_layers``, ``num_attention_heads``, ``intermediate_size``; optional
``num_key_value_heads`` (= heads), ``head_dim`` (= hidden / heads), ``rope_theta``
(1e6), ``tie_word_embeddings`` (false); the MoE triple ``num_experts``,
``num_experts_per_tok``, ``moe_intermediate_size``.  It has none of the keys that make
the architecture Qwen2-MoE rather than Qwen3-MoE (``norm_topk_prob``,
``shared_expert_intermediate_size``, ``decoder_sparse_step``, ``mlp_only_layers``,
``qkv_bias``, ``use_sliding_window`` / ``sliding_window`` / ``layer_types``); those are read
here under their HuggingFace names.  No size stands in this file: every number comes from
the dictionary.

The reference lists ``qwen2_moe`` as supported (README.md:28-30; ``is_moe`` in
src/models/config.cpp:36) and names tensors as in src/models/model.hip:487-512, 530-532,
559, 576, 586-587, 619.  The q/k/v biases, per-expert tensors
``mlp.experts.{e}.{gate,up,down}_proj.weight``, ``mlp.shared_expert.*`` and
``mlp.shared_expert_gate.weight`` are this architecture's own.
"""

from __future__ import annotations

from dataclasses import dataclass, field, fields
from typing import Any, Dict, List, Optional

from ..config.model_config import (ConfigError, LayerCall, LayerSpec, ModelPlan, PartSpec, opt_bool,
                                   opt_float, opt_int, read_config_json, req_int)
from ..registry import register_architecture

LAYER_TYPES = ("full_attention", "sliding_attention")

_NAMES = (("norm1", "input_layernorm"), ("mixer", "self_attn"),
          ("norm2", "post_attention_layernorm"), ("feed_forward", "mlp"))


@dataclass
class Qwen2MoeConfig:
    """``Qwen2MoeForCausalLM`` / ``model_type: "qwen2_moe"``.

    Keys shared with the reference parser keep its defaults (src/models/config.cpp:21-32);
    the Qwen2-MoE keys that the reference never reads take the meaning of the published
    checkpoints' config.json: a layer ``l`` is sparse iff ``l`` is not in ``mlp_only_layers``,
    ``num_experts > 0`` and ``(l + 1) % decoder_sparse_step == 0``.

    Which layers attend through a window is said layer by layer, by ``layer_types``: a list
    with one of ``"full_attention"`` / ``"sliding_attention"`` per layer; a sliding layer sees
    the last ``sliding_window`` keys.  ``use_sliding_window: true`` without ``layer_types`` is
    refused: exporters have derived the windowed layers from ``max_window_layers`` by
    different rules, the reference has no window at all, and a guess would give wrong logits
    without any error.  No published Qwen2-MoE checkpoint sets the flag.
    """

    architecture: str
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    moe_intermediate_size: int
    shared_expert_intermediate_size: int
    num_experts: int
    num_experts_per_tok: int
    norm_topk_prob: bool = False
    decoder_sparse_step: int = 1
    mlp_only_layers: List[int] = field(default_factory=list)
    qkv_bias: bool = True
    rope_theta: float = 1000000.0
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = False
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None
    layer_types: Optional[List[str]] = None
    max_position_embeddings: Optional[int] = None
    hidden_act: str = "silu"
    model_type: str = "qwen2_moe"

    ARCHITECTURE = "Qwen2MoeForCausalLM"

    # ---- reading ------------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "Qwen2MoeConfig":
        archs = d.get("architectures") or []
        arch = archs[0] if archs else cls.ARCHITECTURE
        heads = req_int(d, "num_attention_heads")
        hidden = req_int(d, "hidden_size")
        kv = opt_int(d, "num_key_value_heads", heads)
        if "head_dim" in d and d["head_dim"] is not None:
            head_dim = req_int(d, "head_dim")
        else:
            if heads <= 0 or hidden % heads:
                raise ConfigError(
                    f"config.json: head_dim is absent and hidden_size={hidden} is not a "
                    f"multiple of num_attention_heads={heads}")
            head_dim = hidden // heads
        # rope_theta may sit at the top level or inside rope_parameters (newer exports)
        rope_theta = None
        rp = d.get("rope_parameters")
        if isinstance(rp, dict):
            if rp.get("rope_type", "default") not in ("default", None):
                raise ConfigError(
                    f"config.json: rope_type {rp.get('rope_type')!r} is not supported "
                    "(only unscaled rotary embedding)")
            if rp.get("rope_theta") is not None:
                rope_theta = float(rp["rope_theta"])
        rs = d.get("rope_scaling")
        if isinstance(rs, dict) and rs.get("rope_type", rs.get("type", "default")) not in (
                "default", None):
            raise ConfigError(
                f"config.json: rope_scaling {rs!r} is not supported (only unscaled rotary "
                "embedding)")
        if rope_theta is None:
            rope_theta = opt_float(d, "rope_theta", 1000000.0)
        mlp_only = d.get("mlp_only_layers") or []
        if not isinstance(mlp_only, (list, tuple)) or any(
                isinstance(x, bool) or not isinstance(x, int) for x in mlp_only):
            raise ConfigError("config.json: mlp_only_layers must be a list of integers")
        layer_types = d.get("layer_types")
        if layer_types is not None and (not isinstance(layer_types, (list, tuple)) or any(
                not isinstance(x, str) for x in layer_types)):
            raise ConfigError("config.json: layer_types must be a list of strings")
        cfg = cls(
            architecture=arch,
            vocab_size=req_int(d, "vocab_size"),
            hidden_size=hidden,
            num_hidden_layers=req_int(d, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=kv,
            head_dim=head_dim,
            intermediate_size=req_int(d, "intermediate_size"),
            moe_intermediate_size=opt_int(d, "moe_intermediate_size", 0),
            shared_expert_intermediate_size=opt_int(d, "shared_expert_intermediate_size", 0),
            num_experts=opt_int(d, "num_experts", 0),
            num_experts_per_tok=opt_int(d, "num_experts_per_tok", 0),
            norm_topk_prob=opt_bool(d, "norm_topk_prob", False),
            decoder_sparse_step=opt_int(d, "decoder_sparse_step", 1),
            mlp_only_layers=list(mlp_only),
            qkv_bias=opt_bool(d, "qkv_bias", True),
            rope_theta=rope_theta,
            rms_norm_eps=opt_float(d, "rms_norm_eps", 1e-6),
            tie_word_embeddings=opt_bool(d, "tie_word_embeddings", False),
            use_sliding_window=opt_bool(d, "use_sliding_window", False),
            sliding_window=opt_int(d, "sliding_window", None),
            max_window_layers=opt_int(d, "max_window_layers", None),
            layer_types=list(layer_types) if layer_types is not None else None,
            max_position_embeddings=opt_int(d, "max_position_embeddings", None),
            hidden_act=d.get("hidden_act", "silu") or "silu",
            model_type=d.get("model_type", "qwen2_moe") or "qwen2_moe",
        )
        cfg.validate()
        return cfg

    @classmethod
    def from_file(cls, path: str) -> "Qwen2MoeConfig":
        return cls.from_dict(read_config_json(path))

    # ---- writing ------------------------------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architectures": [self.architecture]}
        for f in fields(self):
            if f.name == "architecture":
                continue
            v = getattr(self, f.name)
            if v is None:
                continue
            out[f.name] = list(v) if isinstance(v, list) else v
        return out

    # ---- checks -------------------------------------------------------------------
    def validate(self) -> None:
        def bad(msg: str) -> None:
            raise ConfigError("config.json: " + msg)

        for name in ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
                     "num_key_value_heads", "head_dim", "intermediate_size"):
            if getattr(self, name) <= 0:
                bad(f"{name} must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads:
            bad(f"num_attention_heads={self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads={self.num_key_value_heads}")
        if self.head_dim % 2:
            bad(f"head_dim={self.head_dim} must be even for the rotary embedding")
        if self.rms_norm_eps <= 0:
            bad(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if self.rope_theta <= 0:
            bad(f"rope_theta must be positive, got {self.rope_theta}")
        if self.hidden_act != "silu":
            bad(f"hidden_act {self.hidden_act!r} is not supported (silu only)")
        if self.decoder_sparse_step < 1:
            bad(f"decoder_sparse_step must be >= 1, got {self.decoder_sparse_step}")
        for l in self.mlp_only_layers:
            if not 0 <= l < self.num_hidden_layers:
                bad(f"mlp_only_layers names layer {l}, but there are "
                    f"{self.num_hidden_layers} layers")
        if self.num_experts < 0 or self.shared_expert_intermediate_size < 0:
            bad("num_experts and shared_expert_intermediate_size must not be negative")
        if any(self.layer_is_sparse(l) for l in range(self.num_hidden_layers)):
            if self.moe_intermediate_size <= 0:
                bad("sparse layers need moe_intermediate_size > 0")
            if not 1 <= self.num_experts_per_tok <= self.num_experts:
                bad(f"num_experts_per_tok={self.num_experts_per_tok} must lie in "
                    f"[1, num_experts={self.num_experts}]")
        if self.layer_types is not None:
            if len(self.layer_types) != self.num_hidden_layers:
                bad(f"layer_types has {len(self.layer_types)} entries for "
                    f"{self.num_hidden_layers} layers")
            for l, t in enumerate(self.layer_types):
                if t not in LAYER_TYPES:
                    bad(f"layer_types[{l}] = {t!r}; known: {list(LAYER_TYPES)}")
        sliding = self.layer_types is not None and "sliding_attention" in self.layer_types
        if sliding and not self.use_sliding_window:
            bad("layer_types names a sliding_attention layer but use_sliding_window is not true")
        if self.use_sliding_window:
            if self.sliding_window is None or self.sliding_window <= 0:
                bad("use_sliding_window is set but sliding_window is not a positive integer")
            if self.layer_types is None:
                bad("use_sliding_window is set but layer_types is absent: which layers use the "
                    "window must be given layer by layer (\"full_attention\" / "
                    "\"sliding_attention\"); max_window_layers alone is read differently by "
                    "different exporters and is not guessed at")

    # ---- derived ------------------------------------------------------------------
    def layer_is_sparse(self, l: int) -> bool:
        return (l not in self.mlp_only_layers and self.num_experts > 0
                and (l + 1) % self.decoder_sparse_step == 0)

    def layer_window(self, l: int) -> Optional[int]:
        if (self.use_sliding_window and self.layer_types is not None
                and self.layer_types[l] == "sliding_attention"):
            return int(self.sliding_window)
        return None


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
