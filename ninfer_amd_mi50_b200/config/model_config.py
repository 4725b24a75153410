"""Typed model configuration read from an architecture's own config.json keys.

The reference parses HuggingFace ``config.json`` in ``ModelConfig::parse``
(src/models/config.cpp:10-58): required integers ``vocab_size``, ``hidden_size``,
``num_hidden_layers``, ``num_attention_heads``, ``intermediate_size``; optional
``num_key_value_heads`` (= heads), ``head_dim`` (= hidden / heads), ``rope_theta``
(1e6), ``tie_word_embeddings`` (false); the MoE triple ``num_experts``,
``num_experts_per_tok``, ``moe_intermediate_size``.  It has none of the keys that make
the architecture Qwen2-MoE rather than Qwen3-MoE (``norm_topk_prob``,
``shared_expert_intermediate_size``, ``decoder_sparse_step``, ``mlp_only_layers``,
``qkv_bias``, ``use_sliding_window`` / ``sliding_window`` / ``max_window_layers``); those
are read here under their HuggingFace names.

Nothing in this module knows a size: every number comes from the dictionary.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, fields
from typing import Any, Dict, List, Optional, Tuple


class ConfigError(ValueError):
    """A config.json that cannot describe a runnable model."""


# --------------------------------------------------------------------------------------
# Part specifications: what a layer is made of.  `kind` selects the implementation in the
# part registries; `params` are that implementation's constructor arguments.
# --------------------------------------------------------------------------------------

@dataclass(frozen=True)
class PartSpec:
    kind: str
    params: Tuple[Tuple[str, Any], ...] = ()

    @staticmethod
    def make(kind: str, **params: Any) -> "PartSpec":
        return PartSpec(kind, tuple(sorted(params.items())))

    def as_dict(self) -> Dict[str, Any]:
        return dict(self.params)

    def __getitem__(self, key: str) -> Any:
        return dict(self.params)[key]


@dataclass(frozen=True)
class LayerSpec:
    """One block: which norm, mixer and feed-forward it is put together from."""
    arrangement: str            # key in the block registry, e.g. "pre_norm"
    norm: PartSpec
    mixer: PartSpec
    feed_forward: PartSpec
    prefix: str = ""            # tensor-name prefix of the layer, e.g. "model.layers.3."
    # tensor-name component of each part below the prefix, as (part, name) pairs:
    # ("norm1", "input_layernorm"), ("mixer", "self_attn"), ...
    names: Tuple[Tuple[str, str], ...] = ()

    def name_of(self, part: str) -> str:
        return self.prefix + dict(self.names)[part] + "."


@dataclass(frozen=True)
class LayerCall:
    """One entry of the execution order.

    `layer` is an index into the model's layers (a layer may be named twice);
    `cache` is the index of the cache slot its mixer reads (another layer's slot lets it
    read that layer's keys and values); `append` says whether this call writes the
    step's new entries into that slot.
    """
    layer: int
    cache: int
    append: bool = True


@dataclass(frozen=True)
class ModelPlan:
    """Architecture-neutral description that the generic decoder model is built from."""
    vocab_size: int
    hidden_size: int
    layers: Tuple[LayerSpec, ...]
    order: Tuple[LayerCall, ...]
    final_norm: PartSpec
    tie_word_embeddings: bool
    embedding_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm."
    head_name: str = "lm_head.weight"


# --------------------------------------------------------------------------------------
# Qwen2-MoE
# --------------------------------------------------------------------------------------

def _req_int(d: Dict[str, Any], key: str) -> int:
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key {key!r} is missing")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
        raise ConfigError(f"config.json: {key!r} must be an integer, got {v!r}")
    return int(v)


def _opt_int(d: Dict[str, Any], key: str, default: Optional[int]) -> Optional[int]:
    if key not in d or d[key] is None:
        return default
    return _req_int(d, key)


def _opt_bool(d: Dict[str, Any], key: str, default: bool) -> bool:
    if key not in d or d[key] is None:
        return default
    if not isinstance(d[key], bool):
        raise ConfigError(f"config.json: {key!r} must be true or false, got {d[key]!r}")
    return d[key]


def _opt_float(d: Dict[str, Any], key: str, default: float) -> float:
    if key not in d or d[key] is None:
        return default
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {key!r} must be a number, got {v!r}")
    return float(v)


@dataclass
class Qwen2MoeConfig:
    """``Qwen2MoeForCausalLM`` / ``model_type: "qwen2_moe"``.

    Keys shared with the reference parser keep its defaults (src/models/config.cpp:21-32);
    the Qwen2-MoE keys that the reference never reads take HuggingFace's meaning:
    a layer ``l`` is sparse iff ``l`` is not in ``mlp_only_layers``, ``num_experts > 0`` and
    ``(l + 1) % decoder_sparse_step == 0``; layers ``l >= max_window_layers`` use a window
    of ``sliding_window`` keys when ``use_sliding_window`` is set.
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
    max_position_embeddings: Optional[int] = None
    hidden_act: str = "silu"
    model_type: str = "qwen2_moe"

    ARCHITECTURE = "Qwen2MoeForCausalLM"

    # ---- reading ------------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "Qwen2MoeConfig":
        archs = d.get("architectures") or []
        arch = archs[0] if archs else cls.ARCHITECTURE
        heads = _req_int(d, "num_attention_heads")
        hidden = _req_int(d, "hidden_size")
        kv = _opt_int(d, "num_key_value_heads", heads)
        if "head_dim" in d and d["head_dim"] is not None:
            head_dim = _req_int(d, "head_dim")
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
            rope_theta = _opt_float(d, "rope_theta", 1000000.0)
        mlp_only = d.get("mlp_only_layers") or []
        if not isinstance(mlp_only, (list, tuple)) or any(
                isinstance(x, bool) or not isinstance(x, int) for x in mlp_only):
            raise ConfigError("config.json: mlp_only_layers must be a list of integers")
        cfg = cls(
            architecture=arch,
            vocab_size=_req_int(d, "vocab_size"),
            hidden_size=hidden,
            num_hidden_layers=_req_int(d, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=kv,
            head_dim=head_dim,
            intermediate_size=_req_int(d, "intermediate_size"),
            moe_intermediate_size=_opt_int(d, "moe_intermediate_size", 0),
            shared_expert_intermediate_size=_opt_int(d, "shared_expert_intermediate_size", 0),
            num_experts=_opt_int(d, "num_experts", 0),
            num_experts_per_tok=_opt_int(d, "num_experts_per_tok", 0),
            norm_topk_prob=_opt_bool(d, "norm_topk_prob", False),
            decoder_sparse_step=_opt_int(d, "decoder_sparse_step", 1),
            mlp_only_layers=list(mlp_only),
            qkv_bias=_opt_bool(d, "qkv_bias", True),
            rope_theta=rope_theta,
            rms_norm_eps=_opt_float(d, "rms_norm_eps", 1e-6),
            tie_word_embeddings=_opt_bool(d, "tie_word_embeddings", False),
            use_sliding_window=_opt_bool(d, "use_sliding_window", False),
            sliding_window=_opt_int(d, "sliding_window", None),
            max_window_layers=_opt_int(d, "max_window_layers", None),
            max_position_embeddings=_opt_int(d, "max_position_embeddings", None),
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
        if self.use_sliding_window:
            if self.sliding_window is None or self.sliding_window <= 0:
                bad("use_sliding_window is set but sliding_window is not a positive integer")
            if self.max_window_layers is None or self.max_window_layers < 0:
                bad("use_sliding_window is set but max_window_layers is missing")

    # ---- derived ------------------------------------------------------------------
    def layer_is_sparse(self, l: int) -> bool:
        return (l not in self.mlp_only_layers and self.num_experts > 0
                and (l + 1) % self.decoder_sparse_step == 0)

    def layer_window(self, l: int) -> Optional[int]:
        if self.use_sliding_window and l >= int(self.max_window_layers):
            return int(self.sliding_window)
        return None


def read_config_json(path: str) -> Dict[str, Any]:
    """Read ``config.json`` from a file or from the model folder that holds it."""
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    if not os.path.exists(path):
        raise ConfigError(f"no config.json at {path}")
    with open(path, "r", encoding="utf-8") as fh:
        try:
            d = json.load(fh)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return d
