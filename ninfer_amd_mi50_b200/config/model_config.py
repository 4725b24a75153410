"""What every architecture's configuration is turned into: a plan of parts.

The reference has one ``ModelConfig`` struct for all its models
(src/models/config.h, src/models/config.cpp:10-58) and one model class that switches on
its flags.  Here an architecture's typed configuration lives with that architecture
(``models/<name>.py``); this module holds only what is neutral: the description of a
model as layers put together from parts (`PartSpec`, `LayerSpec`, `LayerCall`,
`ModelPlan`), the readers of single config.json keys that the typed configurations
share, and the reading of the file.  Nothing here knows a size or a key's meaning.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
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
# Readers of single keys, shared by the architectures' typed configurations
# --------------------------------------------------------------------------------------

def req_int(d: Dict[str, Any], key: str) -> int:
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key {key!r} is missing")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
        raise ConfigError(f"config.json: {key!r} must be an integer, got {v!r}")
    return int(v)


def opt_int(d: Dict[str, Any], key: str, default: Optional[int]) -> Optional[int]:
    if key not in d or d[key] is None:
        return default
    return req_int(d, key)


def opt_bool(d: Dict[str, Any], key: str, default: bool) -> bool:
    if key not in d or d[key] is None:
        return default
    if not isinstance(d[key], bool):
        raise ConfigError(f"config.json: {key!r} must be true or false, got {d[key]!r}")
    return d[key]


def opt_float(d: Dict[str, Any], key: str, default: float) -> float:
    if key not in d or d[key] is None:
        return default
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {key!r} must be a number, got {v!r}")
    return float(v)


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
