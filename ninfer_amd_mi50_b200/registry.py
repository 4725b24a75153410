"""Registries: architecture name -> model plan, and part kind -> part class.

The reference has no registry: one ``Model`` class switches on ``is_moe`` /
``use_qk_norm`` and only logs the architecture string (src/models/config.cpp:34-56).
Here ``config.json``'s ``architectures[0]`` picks an entry that (1) parses the
architecture's own keys into a typed configuration and (2) turns that configuration
into a `ModelPlan`: a list of layers, each put together from registered parts, and
the order in which they run.  Adding an architecture is one `register_architecture`
call; adding a mixer, feed-forward, norm, position encoding or block arrangement is
one `register_part` call.  Neither needs a change to the engine.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict

from .config.model_config import ConfigError, ModelPlan, PartSpec

PART_CATEGORIES = ("norm", "position", "mixer", "feed_forward", "block")


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[Dict[str, Any]], Any]   # config.json dict -> typed config
    build_plan: Callable[[Any], ModelPlan]          # typed config -> ModelPlan


_ARCHITECTURES: Dict[str, Architecture] = {}
_PARTS: Dict[str, Dict[str, type]] = {c: {} for c in PART_CATEGORIES}


def register_architecture(name: str, parse_config, build_plan, *, replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = Architecture(name, parse_config, build_plan)


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def architecture_names():
    _load_builtin()
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    _load_builtin()
    if name not in _ARCHITECTURES:
        raise ConfigError(
            f"architecture {name!r} is not registered; registered: {sorted(_ARCHITECTURES)}")
    return _ARCHITECTURES[name]


def architecture_of(config_dict: Dict[str, Any]) -> Architecture:
    archs = config_dict.get("architectures")
    if not archs or not isinstance(archs, list) or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a non-empty list of names; "
                          f"registered: {architecture_names()}")
    return get_architecture(archs[0])


def register_part(category: str, kind: str, *, replace: bool = False):
    """Class decorator: make `cls` the implementation of `PartSpec(kind=...)`."""
    if category not in _PARTS:
        raise ValueError(f"unknown part category {category!r}; one of {PART_CATEGORIES}")

    def deco(cls):
        if kind in _PARTS[category] and not replace:
            raise ValueError(f"{category} part {kind!r} is already registered")
        _PARTS[category][kind] = cls
        return cls
    return deco


def unregister_part(category: str, kind: str) -> None:
    _PARTS[category].pop(kind, None)


def part_class(category: str, kind: str) -> type:
    _load_builtin()
    table = _PARTS[category]
    if kind not in table:
        raise ConfigError(f"no {category} part {kind!r}; registered: {sorted(table)}")
    return table[kind]


def build_part(category: str, spec: PartSpec, **extra: Any):
    """Instantiate the part named by `spec` with its parameters (+ `extra` context)."""
    return part_class(category, spec.kind)(**spec.as_dict(), **extra)


_loaded = False


def _load_builtin() -> None:
    """Import the built-in parts and models once, so that they register themselves."""
    global _loaded
    if _loaded:
        return
    _loaded = True
    from . import parts  # noqa: F401
    from . import models  # noqa: F401
