"""Random-weights mode: write a model folder from a configuration and a seed.

The folder holds ``config.json`` and ``model.safetensors`` with exactly the tensors the
architecture's parts declare, under their checkpoint names, so that it loads through
the same path as a real checkpoint.  The reference has no such mode.
"""

from __future__ import annotations

import json
import os
from typing import Any, Dict

import torch

from ..config.model_config import ConfigError
from ..registry import architecture_of
from .loader import RandomSource
from .safetensors_io import write_safetensors

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def write_random_model(config: Dict[str, Any], seed: int, out_dir: str,
                       store_dtype: str = "bfloat16") -> str:
    """`config` is a config.json dictionary (it must name its architecture)."""
    from ..parts.model import DecoderModel
    if store_dtype not in _STORE:
        raise ConfigError(f"store_dtype must be one of {sorted(_STORE)}")
    arch = architecture_of(config)
    typed = arch.parse_config(config)
    model = DecoderModel(arch.build_plan(typed))
    specs = model.tensor_specs()
    src = RandomSource(specs, seed, gen_device="cpu")
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(config, fh, indent=1)

    def items():
        seen = set()
        for s in specs:
            if s.name in seen:
                continue
            seen.add(s.name)
            # every value is a bfloat16 number; stored widened when float32 is asked for
            yield s.name, src.generate(s.name, _STORE[store_dtype])

    write_safetensors(os.path.join(out_dir, "model.safetensors"), items(),
                      metadata={"format": "pt", "seed": str(seed)})
    return out_dir
