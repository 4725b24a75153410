"""Binding checkpoint tensors to the parts that ask for them, by tensor name.

The reference opens ``model.safetensors.index.json`` (``weight_map`` -> shard files) or a
single ``model.safetensors`` (src/models/model.hip:85-113), looks tensors up by name and
throws ``missing tensor in checkpoint: <name>`` at the first miss (model.hip:116-119); it
never checks a shape.  Here every tensor the model's parts declare is checked against
the file headers before a byte is read, and one error lists everything that is missing,
everything that no part asked for, and every wrong shape.  A file that only holds tensors
nobody asked for beside all that are needed (older exports carry ``rotary_emb.inv_freq``
buffers) still loads: the extra names are listed in a warning, or, with ``strict``, in the
same error.

Held dtypes (see `TensorSpec.role`): matrices in the engine dtype, norm weights, biases
and routing matrices in float32, integer tables in int32.
"""

from __future__ import annotations

import json
import os
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from .. import log
from ..parts.base import TensorSpec
from . import counter_rng
from .safetensors_io import SafetensorsError, SafetensorsFile


class WeightError(RuntimeError):
    """The checkpoint does not fit the model; the message lists every problem."""

    def __init__(self, message: str, missing=(), unexpected=(), wrong_shape=()):
        super().__init__(message)
        self.missing, self.unexpected, self.wrong_shape = list(missing), list(unexpected), list(wrong_shape)


ENGINE_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def held_dtype(role: str, engine_dtype: torch.dtype) -> torch.dtype:
    if role == "matrix":
        return engine_dtype
    if role in ("vector", "router"):
        return torch.float32
    if role == "table":
        return torch.int32
    raise ValueError(f"unknown tensor role {role!r}")


class CheckpointSource:
    """The tensors of a model folder, across its shard files."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        index = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        files: List[str] = []
        if os.path.exists(index):
            with open(index, "r", encoding="utf-8") as fh:
                wm = json.load(fh).get("weight_map")
            if not isinstance(wm, dict) or not wm:
                raise WeightError(f"{index}: no weight_map")
            files = sorted(set(wm.values()))
        elif os.path.exists(single):
            files = ["model.safetensors"]
        else:
            raise WeightError(f"no model.safetensors or model.safetensors.index.json in {model_dir}")
        self.files = [SafetensorsFile(os.path.join(model_dir, f)) for f in files]
        self.by_name: Dict[str, SafetensorsFile] = {}
        for f in self.files:
            for n in f.names():
                self.by_name[n] = f

    def names(self) -> List[str]:
        return list(self.by_name)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.by_name[name].tensors[name].shape

    def read(self, name: str, spec: TensorSpec, dtype: torch.dtype, device) -> torch.Tensor:
        t = self.by_name[name].read(name)
        if dtype == torch.int32 and t.is_floating_point():
            raise WeightError(f"tensor {name!r} should be an integer table, file has {t.dtype}")
        return t.to(device=device, dtype=dtype, non_blocking=False)

    def close(self) -> None:
        for f in self.files:
            f.close()


class RandomSource:
    """Seeded random tensors for exactly the names the model declares.

    Linear weights and biases N(0, 0.02); norm weights 1 + N(0, 0.05); every value a
    bfloat16 number.  An element is a function of (seed, tensor name, element index) alone
    (`counter_rng`): the values do not depend on the order in which tensors are asked for,
    nor on the device that draws them, so a model drawn in place on the GPU, a folder written
    by `write_random_model` on the CPU and a plain implementation that restates the function
    all hold the same numbers.
    """

    def __init__(self, specs: Sequence[TensorSpec], seed: int, gen_device="cpu"):
        self.specs = {s.name: s for s in specs}
        self.seed, self.gen_device = int(seed), torch.device(gen_device)

    def names(self) -> List[str]:
        return list(self.specs)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.specs[name].shape

    def generate(self, name: str, dtype: torch.dtype = torch.float32, device=None) -> torch.Tensor:
        spec = self.specs[name]
        device = torch.device(device) if device is not None else self.gen_device
        if spec.role == "table":
            return torch.zeros(spec.shape, dtype=torch.int32, device=device)
        out = torch.empty(spec.shape, dtype=dtype, device=device)
        return counter_rng.fill(out, counter_rng.tensor_keys(self.seed, name), spec.init)

    def read(self, name: str, spec: TensorSpec, dtype: torch.dtype, device) -> torch.Tensor:
        device = torch.device(device)
        if dtype in (torch.float32, torch.bfloat16) and device.type == self.gen_device.type:
            return self.generate(name, dtype, device)       # drawn where it stays, in its held dtype
        return self.generate(name).to(device=device, dtype=dtype)

    def close(self) -> None:
        pass


def check_specs(specs: Sequence[TensorSpec], source, strict: bool = False) -> List[str]:
    """Raise one `WeightError` naming every missing, unexpected and misshapen tensor.

    Missing and misshapen tensors are always fatal.  Tensors that no part asked for are
    fatal with `strict`; otherwise they are returned (and the caller warns)."""
    want = {}
    for s in specs:
        if s.name in want and want[s.name].shape != s.shape:
            raise ValueError(f"two parts ask for {s.name!r} with different shapes")
        want[s.name] = s
    have = set(source.names())
    missing = sorted(n for n in want if n not in have)
    unexpected = sorted(n for n in have if n not in want)
    wrong = []
    for n, s in want.items():
        if n in have and tuple(source.shape(n)) != tuple(s.shape):
            wrong.append((n, tuple(s.shape), tuple(source.shape(n))))
    if not (missing or wrong or (unexpected and strict)):
        return unexpected

    def some(items, fmt=str, limit=12):
        shown = ", ".join(fmt(i) for i in items[:limit])
        return shown + (f", ... ({len(items) - limit} more)" if len(items) > limit else "")

    parts = []
    if missing:
        parts.append(f"{len(missing)} missing: {some(missing)}")
    if unexpected:
        parts.append(f"{len(unexpected)} unexpected: {some(unexpected)}")
    if wrong:
        parts.append(f"{len(wrong)} with a wrong shape: " + some(
            wrong, lambda w: f"{w[0]} (model wants {list(w[1])}, file has {list(w[2])})"))
    raise WeightError("checkpoint does not match the model configuration; " + "; ".join(parts),
                      missing, unexpected, wrong)


def load_model(model, source, engine_dtype: torch.dtype, device, strict: bool = False) -> None:
    """Check everything, then let each part pull its tensors."""
    specs = model.tensor_specs()
    extra = check_specs(specs, source, strict)
    if extra:
        shown = ", ".join(extra[:12]) + (f", ... ({len(extra) - 12} more)" if len(extra) > 12 else "")
        log.warn(f"checkpoint holds {len(extra)} tensors that no part of the model asked for "
                 f"(not loaded): {shown}")
    by_name = {s.name: s for s in specs}

    def fetch(name: str) -> torch.Tensor:
        spec = by_name[name]
        return source.read(name, spec, held_dtype(spec.role, engine_dtype), device)

    model.load(fetch)
