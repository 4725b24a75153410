"""From a model folder (or a configuration and a seed) to a runner that can step.

Reference: ``Impl::load`` (src/models/model.hip:833-948) reads config.json, loads every
tensor, allocates workspaces and the cache.  Here the same happens through the registry:
config.json's architecture name picks the configuration class and the plan of parts.
"""

from __future__ import annotations

from typing import Any, Dict, Optional

import torch

from .. import log
from ..cache.manager import CacheManager
from ..config.engine_options import EngineOptions
from ..config.model_config import read_config_json
from ..parts.model import DecoderModel
from ..registry import architecture_of
from ..weights.loader import ENGINE_DTYPES, CheckpointSource, RandomSource, load_model
from .step import ModelRunner


def build_model(config: Dict[str, Any]):
    arch = architecture_of(config)
    typed = arch.parse_config(config)
    return typed, DecoderModel(arch.build_plan(typed))


def load_runner(model_dir: Optional[str] = None, *, config: Optional[Dict[str, Any]] = None,
                random_seed: Optional[int] = None, options: Optional[EngineOptions] = None
                ) -> ModelRunner:
    """`model_dir` holds config.json and safetensors; or give `config` and `random_seed`
    to draw the weights on the device without touching a file."""
    options = options or EngineOptions()
    device = torch.device(options.device)
    dtype = ENGINE_DTYPES[options.dtype]
    if config is None:
        if model_dir is None:
            raise ValueError("give a model folder or a configuration")
        config = read_config_json(model_dir)
    typed, model = build_model(config)
    model.check_limits(dtype, options.max_context, options.page_size)
    if random_seed is not None:
        source = RandomSource(model.tensor_specs(), random_seed,
                              gen_device=device if device.type == "cuda" else "cpu")
    else:
        source = CheckpointSource(model_dir)
    log.info(f"loading {config.get('architectures', ['?'])[0]} as {options.dtype} on {device}")
    load_model(model, source, dtype, device)
    source.close()
    cache = CacheManager(model.cache_specs(), model.state_specs(), page_size=options.page_size,
                         num_pages=options.num_pages, max_requests=options.num_sequences,
                         max_context=options.max_context, dtype=dtype, device=device,
                         clear_reused_pages=options.clear_reused_pages)
    runner = ModelRunner(model, cache, dtype, device, use_graph=options.use_graph)
    runner.config = typed
    runner.options = options
    log.info(f"ready: weights {model.weight_bytes() / 2**20:.1f} MiB, cache "
             f"{cache.total_bytes() / 2**20:.1f} MiB in {options.num_pages} pages of {options.page_size}")
    return runner
