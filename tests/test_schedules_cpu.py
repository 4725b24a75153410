"""All four ways of cutting requests, on the CPU with plain kernels, against the plain model."""

import pytest
import torch

import plain_kernels
import plain_model
import schedules
from tiny_configs import CONFIGS, random_tokens

from ninfer_amd_mi50_b200.config import EngineOptions
from ninfer_amd_mi50_b200.engine import load_runner
from ninfer_amd_mi50_b200.weights import write_random_model


@pytest.mark.parametrize("name", ["A", "C"])
def test_schedules_agree_with_plain(name, tmp_path, monkeypatch):
    cfg, seed = CONFIGS[name]
    d = str(tmp_path / name)
    write_random_model(cfg, seed, d)
    plain_kernels.install(monkeypatch)
    pcfg, weights = plain_model.read_model_folder(d)
    reqs = {f"r{i}": random_tokens(n, cfg["vocab_size"], 30 + i) for i, n in enumerate([33, 70, 18, 49, 90])}
    want = {r: plain_model.plain_forward(pcfg, weights, t) for r, t in reqs.items()}
    for make, pool in ((schedules.whole, 128), (schedules.tail_decoded, 128),
                       (schedules.portions, 128), (lambda r: schedules.mixed(r, page=16, pool_tokens=224), 224)):
        runner = load_runner(d, options=EngineOptions(dtype="float32", device="cpu", page_size=16,
                                                       num_sequences=4, max_context=pool, cache_tokens=pool))
        got = schedules.run_schedule(runner, make(reqs))
        assert all(f == runner.cache.groups[g].pool.num_pages for g, f in enumerate(runner.cache.pages_free()))
        for r in reqs:
            torch.testing.assert_close(got[r], want[r], rtol=1e-4, atol=1e-5)
