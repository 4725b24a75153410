"""The engine's own logic (packing, cache pages, block tables, the order of parts) on the
CPU, with the CUDA kernels replaced by their plain twins, against the plain model."""

import pytest
import torch

import plain_kernels
import plain_model
from tiny_configs import CONFIGS, random_tokens

from ninfer_amd_mi50_b200.config import EngineOptions
from ninfer_amd_mi50_b200.engine import StepEntry, load_runner
from ninfer_amd_mi50_b200.weights import write_random_model


@pytest.fixture(params=["A", "B", "C", "D"])
def tiny(request, tmp_path, monkeypatch):
    cfg, seed = CONFIGS[request.param]
    d = str(tmp_path / request.param)
    write_random_model(cfg, seed, d)
    plain_kernels.install(monkeypatch)
    runner = load_runner(d, options=EngineOptions(dtype="float32", device="cpu", page_size=16,
                                                   num_sequences=4, max_context=256, cache_tokens=512))
    pcfg, weights = plain_model.read_model_folder(d)
    return cfg, runner, pcfg, weights


def test_whole_prompt_matches_plain(tiny):
    cfg, runner, pcfg, weights = tiny
    toks = random_tokens(50, cfg["vocab_size"], 5)
    want = plain_model.plain_forward(pcfg, weights, toks)
    runner.open("a")
    got = runner.step([StepEntry("a", toks, list(range(len(toks))))])
    runner.close("a")
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5)


def test_portions_and_decode_match_plain(tiny):
    cfg, runner, pcfg, weights = tiny
    toks = random_tokens(61, cfg["vocab_size"], 6)
    want = plain_model.plain_forward(pcfg, weights, toks)
    runner.open("a")
    got = []
    cuts = [7, 2, 13, 2, 5, 17]
    i = 0
    for c in cuts:
        got.append(runner.step([StepEntry("a", toks[i:i + c], list(range(c)))]))
        i += c
    while i < len(toks):
        got.append(runner.step([StepEntry("a", toks[i:i + 1], [0])]))
        i += 1
    runner.close("a")
    runner.cache.check()
    torch.testing.assert_close(torch.cat(got), want, rtol=1e-4, atol=1e-5)


def test_mixed_batch_with_page_reuse(tiny):
    cfg, runner, pcfg, weights = tiny
    V = cfg["vocab_size"]
    reqs = {n: random_tokens(L, V, 10 + i) for i, (n, L) in enumerate(
        [("a", 40), ("b", 23), ("c", 57), ("d", 31), ("e", 45), ("f", 18)])}
    want = {n: plain_model.plain_forward(pcfg, weights, t) for n, t in reqs.items()}
    # a pool of 12 pages of 16: requests must reuse pages freed by earlier ones
    runner.cache = type(runner.cache)(runner.model.cache_specs(), runner.model.state_specs(),
                                      page_size=16, num_pages=12, max_requests=4, max_context=256,
                                      dtype=torch.float32, device="cpu")
    got = {n: [] for n in reqs}
    done = {n: 0 for n in reqs}
    waiting = list(reqs)
    live = []
    chunk = {"a": 9, "b": 5, "c": 16, "d": 2, "e": 11, "f": 7}
    step = 0
    while waiting or live:
        while waiting and len(live) < 4:
            n = waiting[0]
            runner.open(n)
            pages = sum(runner.cache.pages_needed(x, len(reqs[x]))[0] for x in live + [n])
            if pages > runner.cache.groups[0].pool.num_free and live:
                runner.close(n)
                break
            live.append(waiting.pop(0))
        entries = []
        for n in live:
            left = len(reqs[n]) - done[n]
            # prompt portions first, the last 6 tokens one by one
            c = 1 if left <= 6 else min(chunk[n], left - 6)
            entries.append(StepEntry(n, reqs[n][done[n]:done[n] + c], list(range(c))))
        out = runner.step(entries)
        r = 0
        for e in entries:
            c = len(e.tokens)
            got[e.req].append(out[r:r + c])
            r += c
            done[e.req] += c
        for n in list(live):
            if done[n] == len(reqs[n]):
                runner.close(n)
                live.remove(n)
        runner.cache.check()
        step += 1
    assert step > 8
    for n in reqs:
        torch.testing.assert_close(torch.cat(got[n]), want[n], rtol=1e-4, atol=1e-5, msg=lambda m: f"{n}: {m}")
