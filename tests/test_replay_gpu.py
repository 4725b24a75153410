"""The engine on the GPU, in 32-bit and in bfloat16, under every way of cutting the work,
against the plain whole-sequence model; then the same through ``bin/trace_run``."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_model
import schedules
from tiny_configs import CONFIGS, random_tokens

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LENGTHS = [33, 150, 7, 97, 70, 201]

# float32: the engine and the plain model differ by summation order only: 1e-4 of the
# largest logit (measured: about 1e-6).
# bfloat16: activations between kernels are rounded to 8 bits of mantissa (unit roundoff
# 2^-9): a random walk over some twenty roundings, measured at 0.4 % of the largest logit for
# the worst element of a typical row; bound 1.5 %, for every row.  Such a rounding in the
# router's input also swaps the k-th and (k+1)-th expert wherever their probabilities are
# closer than that (about one row in fifty), and the row then carries another expert's
# output.  That is no error of the engine, so the plain model is run with the experts the
# engine chose (its own probabilities, the engine's selection), and the selection is checked
# apart: the least probable expert the engine chose may fall short of the plain model's k-th
# by 5 % of that probability at most, which only a near-tie does.
def check(got, want, dtype, what, bf16_bound=1.5e-2):
    scale = want.abs().max().item()
    row_err = (got - want).abs().max(dim=1).values
    bound = 1e-4 if dtype == "float32" else bf16_bound
    worst = int(row_err.argmax())
    assert row_err.max().item() <= bound * scale, \
        f"{what}: row {worst} differs by {row_err.max().item():.3e}, scale {scale:.3f}"
    return row_err.median().item() / scale


def check_loose(got, want, dtype, what):
    """For two bfloat16 runs whose expert choices are not known to be the same (another way of
    cutting, another process): rows that differ only by rounding stay within 1.5 %; a row in
    which a near-tie fell the other way carries another expert's output, a few per cent.  At
    most one row in ten may pass the first bound and none 10 %.  The strict comparison with
    the plain model is `test_schedule_matches_plain`."""
    if dtype == "float32":
        return check(got, want, dtype, what)
    scale = want.abs().max().item()
    row_err = (got - want).abs().max(dim=1).values
    over = (row_err > 1.5e-2 * scale).sum().item()
    assert over <= max(1, len(row_err) // 10), \
        f"{what}: {over} of {len(row_err)} rows beyond 1.5 % of scale {scale:.3f}"
    assert row_err.max().item() <= 0.1 * scale, \
        f"{what}: max error {row_err.max().item():.3e}, scale {scale:.3f}"
    return row_err.median().item() / scale


def want_for(model, reqs, want, dtype, routing, what):
    """The plain logits to compare with: in float32 the plain model's own; in bfloat16 the
    plain model run with the engine's expert choice, after checking that choice."""
    if dtype == "float32":
        return want
    pcfg, weights = model
    out = {}
    for r, toks in reqs.items():
        slack = []
        out[r] = plain_model.plain_forward(pcfg, weights, toks, forced=routing[r], slack=slack)
        for s in slack:
            assert s.max().item() <= 0.05, f"{what} {r}: an expert was chosen that is no near-tie ({s.max().item():.3f})"
    return out


@pytest.fixture(scope="module", params=["A", "B", "C", "D"])
def folder(request, tmp_path_factory):
    from ninfer_amd_mi50_b200.weights import write_random_model
    cfg, seed = CONFIGS[request.param]
    d = str(tmp_path_factory.mktemp("model") / request.param)
    write_random_model(cfg, seed, d)
    pcfg, weights = plain_model.read_model_folder(d)
    reqs = {f"r{i}": random_tokens(n, cfg["vocab_size"], 40 + i) for i, n in enumerate(LENGTHS)}
    want = {r: plain_model.plain_forward(pcfg, weights, t) for r, t in reqs.items()}
    return d, cfg, reqs, want, (pcfg, weights)


def make_runner(d, dtype, tokens):
    from ninfer_amd_mi50_b200.config import EngineOptions
    from ninfer_amd_mi50_b200.engine import load_runner
    return load_runner(d, options=EngineOptions(dtype=dtype, page_size=64, num_sequences=4,
                                                 max_context=tokens, cache_tokens=tokens, use_graph=False))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("how", ["whole", "tail_decoded", "portions", "mixed"])
def test_schedule_matches_plain(folder, dtype, how):
    d, cfg, reqs, want, model = folder
    if how == "mixed":
        steps = schedules.mixed(reqs, page=64, pool_tokens=448)
        runner = make_runner(d, dtype, 448)
    else:
        steps = getattr(schedules, how)(reqs)
        runner = make_runner(d, dtype, 256)
    routing = {}
    got = schedules.run_schedule(runner, steps, routing)
    assert runner.cache.pages_free() == [g.pool.num_pages for g in runner.cache.groups]
    want = want_for(model, reqs, want, dtype, routing, how)
    worst = max(check(got[r], want[r], dtype, f"{how} {r}") for r in reqs)
    print(f"\n[{dtype} {how}] worst error / scale = {worst:.2e}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cuts_agree_with_each_other(folder, dtype):
    """Whole prompts against portions and decoded tails: in 32-bit the same kernels see the
    same rows, so the logits agree to rounding of the last bits."""
    d, cfg, reqs, want, _ = folder
    a = schedules.run_schedule(make_runner(d, dtype, 256), schedules.whole(reqs))
    b = schedules.run_schedule(make_runner(d, dtype, 256), schedules.portions(reqs))
    c = schedules.run_schedule(make_runner(d, dtype, 256), schedules.tail_decoded(reqs))
    for r in reqs:
        check_loose(b[r], a[r], dtype, f"portions vs whole {r}")
        check_loose(c[r], a[r], dtype, f"tail vs whole {r}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(folder, dtype, tmp_path):
    d, cfg, reqs, want, _ = folder
    steps = schedules.mixed(reqs, page=64, pool_tokens=448)
    out = tmp_path / "out"
    lines = "".join(json.dumps({"step": i, **st}) + "\n" for i, st in enumerate(steps))
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype,
                        "--out", str(out), "--max-tokens", "448"], input=lines, capture_output=True,
                       text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert p.stdout.split() == [x for i in range(len(steps)) for x in ("done", str(i))]
    V = cfg["vocab_size"]
    got = {}
    for i, st in enumerate(steps):
        n = sum(len(e["want"]) for e in st["entries"])
        arr = np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(n, V)
        r = 0
        for e in st["entries"]:
            got.setdefault(e["id"], []).append(torch.from_numpy(arr[r:r + len(e["want"])].copy()))
            r += len(e["want"])
    for r in reqs:
        check_loose(torch.cat(got[r]), want[r], dtype, f"trace_run {r}")
    # the program drives the very runner, cache and kernels of the in-process schedule above:
    # same steps, same pool, same pages, hence the same bits
    same = schedules.run_schedule(make_runner(d, dtype, 448), steps)
    for r in reqs:
        assert torch.equal(torch.cat(got[r]), same[r]), f"trace_run {r} differs from the in-process run"


def test_a_reused_page_with_non_finite_leftovers_does_no_harm(tmp_path):
    """The tensor-core attention copies whole pages and multiplies what lies beyond a request's
    position by zero probabilities, so leftovers of a page's earlier owner must be finite.  The
    cache manager zeroes a page when it hands it out again: a request that inherits pages full of
    NaN gets the plain model's logits.  With the clearing switched off the same request shows
    what the rule is for."""
    from ninfer_amd_mi50_b200.config import EngineOptions
    from ninfer_amd_mi50_b200.engine import StepEntry, load_runner
    from ninfer_amd_mi50_b200.weights import write_random_model
    cfg, seed = CONFIGS["A"]
    d = str(tmp_path / "A")
    write_random_model(cfg, seed, d)
    pcfg, weights = plain_model.read_model_folder(d)
    first, second = random_tokens(256, cfg["vocab_size"], 7), random_tokens(150, cfg["vocab_size"], 8)
    want = plain_model.plain_forward(pcfg, weights, second)
    for clear in (True, False):
        runner = load_runner(d, options=EngineOptions(dtype="bfloat16", page_size=64, num_sequences=2, max_context=256,
                                                       cache_tokens=256, use_graph=False, clear_reused_pages=clear))
        runner.open("a")
        runner.step([StepEntry("a", first, [])])
        runner.close("a")
        for g in runner.cache.groups:
            g.pages[:, :g.pool.num_pages] = float("nan")          # what an earlier owner might have left
        runner.open("b")
        SparseRouting = {}
        got = schedules.run_schedule(runner, [{"entries": [{"id": "b", "tokens": second, "want": list(range(150))}],
                                              "end": ["b"]}], SparseRouting)["b"]
        if clear:
            ref = want_for((pcfg, weights), {"b": second}, {"b": want}, "bfloat16", SparseRouting, "reused page")["b"]
            check(got, ref, "bfloat16", "reused page")
            assert runner.cache.pages_cleared == 1          # 150 tokens: two pages covered whole, the third in part
        else:
            assert not bool(torch.isfinite(got).all())
