"""Representative kernel workloads, one layer's worth, for profilers and quick timing; the layer
sizes come from a named set (`--sizes`, by default those of Qwen1.5-MoE-A2.7B):

    python -m ninfer_amd_mi50_b200.kernels.cases moe_prefill
    ncu --set full --clock-control none -k regex:grouped_gemm_tc -c 2 \
        python -m ninfer_amd_mi50_b200.kernels.cases moe_prefill

(run the plain command first and profile only after it exits 0; without `--clock-control none`
a profiler locks the clocks of a GPU that others share.)

Each case warms its kernels up and then runs them a few times; with `--time` it prints the
median time per call from CUDA events (launch included) with an L2 flush between calls.  A case holds about
1.5 GB on the device, larger than L2, so DRAM figures mean something.
"""

from __future__ import annotations

import argparse
import math
import sys
from types import SimpleNamespace

import torch

# name -> layer sizes (config.json's meanings): the two large configurations that are measured
SIZES = {
    "a2.7b": dict(H=2048, I=1408, IS=5632, E=60, K_TOP=4, V=151936, HQ=16, HKV=16, D=128),
    "57b-a14b": dict(H=3584, I=2560, IS=20480, E=64, K_TOP=8, V=151936, HQ=28, HKV=4, D=128),
}
PAGE = 64
H = I = IS = E = K_TOP = V = HQ = HKV = D = 0     # set from SIZES by `use_sizes`


def use_sizes(name: str) -> None:
    globals().update(SIZES[name])


use_sizes("a2.7b")


def _routing(tokens: int, seed: int, device):
    g = torch.Generator().manual_seed(seed)
    idx = torch.stack([torch.randperm(E, generator=g)[:K_TOP] for _ in range(tokens)])
    return idx.to(torch.int32).to(device)


def _experts(device):
    from . import pack_weights
    w13 = pack_weights((torch.randn(E, 2 * I, H, device=device) * 0.02).bfloat16(), True)
    w2 = pack_weights((torch.randn(E, H, I, device=device) * 0.02).bfloat16(), False)
    return w13, w2


def case_moe(tokens: int, device):
    """Routed experts: both products for `tokens` tokens with uniform random routing."""
    from . import moe_gemm1, moe_gemm2, moe_plan
    w13, w2 = _experts(device)
    x = torch.randn(tokens, H, device=device).bfloat16()
    plan = moe_plan(_routing(tokens, tokens, device), E)
    act = moe_gemm1(x, w13, plan, K_TOP)
    return [("moe_gemm1", lambda: moe_gemm1(x, w13, plan, K_TOP)),
            ("moe_gemm2", lambda: moe_gemm2(act, w2, plan))]


def case_moe_stream(tokens: int, device, whole_block: bool):
    """The persistent launch of a decode step: both products of the routed experts for `tokens`
    tokens (plan given), or with `whole_block` the routing and the shared expert as well."""
    from . import TUNING, moe_experts, moe_plan, pack_shared_expert, route_and_run_experts
    TUNING.update(moe_stream_min_tokens=1, moe_stream_max_tokens=64, moe_stream_route_max_tokens=64,
                  moe_stream_shared_max_tokens=64)
    w13, w2 = _experts(device)
    x = torch.randn(tokens, H, device=device).bfloat16()
    if not whole_block:
        plan = moe_plan(_routing(tokens, tokens, device), E)
        return [("moe_experts", lambda: moe_experts(x, w13, w2, plan, K_TOP))]
    wr = torch.randn(E + 1, H, device=device) * 0.05
    shared = pack_shared_expert((torch.randn(2 * IS, H, device=device) * 0.02).bfloat16(),
                                (torch.randn(H, IS, device=device) * 0.02).bfloat16(), I)
    return [("route_experts_shared", lambda: route_and_run_experts(x, wr, E, K_TOP, False, w13, w2, shared=shared))]


def case_attention_prefill(tokens: int, device):
    """One fresh prompt of `tokens` tokens: flash prefill attention over the paged cache."""
    from . import paged_attention
    from ..parts.base import StepContext
    n_pages = (tokens + PAGE - 1) // PAGE
    pages = torch.randn(n_pages + 1, 2, HKV, PAGE, D, device=device).bfloat16()
    bt = torch.arange(n_pages, dtype=torch.int32, device=device).view(1, -1)
    mk = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
    ctx = StepContext(dtype=torch.bfloat16, device=torch.device(device), T=tokens, S=1, token_ids=mk([0]),
                      positions=torch.arange(tokens, dtype=torch.int32, device=device),
                      row_seg=torch.zeros(tokens, dtype=torch.int32, device=device), seg_row0=mk([0, tokens]),
                      seg_pos0=mk([0]), seg_slot=mk([0]), logit_rows=mk([]), seg_len_host=[tokens],
                      seg_pos0_host=[0], max_rows_per_seg=tokens, max_context=tokens)
    qkv = torch.randn(tokens, (HQ + 2 * HKV) * D, device=device).bfloat16()
    return [("prefill_attention", lambda: paged_attention(qkv, HQ, HKV, D, pages, bt, PAGE, ctx, 0, 1 / math.sqrt(D)))]


def case_attention_decode(batch: int, context: int, device):
    """`batch` requests of `context` tokens each, one new row per request."""
    from . import paged_attention
    per = context // PAGE + 1
    pages = torch.randn(batch * per + 1, 2, HKV, PAGE, D, device=device).bfloat16()
    bt = torch.arange(batch * per, dtype=torch.int32, device=device).view(batch, per)
    ctx = SimpleNamespace(positions=torch.full((batch,), context, dtype=torch.int32, device=device),
                          row_seg=torch.arange(batch, dtype=torch.int32, device=device), all_single=True,
                          max_context=context + 1)
    qkv = torch.randn(batch, (HQ + 2 * HKV) * D, device=device).bfloat16()
    return [("decode_attention", lambda: paged_attention(qkv, HQ, HKV, D, pages, bt, PAGE, ctx, 0, 1 / math.sqrt(D)))]


def case_dense_decode(batch: int, device):
    """The dense products of a decode step: QKV, O, shared expert, LM head."""
    from . import linear, linear_swiglu
    mk = lambda n, k: (torch.randn(n, k, device=device) * 0.02).bfloat16()
    wqkv, wo, ws13, ws2, head = mk((HQ + 2 * HKV) * D, H), mk(H, HQ * D), mk(2 * IS, H), mk(H, IS), mk(V, H)
    x, xs = torch.randn(batch, H, device=device).bfloat16(), torch.randn(batch, IS, device=device).bfloat16()
    return [("qkv", lambda: linear(x, wqkv)), ("o_proj", lambda: linear(x, wo)),
            ("shared_gate_up", lambda: linear_swiglu(x, ws13)), ("shared_down", lambda: linear(xs, ws2)),
            ("lm_head", lambda: linear(x, head, out_dtype=torch.float32))]


def case_small_decode(batch: int, device):
    """The short kernels between a decode step's products: norm with residual add, router with
    plan, weighted sum of the experts' outputs joined with the next norm."""
    from . import add_rmsnorm, moe_combine_add_rmsnorm, moe_plan, route
    h = torch.randn(batch, H, device=device)
    delta = torch.randn(batch, H, device=device).bfloat16()
    w = torch.ones(H, device=device)
    out = torch.empty(batch, H, device=device, dtype=torch.bfloat16)
    wr = torch.randn(E + 1, H, device=device) * 0.02
    plan = moe_plan(_routing(batch, batch, device), E)
    y = torch.randn(batch * K_TOP, H, device=device).bfloat16()
    wts = torch.rand(batch, K_TOP, device=device)
    gate = torch.randn(batch, 1, device=device)
    return [("add_rmsnorm", lambda: add_rmsnorm(h, delta, w, 1e-6, out)),
            ("route", lambda: route(out, wr, E, K_TOP, False)),
            ("combine_add_rmsnorm", lambda: moe_combine_add_rmsnorm(y, plan, wts, delta, gate, h, None, w, 1e-6, out))]


CASES = {
    "moe_prefill": lambda dev: case_moe(2048, dev),
    "moe_decode8": lambda dev: case_moe(8, dev),
    "moe_decode64": lambda dev: case_moe(64, dev),
    "moe_stream_decode8": lambda dev: case_moe_stream(8, dev, False),
    "moe_stream_decode16": lambda dev: case_moe_stream(16, dev, False),
    "moe_stream_decode64": lambda dev: case_moe_stream(64, dev, False),
    "moe_block_decode8": lambda dev: case_moe_stream(8, dev, True),
    "attention_prefill": lambda dev: case_attention_prefill(2048, dev),
    "attention_decode8": lambda dev: case_attention_decode(8, 2048, dev),
    "attention_decode64": lambda dev: case_attention_decode(64, 2048, dev),
    "dense_decode8": lambda dev: case_dense_decode(8, dev),
    "dense_decode1": lambda dev: case_dense_decode(1, dev),
    "small_decode8": lambda dev: case_small_decode(8, dev),
}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("case", choices=sorted(CASES))
    ap.add_argument("--sizes", default="a2.7b", choices=sorted(SIZES))
    ap.add_argument("--repeat", type=int, default=3)
    ap.add_argument("--time", action="store_true", help="print the median time per call")
    args = ap.parse_args(argv)
    from . import load, tensor_core_status
    use_sizes(args.sizes)
    load()
    ops = CASES[args.case]("cuda")
    for _, fn in ops:
        for _ in range(2):
            fn()
    torch.cuda.synchronize()
    # L2 is flushed by writing one buffer larger than it and then reading another: the read pushes
    # the written lines out, so that the timed call does not pay for their write-back
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if args.time else None
    clean = torch.zeros(256 << 20, dtype=torch.uint8, device="cuda") if args.time else None
    for name, fn in ops:
        times = []
        for _ in range(args.repeat if not args.time else max(args.repeat, 15)):
            if flush is not None:
                flush.zero_()
                clean.sum()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) * 1e3)
        if args.time:
            times.sort()
            print(f"{args.case}/{name}: {times[len(times) // 2]:.1f} us")
    status = tensor_core_status()
    if status:
        print(f"a tensor-core kernel gave up on a wait (code {status})")
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
