#!/usr/bin/env python3
"""Decode and prefill throughput at Qwen1.5-MoE-A2.7B layer sizes with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]
    python bench.py --config 57b           # Qwen2-57B-A14B layer sizes: decode at batch 1 / 8 / 32 after 1,024-token contexts
    python bench.py --long-prefill         # adds prefill of 8,192 and 32,768 tokens in portions of 2,048 (--portion)
    python bench.py --config check-fp32    # the whole model in 32-bit at A2.7B sizes against the plain model

One JSON line on stdout.  A "step" is one decode step of a batch of 8 requests, each
holding a context of about 2,048 tokens (the context length of the named configuration's
decode workload).  `value` is decoded tokens per second from CUDA events around K steps;
`e2e` is the same through the Python entry point's scheduler-driven engine, host token ids
in and sampled token ids out, by the wall clock around K steps.  `prefill` times one
prompt of 2,048 tokens, `points` holds decode at batch 1 and 64, `roofline` compares the
bytes a decode step must read (each weight it uses once, and the cache of the live
requests) with the measured copy bandwidth.

The reference (HIP for gfx906 + rocBLAS) cannot be built on this machine: `--impl reference`
says so and exits 0.
"""

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Qwen1.5-MoE-A2.7B layer sizes (the third of the build's named configurations)
CONFIG = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "num_hidden_layers": 24, "hidden_size": 2048, "num_attention_heads": 16,
    "num_key_value_heads": 16, "head_dim": 128, "intermediate_size": 5632,
    "num_experts": 60, "num_experts_per_tok": 4, "moe_intermediate_size": 1408,
    "shared_expert_intermediate_size": 5632, "norm_topk_prob": False,
    "decoder_sparse_step": 1, "mlp_only_layers": [], "vocab_size": 151936,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "use_sliding_window": False, "qkv_bias": True,
}
FULL_LAYERS = 24
CONTEXT = 4096
PROMPT = 2048
# Qwen2-57B-A14B layer sizes (the fourth named configuration): 114.8 GB of bfloat16 weights
CONFIG_57B = dict(CONFIG, num_hidden_layers=28, hidden_size=3584, num_attention_heads=28,
                  num_key_value_heads=4, intermediate_size=18944, num_experts=64, num_experts_per_tok=8,
                  moe_intermediate_size=2560, shared_expert_intermediate_size=20480)
# name -> (config.json, its layer count, model name, tokens each request holds when decode is timed,
#          batch of `value`, batches of `points`)
PROFILES = {
    "a2.7b": (CONFIG, 24, "Qwen1.5-MoE-A2.7B", 2048, 8, (1, 64)),
    "57b": (CONFIG_57B, 28, "Qwen2-57B-A14B", 1024, 8, (1, 32)),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "source": "measured"}
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed region."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc:
            self.proc.terminate()
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.rows)}


def check_fp32(args) -> int:
    """The fifth named configuration: the whole model in true 32-bit at Qwen1.5-MoE-A2.7B layer
    sizes (57 GB of weights drawn on the device from seed 7) against the plain implementation of
    tests/plain_model.py, which restates the same weights from the seed and runs in float32 on
    the device too.  Requests with prompt lengths uniform in [1, 1024] go through the engine
    whole, in portions of 256, mixed (up to four live, portions of some beside single tokens of
    others, a pool so small that pages are used again) and, for the first eight, with the last
    32 tokens one by one; every position's logits are compared.  Where the engine and the plain
    model pick different experts for a row (two router probabilities that agree to 1e-4 of their
    value: among hundreds of thousands of selections a few fall that close), the plain model is
    run again with the engine's choice, so that a tie broken the other way is not counted as an
    error of 1e-2.  Prints one JSON line."""
    import random

    import torch
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import plain_model
    import schedules
    from ninfer_amd_mi50_b200 import kernels
    from ninfer_amd_mi50_b200.config import EngineOptions
    from ninfer_amd_mi50_b200.engine import load_runner

    kernels.load()
    cfg = dict(CONFIG, num_hidden_layers=args.layers or FULL_LAYERS)
    seed, n = 7, args.requests
    rnd = random.Random(11)
    reqs = {f"r{i}": [rnd.randrange(cfg["vocab_size"]) for _ in range(rnd.randint(1, 1024))] for i in range(n)}

    class Kept:
        def __init__(self, drawn):
            self.drawn, self.kept = drawn, {}

        def __contains__(self, name):
            return name in self.drawn

        def __getitem__(self, name):
            if name not in self.kept:
                self.kept[name] = self.drawn[name]
            return self.kept[name]

    t0 = time.time()
    weights = Kept(plain_model.RandomWeights(cfg, seed, device="cuda"))
    pool = 4 * 1024
    runner = load_runner(config=cfg, random_seed=seed,
                         options=EngineOptions(dtype="float32", page_size=64, num_sequences=4, max_context=1024,
                                               cache_tokens=pool, use_graph=False))
    sys.stderr.write(f"[check-fp32] engine ready in {time.time() - t0:.0f}s\n")
    # Eight requests at a time, so that the logits of all positions (0.6 MB a token) fit in memory.
    names = list(reqs)
    worst = {"whole": 0.0, "portions_of_256": 0.0, "mixed": 0.0, "tail_decoded": 0.0}
    steps_run = {k: 0 for k in worst}
    ties = 0
    for g0 in range(0, n, 8):
        group = {r: reqs[r] for r in names[g0:g0 + 8]}
        plans = {"whole": schedules.whole(group),
                 "portions_of_256": schedules.portions(group, cuts=[256]),
                 "mixed": schedules.mixed(group, page=64, pool_tokens=pool, cuts=[256, 64, 7, 2, 130])}
        if g0 == 0:
            plans["tail_decoded"] = schedules.tail_decoded(group)
        want, own = {}, {}
        for r, t in group.items():
            own[r] = {}
            want[r] = plain_model.plain_forward(cfg, weights, t, chosen=own[r]).cpu()
        for how, steps in plans.items():
            routing = {}
            got = schedules.run_schedule(runner, steps, routing)
            kernels.check_status(how)
            steps_run[how] += len(steps)
            for r, toks in group.items():
                ref = want[r]
                if any(not torch.equal(routing[r][l], own[r][l]) for l in own[r]):
                    slack = []
                    ref = plain_model.plain_forward(cfg, weights, toks, forced=routing[r], slack=slack).cpu()
                    ties += sum(int((routing[r][l] != own[r][l]).any(dim=1).sum()) for l in own[r])
                    assert max(s.max().item() for s in slack) <= 1e-4, "the engine chose an expert that is no tie"
                scale = ref.abs().max().item()
                worst[how] = max(worst[how], (got[r] - ref).abs().max().item() / scale)
            del got
        sys.stderr.write(f"[check-fp32] requests {g0}..{g0 + len(group) - 1}: worst error / largest logit so far "
                         + ", ".join(f"{k} {v:.2e}" for k, v in worst.items()) + f" ({time.time() - t0:.0f}s)\n")
    ok = all(v <= 1e-4 for v in worst.values())
    print(json.dumps({"check": "float32 whole model against the plain model", "model": "Qwen1.5-MoE-A2.7B sizes",
                      "layers": cfg["num_hidden_layers"], "requests": n, "tokens": sum(len(t) for t in reqs.values()),
                      "steps": steps_run, "rows_with_a_tie_broken_the_other_way": ties,
                      "worst_error_over_largest_logit": {k: float(f"{v:.3e}") for k, v in worst.items()},
                      "bound": 1e-4, "ok": ok}))
    return 0 if ok else 1


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="a2.7b", choices=sorted(PROFILES) + ["check-fp32"])
    ap.add_argument("--layers", type=int, default=None, help="fewer layers, for a quick look")
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--long-prefill", action="store_true", help="also time prompts of 8,192 and 32,768 tokens")
    ap.add_argument("--portion", type=int, default=2048,
                    help="tokens a step of the long prompts (the 2,048-token prompt is always one step)")
    ap.add_argument("--requests", type=int, default=64, help="check-fp32: number of requests")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is HIP for gfx906 with rocBLAS (CMake refuses any other "
                          "architecture); no ROCm here and no Python package to install"}))
        return 0
    if args.gpus != 1:
        print("bench.py: this engine runs on one GPU; --gpus %d is not supported" % args.gpus)
        return 2
    W = max(3, args.warmup)
    K = max(1, args.steps)
    if args.config == "check-fp32":
        return check_fp32(args)
    CONFIG, FULL_LAYERS, model_name, PROMPT, value_batch, point_batches = PROFILES[args.config]
    args.layers = args.layers or FULL_LAYERS
    args.batch = args.batch or value_batch
    long_context = 32768 if args.long_prefill else CONTEXT

    import torch
    from ninfer_amd_mi50_b200 import kernels
    from ninfer_amd_mi50_b200.config import EngineOptions
    from ninfer_amd_mi50_b200.engine import Engine, StepEntry
    from ninfer_amd_mi50_b200.kernels import lib as klib
    from ninfer_amd_mi50_b200.sampling import SamplingParams

    kernels.load()
    pk = peaks()
    cfg = dict(CONFIG, num_hidden_layers=args.layers)
    max_batch = max(point_batches + (args.batch,)) if not args.skip_points else args.batch
    opts = EngineOptions(dtype="bfloat16", max_context=long_context, prefill_chunk=max(2048, args.portion),
                         num_sequences=max_batch, page_size=64, cache_tokens=max_batch * CONTEXT,
                         max_batched_tokens=max(2048, args.portion))
    t0 = time.time()
    engine = Engine(config=cfg, random_seed=2, options=opts)
    runner, cache, model = engine.runner, engine.cache, engine.runner.model
    sys.stderr.write(f"[bench] model ready in {time.time() - t0:.0f}s: weights "
                     f"{model.weight_bytes() / 1e9:.2f} GB, cache {cache.total_bytes() / 1e9:.1f} GB\n")
    g = torch.Generator().manual_seed(0)
    V = cfg["vocab_size"]

    # cache contents for synthetic contexts: unit-variance keys and values
    for grp in cache.groups:
        grp.pages.normal_(0, 1)

    def open_synthetic(n, length):
        """n requests that already hold `length` tokens (cache contents synthetic)."""
        ids = []
        for i in range(n):
            rid = ("bench", i)
            cache.open(rid)
            cache.reserve(rid, length)
            cache.commit(rid, length)
            ids.append(rid)
        return ids

    def close_all(ids):
        for r in ids:
            cache.close(r)

    def time_decode(batch, steps, warm):
        ids = open_synthetic(batch, PROMPT)
        toks = torch.randint(0, V, (warm + steps, batch), generator=g).tolist()
        for s in range(warm):
            runner.step([StepEntry(r, [toks[s][i]], [0]) for i, r in enumerate(ids)])
        torch.cuda.synchronize()
        launches0 = klib.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for s in range(warm, warm + steps):
            runner.step([StepEntry(r, [toks[s][i]], [0]) for i, r in enumerate(ids)])
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        launches = klib.launch_count() - launches0
        close_all(ids)
        return ms, launches

    def decode_bytes(batch):
        """Bytes one decode step must read: every weight it uses once (the routed experts
        that this batch's tokens select, counted from the routing itself) and the cache of
        the live requests."""
        from ninfer_amd_mi50_b200.parts.feedforward import SparseMoeSwiglu
        ids = open_synthetic(batch, PROMPT)
        SparseMoeSwiglu.record_routing = []
        graphs, runner.graphs = runner.graphs, None      # routing is recorded by the host-driven step
        runner.step([StepEntry(r, [int(torch.randint(0, V, (1,), generator=g))], [0]) for r in ids])
        torch.cuda.synchronize()
        runner.graphs = graphs
        routed = SparseMoeSwiglu.record_routing
        SparseMoeSwiglu.record_routing = None
        total = model.head.numel() * model.head.element_size() + batch * model.hidden_size * 2  # head, embedding rows
        li = 0
        for blk in model.blocks:
            ff = blk.feed_forward
            total += blk.norm1.weight_bytes() + blk.norm2.weight_bytes() + blk.mixer.weight_bytes()
            if isinstance(ff, SparseMoeSwiglu):
                used = int(torch.unique(routed[li]).numel())
                li += 1
                total += ff.weight_bytes() - (ff.num_experts - used) * ff.expert_bytes()
            else:
                total += ff.weight_bytes()
        kv = batch * (PROMPT + 1) * cache.bytes_per_token()
        close_all(ids)
        return total, kv

    clocks = ClockSampler()
    clocks.start()
    ms, launches = time_decode(args.batch, K, W)
    clk = clocks.stop()
    value = args.batch / (ms / 1e3)
    wbytes, kvbytes = decode_bytes(args.batch)
    achieved = (wbytes + kvbytes) / (ms / 1e3) / 1e9

    # ---- prefill of one 2,048-token prompt -------------------------------------------------
    PREFILL = 2048
    ptoks = torch.randint(0, V, (32768 if args.long_prefill else PREFILL,), generator=g).tolist()

    def prefill_once(tokens=PREFILL, portion=PREFILL):
        cache.open("prefill")
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for a in range(0, tokens, portion):
            part = ptoks[a:min(a + portion, tokens)]
            runner.step([StepEntry("prefill", part, [len(part) - 1] if a + portion >= tokens else [])])
        e1.record()
        torch.cuda.synchronize()
        cache.close("prefill")
        return e0.elapsed_time(e1)

    for _ in range(3):
        prefill_once()
    pms = min(prefill_once() for _ in range(3))
    c = cfg
    H, L = c["hidden_size"], c["num_hidden_layers"]
    qkvo = 2 * H * (c["num_attention_heads"] + 2 * c["num_key_value_heads"]) * c["head_dim"] \
        + 2 * H * c["num_attention_heads"] * c["head_dim"]
    experts = c["num_experts_per_tok"] * 6 * H * c["moe_intermediate_size"]
    shared = 6 * H * c["shared_expert_intermediate_size"]
    router = 2 * H * (c["num_experts"] + 1)
    def prefill_flops(tokens):
        attn = 4 * c["num_attention_heads"] * c["head_dim"] * (tokens + 1) / 2      # causal half, per token
        return tokens * L * (qkvo + experts + shared + router + attn) + 2 * H * V

    prefill = {"value": round(PREFILL / (pms / 1e3), 1), "tokens": PREFILL, "ms": round(pms, 3),
               "frac": round(prefill_flops(PREFILL) / (pms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
    if args.long_prefill:
        for n in (8192, 32768):
            prefill_once(n, args.portion)
            lms = min(prefill_once(n, args.portion) for _ in range(2))
            prefill[f"tokens_{n}"] = {"value": round(n / (lms / 1e3), 1), "ms": round(lms, 3), "portion": args.portion, "frac": round(
                prefill_flops(n) / (lms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}

    # ---- decode at batch 1 and 64 ----------------------------------------------------------
    points, points_frac = {}, {}
    if not args.skip_points:
        for b in point_batches:
            pm, _ = time_decode(b, max(8, K // 2), W)
            points[f"decode_b{b}"] = round(b / (pm / 1e3), 1)
            pw, pkv = decode_bytes(b)
            points_frac[f"decode_b{b}"] = round((pw + pkv) / (pm / 1e3) / 1e9 / pk["hbm_gbs"], 4)

    # ---- end to end through the entry point's engine -----------------------------------------
    e2e = None
    if not args.skip_e2e:
        prompts = torch.randint(0, V, (args.batch, PROMPT), generator=g).tolist()
        # long enough that no request finishes (and no smaller graph is built) inside the timed steps
        sp = SamplingParams(temperature=0.0, max_new_tokens=W + K + 3 * args.batch + 16)
        for p in prompts:
            engine.submit(p, sp)
        while any(r.remaining != 1 or not r.generated for r in engine.scheduler.running) or engine.scheduler.waiting:
            engine.step()
        for _ in range(W):
            engine.step()
        torch.cuda.synchronize()
        h2d0, d2h0 = engine.io_bytes()
        t0 = time.perf_counter()
        for _ in range(K):
            engine.step()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        h2d1, d2h1 = engine.io_bytes()
        e2e = {"value": round(args.batch * K / dt, 1), "unit": "tokens/s",
               "h2d_bytes_per_step": (h2d1 - h2d0) // K, "d2h_bytes_per_step": (d2h1 - d2h0) // K}
        for r in list(engine.scheduler.running):
            engine.scheduler._finish(r, "length")

    out = {
        "metric": f"decode tok/s @ batch {args.batch} ({model_name} layer sizes, context {PROMPT}+)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights, random token ids, random cache)",
        "impl": "ours",
        "config": {"model": f"{model_name} sizes", "layers": L, "layers_full": FULL_LAYERS,
                   "hidden": H, "heads": c["num_attention_heads"], "kv_heads": c["num_key_value_heads"],
                   "head_dim": c["head_dim"], "experts": c["num_experts"], "top_k": c["num_experts_per_tok"],
                   "moe_intermediate": c["moe_intermediate_size"],
                   "shared_intermediate": c["shared_expert_intermediate_size"], "vocab": V,
                   "global_batch": args.batch, "seq_len": PROMPT, "context": CONTEXT,
                   "page_size": 64, "parallelism": "single GPU",
                   "l2": "step inputs (weights + cache) exceed L2 many times over; no flush needed"},
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk["source"],
                     "weight_bytes": wbytes, "cache_bytes": kvbytes},
        "points": points, "points_roofline_frac": points_frac, "e2e": e2e, "gpu_launches": launches, "clocks": clk,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
