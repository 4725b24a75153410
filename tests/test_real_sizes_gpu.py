"""The whole model at the layer sizes of the two large configurations, fewer layers: two layers
of Qwen1.5-MoE-A2.7B sizes (width 2048, 16 heads of 128 with 16 kv heads, 60 experts of 1408 with
4 a token, shared expert 5632) and two of Qwen2-57B-A14B sizes (width 3584, 28 heads with 4 kv
heads - seven heads a group -, 64 experts of 2560 with 8 a token, shared expert 20480), both
with the full vocabulary of 151,936.  At these sizes the engine takes other kernels than at the
tiny ones: the cluster router, the streaming products with their wide tiles, the tensor-core
grouped products and attention, the library's dense products.

No file is written: the engine draws its weights on the device from a seed, and the plain
model restates the same function of (seed, tensor name, index), also on the device, in float32
(plain torch operations; TF32 is off).  Requests of 33 to 260 tokens go through the four ways
of cutting, with a pool so small that pages are used again, in 32-bit and in bfloat16.

Bounds.  float32: 1e-4 of the largest logit, as at the tiny sizes.  bfloat16: at these widths
attention is a real softmax (scores of a few units instead of a few tenths), so the rounding of
queries, keys and probabilities to 8 bits moves a row more than at the tiny sizes: measured
0.4-0.6 % of the largest logit at a prompt's first position, 0.9 % (width 2048) and 1.2 %
(width 3584) for the median row, 2.2 % for the worst of 540 rows.  The bound is 3 % for every
row, and a second one that needs no number: the engine must be closer to the 32-bit plain
model than the plain model's own evaluation in bfloat16 is (every product and sum rounded to
bfloat16, residual stream included; measured 2 to 10 times the engine's error).
"""

import pytest
import torch

import plain_model
import schedules
from tiny_configs import random_tokens

pytestmark = pytest.mark.gpu

BASE = {"architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe", "num_hidden_layers": 2,
        "head_dim": 128, "vocab_size": 151936, "norm_topk_prob": False, "decoder_sparse_step": 1,
        "mlp_only_layers": [], "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
        "use_sliding_window": False, "qkv_bias": True, "hidden_act": "silu"}
SIZES = {
    "a2.7b": dict(BASE, hidden_size=2048, num_attention_heads=16, num_key_value_heads=16,
                  intermediate_size=5632, num_experts=60, num_experts_per_tok=4,
                  moe_intermediate_size=1408, shared_expert_intermediate_size=5632),
    "57b-a14b": dict(BASE, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4,
                     intermediate_size=18944, num_experts=64, num_experts_per_tok=8,
                     moe_intermediate_size=2560, shared_expert_intermediate_size=20480),
}
LENGTHS = [150, 33, 260, 97]
POOL = 448


class Kept:
    """The plain model's weights, each drawn once on the device and kept for the module."""

    def __init__(self, drawn):
        self.drawn, self.kept = drawn, {}

    def __contains__(self, name):
        return name in self.drawn

    def __getitem__(self, name):
        if name not in self.kept:
            self.kept[name] = self.drawn[name]
        return self.kept[name]


@pytest.fixture(scope="module", params=list(SIZES))
def model(request):
    assert torch.backends.cuda.matmul.allow_tf32 is False
    cfg, seed = SIZES[request.param], 7
    weights = Kept(plain_model.RandomWeights(cfg, seed, device="cuda"))
    reqs = {f"r{i}": random_tokens(n, cfg["vocab_size"], 140 + i) for i, n in enumerate(LENGTHS)}
    want = {r: plain_model.plain_forward(cfg, weights, t).cpu() for r, t in reqs.items()}
    yield cfg, seed, weights, reqs, want
    weights.kept.clear()
    torch.cuda.empty_cache()


@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def runner(request, model):
    from ninfer_amd_mi50_b200.config import EngineOptions
    from ninfer_amd_mi50_b200.engine import load_runner
    cfg, seed = model[0], model[1]
    r = load_runner(config=cfg, random_seed=seed,
                    options=EngineOptions(dtype=request.param, page_size=64, num_sequences=4, max_context=POOL,
                                          cache_tokens=POOL, use_graph=False))
    yield request.param, r
    del r
    torch.cuda.empty_cache()


@pytest.mark.parametrize("how", ["whole", "tail_decoded", "portions", "mixed"])
def test_real_layer_sizes_match_the_plain_model(model, runner, how):
    from test_replay_gpu import check
    cfg, seed, weights, reqs, want = model
    dtype, r = runner
    steps = schedules.mixed(reqs, page=64, pool_tokens=POOL) if how == "mixed" else getattr(schedules, how)(reqs)
    routing = {}
    got = schedules.run_schedule(r, steps, routing)
    assert r.cache.pages_free() == [g.pool.num_pages for g in r.cache.groups]
    from ninfer_amd_mi50_b200 import kernels
    kernels.check_status(how)
    worst = 0.0
    for name, toks in reqs.items():
        ref = want[name]
        if dtype == "bfloat16":
            slack = []
            ref = plain_model.plain_forward(cfg, weights, toks, forced=routing[name], slack=slack).cpu()
            for s in slack:
                assert s.max().item() <= 0.05, f"{how} {name}: an expert was chosen that is no near-tie"
            rounded = plain_model.plain_forward(cfg, weights, toks, dtype=torch.bfloat16,
                                                forced=routing[name]).float().cpu()
            ours = (got[name] - ref).abs().max(dim=1).values.median().item()
            plain = (rounded - ref).abs().max(dim=1).values.median().item()
            assert ours <= plain, f"{how} {name}: median row error {ours:.3e}, the plain model in bfloat16 has {plain:.3e}"
        worst = max(worst, check(got[name], ref, dtype, f"{how} {name}", bf16_bound=3e-2))
    print(f"\n[{cfg['hidden_size']} {dtype} {how}] median row error / scale = {worst:.2e}")


def test_weights_drawn_on_the_device_are_the_plain_model_s(model):
    """The kernel that fills the engine's tensors and the plain restatement give the same bits."""
    from ninfer_amd_mi50_b200.weights import counter_rng
    cfg, seed, weights, _, _ = model
    for name, init in (("model.layers.1.mlp.experts.3.down_proj.weight", "linear"),
                       ("model.layers.0.input_layernorm.weight", "norm"), ("lm_head.weight", "linear")):
        want = weights[name]
        for dtype in (torch.float32, torch.bfloat16):
            got = counter_rng.fill(torch.empty(want.shape, dtype=dtype, device="cuda"),
                                   counter_rng.tensor_keys(seed, name), init)
            assert torch.equal(got.float(), want), name
        assert torch.equal(counter_rng.draw(0, min(want.numel(), 100000), counter_rng.tensor_keys(seed, name), init),
                           want.reshape(-1)[:100000].cpu())
