"""Generality of the parts: a toy architecture defined here - a mixer with per-request state
of its own, a feed-forward that routes rows between two matrices, a position encoding of
another form (adjacent pairs turned, not half-split), a layer that reads another layer's
cache, a layer named twice in the order - is registered, written as a random model folder,
loaded and stepped under every way of cutting the work, without a change to the package's
files.  It is no model of anyone's."""

import json
import math
import os

import pytest
import torch

import plain_model as PM
import schedules
from tiny_configs import random_tokens

pytestmark = pytest.mark.gpu

TOY = {"architectures": ["ToyStateForCausalLM"], "vocab_size": 301, "hidden_size": 96, "state_size": 40,
       "num_heads": 3, "num_kv_heads": 1, "head_dim": 32, "intermediate_size": 136, "eps": 2e-6,
       "theta": 7000.0}


@pytest.fixture(scope="module")
def toy_registered():
    from ninfer_amd_mi50_b200 import kernels
    from ninfer_amd_mi50_b200.config import LayerCall, LayerSpec, ModelPlan, PartSpec
    from ninfer_amd_mi50_b200.parts.base import FeedForward, Mixer, PositionEncoding, StateSpec, TensorSpec
    from ninfer_amd_mi50_b200.registry import (register_architecture, register_part,
                                               unregister_architecture, unregister_part)

    @register_part("mixer", "toy_running_state")
    class ToyRunningState(Mixer):
        """s_t = sigmoid(decay) * s_{t-1} + W_in x_t ;  y_t = W_out s_t.  The state lives in the
        request's slot and is carried from one portion of a prompt to the next."""

        def __init__(self, hidden_size, state_size, prefix):
            self.H, self.S, self.prefix = hidden_size, state_size, prefix

        def tensor_specs(self):
            p = self.prefix
            return [TensorSpec(p + "in_proj.weight", (self.S, self.H)),
                    TensorSpec(p + "out_proj.weight", (self.H, self.S)),
                    TensorSpec(p + "decay", (self.S,), role="vector")]

        def load(self, fetch):
            p = self.prefix
            self.w_in, self.w_out = fetch(p + "in_proj.weight"), fetch(p + "out_proj.weight")
            self.decay = fetch(p + "decay")

        def state_spec(self):
            return StateSpec((self.S,), torch.float32)

        def forward(self, x, ctx, cache, state):
            assert cache is None and state is not None
            u = kernels.linear(x, self.w_in, out_dtype=torch.float32)
            a = torch.sigmoid(self.decay)
            out = torch.empty_like(u)
            row = 0
            for slot, n in zip(ctx.seg_slot.tolist(), ctx.seg_len_host):
                s = state[slot]
                for i in range(row, row + n):
                    s = a * s + u[i]
                    out[i] = s
                state[slot] = s
                row += n
            return kernels.linear(out.to(x.dtype), self.w_out)

    @register_part("feed_forward", "toy_sign_router")
    class ToySignRouter(FeedForward):
        """A row goes through matrix 1 if its projection on a routing vector is positive, else
        through matrix 0 (the decision is taken in float32 on the row as the engine holds it)."""

        def __init__(self, hidden_size, prefix):
            self.H, self.prefix = hidden_size, prefix

        def tensor_specs(self):
            p = self.prefix
            return [TensorSpec(p + "route", (self.H,), role="vector"),
                    TensorSpec(p + "w0.weight", (self.H, self.H)), TensorSpec(p + "w1.weight", (self.H, self.H))]

        def load(self, fetch):
            p = self.prefix
            self.route, self.w = fetch(p + "route"), [fetch(p + "w0.weight"), fetch(p + "w1.weight")]

        def forward(self, x, ctx):
            up = (x.float() @ self.route) > 0
            out = torch.empty_like(x)
            for e in (0, 1):
                rows = torch.nonzero(up == bool(e)).flatten()
                if rows.numel():
                    out[rows] = kernels.linear(x[rows].contiguous(), self.w[e])
            return out

    @register_part("position", "toy_adjacent_pairs")
    class ToyAdjacentPairs(PositionEncoding):
        """Dims (2i, 2i + 1) are turned by pos * theta^(-2i/D): not the half-split form, so
        there is no table for the fused kernel and `apply` does the work."""

        def __init__(self, head_dim, theta):
            self.D, self.theta = head_dim, theta

        def apply(self, q, k, positions):
            inv = torch.tensor([self.theta ** (-2.0 * i / self.D) for i in range(self.D // 2)],
                               dtype=torch.float32, device=q.device)
            ang = positions.float()[:, None] * inv[None, :]
            c, sn = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
            for t in (q, k):
                a, b = t[..., 0::2].float().clone(), t[..., 1::2].float().clone()
                t[..., 0::2] = (a * c - b * sn).to(t.dtype)
                t[..., 1::2] = (a * sn + b * c).to(t.dtype)

    def build_plan(c):
        norm = PartSpec.make("rms_norm", size=c["hidden_size"], eps=c["eps"])
        ffn = PartSpec.make("dense_swiglu", hidden_size=c["hidden_size"], intermediate_size=c["intermediate_size"])
        att = PartSpec.make("paged_gqa_attention", hidden_size=c["hidden_size"], num_heads=c["num_heads"],
                            num_kv_heads=c["num_kv_heads"], head_dim=c["head_dim"], qkv_bias=False,
                            position=PartSpec.make("rotary_half_split", head_dim=c["head_dim"], theta=c["theta"]))
        toy = PartSpec.make("toy_running_state", hidden_size=c["hidden_size"], state_size=c["state_size"])
        att2 = PartSpec.make("paged_gqa_attention", hidden_size=c["hidden_size"], num_heads=c["num_heads"],
                             num_kv_heads=c["num_kv_heads"], head_dim=c["head_dim"], qkv_bias=False,
                             position=PartSpec.make("toy_adjacent_pairs", head_dim=c["head_dim"], theta=c["theta"]))
        routed = PartSpec.make("toy_sign_router", hidden_size=c["hidden_size"])
        names = (("norm1", "ln1"), ("mixer", "mix"), ("norm2", "ln2"), ("feed_forward", "ff"))
        layers = tuple(LayerSpec("pre_norm", norm, m, f, prefix=f"toy.l{i}.", names=names)
                       for i, (m, f) in enumerate(((toy, ffn), (att, ffn), (att, ffn), (att2, routed))))
        # layer 2 reads layer 1's cache; layer 1 runs a second time, reading what it wrote;
        # layer 3 has the other position encoding, the routed feed-forward and a cache of its own
        order = (LayerCall(0, 0), LayerCall(1, 1, True), LayerCall(2, 1, False), LayerCall(1, 1, False),
                 LayerCall(3, 3, True))
        return ModelPlan(c["vocab_size"], c["hidden_size"], layers, order, norm, True,
                         embedding_name="toy.embed.weight", final_norm_name="toy.norm.", head_name="toy.head.weight")

    register_architecture("ToyStateForCausalLM", lambda d: d, build_plan)
    yield
    unregister_architecture("ToyStateForCausalLM")
    unregister_part("mixer", "toy_running_state")
    unregister_part("feed_forward", "toy_sign_router")
    unregister_part("position", "toy_adjacent_pairs")


def toy_plain(cfg, W, tokens):
    """Whole-sequence restatement of the toy model with the plain model's part functions."""
    H, Hq, Hkv, D = cfg["hidden_size"], cfg["num_heads"], cfg["num_kv_heads"], cfg["head_dim"]
    T = len(tokens)
    inv = PM.plain_inv_freq(D, cfg["theta"])
    pos = torch.arange(T)
    h = PM.plain_embedding(W["toy.embed.weight"], tokens)

    def ffn(i, x):
        p = f"toy.l{i}.ff."
        return PM.plain_swiglu_mlp(x, W[p + "gate_proj.weight"], W[p + "up_proj.weight"], W[p + "down_proj.weight"])

    def attn(i, x, kv=None):
        p = f"toy.l{i}.mix."
        q = PM.plain_rope((x @ W[p + "q_proj.weight"].T).view(T, Hq, D), pos, inv)
        if kv is None:
            k = PM.plain_rope((x @ W[p + "k_proj.weight"].T).view(T, Hkv, D), pos, inv)
            kv = (k, (x @ W[p + "v_proj.weight"].T).view(T, Hkv, D))
        return PM.plain_attention(q, kv[0], kv[1]) @ W[p + "o_proj.weight"].T, kv

    # layer 0: the running state
    x = PM.plain_rms_norm(h, W["toy.l0.ln1.weight"], cfg["eps"])
    u = x @ W["toy.l0.mix.in_proj.weight"].T
    a = torch.sigmoid(W["toy.l0.mix.decay"])
    s = torch.zeros(cfg["state_size"])
    ys = []
    for t in range(T):
        s = a * s + u[t]
        ys.append(s)
    h = h + torch.stack(ys) @ W["toy.l0.mix.out_proj.weight"].T
    h = h + ffn(0, PM.plain_rms_norm(h, W["toy.l0.ln2.weight"], cfg["eps"]))
    # layer 1 (writes the cache), layer 2 (reads it), layer 1 again (reads it)
    kv = None
    for i in (1, 2, 1):
        o, kv_new = attn(i, PM.plain_rms_norm(h, W[f"toy.l{i}.ln1.weight"], cfg["eps"]), kv)
        kv = kv or kv_new
        h = h + o
        h = h + ffn(i, PM.plain_rms_norm(h, W[f"toy.l{i}.ln2.weight"], cfg["eps"]))
    # layer 3: adjacent pairs turned, then the routed feed-forward
    p = "toy.l3.mix."
    x = PM.plain_rms_norm(h, W["toy.l3.ln1.weight"], cfg["eps"])
    ang = pos.float()[:, None] * torch.tensor([cfg["theta"] ** (-2.0 * i / D) for i in range(D // 2)])[None, :]
    c, sn = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]

    def turn(t):
        a, b = t[..., 0::2], t[..., 1::2]
        out = torch.empty_like(t)
        out[..., 0::2], out[..., 1::2] = a * c - b * sn, a * sn + b * c
        return out
    q = turn((x @ W[p + "q_proj.weight"].T).view(T, Hq, D))
    k = turn((x @ W[p + "k_proj.weight"].T).view(T, Hkv, D))
    v = (x @ W[p + "v_proj.weight"].T).view(T, Hkv, D)
    h = h + PM.plain_attention(q, k, v) @ W[p + "o_proj.weight"].T
    x = PM.plain_rms_norm(h, W["toy.l3.ln2.weight"], cfg["eps"])
    side = x @ W["toy.l3.ff.route"]
    up = side > 0
    # how far a row is from the switch, as the cosine between the row and the routing vector: a
    # row within rounding of it may go either way in bfloat16 (the layer is the last, so only
    # the row's own logits depend on it)
    margin = side.abs() / (x.norm(dim=-1) * W["toy.l3.ff.route"].norm())
    h = h + torch.where(up[:, None], x @ W["toy.l3.ff.w1.weight"].T, x @ W["toy.l3.ff.w0.weight"].T)
    return PM.plain_rms_norm(h, W["toy.norm.weight"], cfg["eps"]) @ W["toy.embed.weight"].T, margin


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_steps_under_every_cut(toy_registered, tmp_path, dtype):
    from ninfer_amd_mi50_b200.config import EngineOptions
    from ninfer_amd_mi50_b200.engine import load_runner
    from ninfer_amd_mi50_b200.weights import write_random_model
    from test_replay_gpu import check
    d = str(tmp_path / "toy")
    write_random_model(TOY, 4, d)
    cfg, W = PM.read_model_folder(d)
    reqs = {f"r{i}": random_tokens(n, TOY["vocab_size"], 60 + i) for i, n in enumerate([40, 9, 77, 23, 58])}
    want, clear = {}, {}
    for r, t in reqs.items():
        want[r], margin = toy_plain(cfg, W, t)
        # float32 decides like the plain model; bfloat16 is judged on the rows that are not within
        # rounding of the switch (every one of them, to the rounding bound)
        clear[r] = torch.ones_like(margin, dtype=torch.bool) if dtype == "float32" else margin > 0.01
    assert sum(c.sum().item() for c in clear.values()) >= 0.8 * sum(len(t) for t in reqs.values())
    for make in (schedules.whole, schedules.portions, lambda r: schedules.mixed(r, page=16, pool_tokens=192)):
        runner = load_runner(d, options=EngineOptions(dtype=dtype, page_size=16, num_sequences=4,
                                                       max_context=192, cache_tokens=192, use_graph=False))
        assert [s is not None for s in runner.model.state_specs()] == [True, False, False, False]
        assert len(runner.cache.groups) == 1 and runner.cache.groups[0].slots == [1, 2, 3]
        got = schedules.run_schedule(runner, make(reqs))
        for r in reqs:
            check(got[r][clear[r]], want[r][clear[r]], dtype, f"toy {r}")
