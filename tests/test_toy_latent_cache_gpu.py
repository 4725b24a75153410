"""Two more things a layer may keep between steps, shown with toy parts defined here and
registered without a change to the package's files (no model of anyone's):

* a mixer whose cache is not keys and values but one latent row per token (`CacheSpec` with
  `row_width`: pages of ``[page_size, row_width]`` that the mixer reads and writes itself through
  the step's block table);
* a block arrangement whose *feed-forward* keeps state of fixed size per request (the block
  answers `state_spec` for it and hands it the slab).

Stepped whole, in portions and mixed with page reuse, in 32-bit and in bfloat16, against a
whole-sequence restatement."""

import math

import pytest
import torch

import plain_model as PM
import schedules
from tiny_configs import random_tokens

pytestmark = pytest.mark.gpu

TOY = {"architectures": ["ToyLatentForCausalLM"], "vocab_size": 211, "hidden_size": 80, "latent": 24,
       "layers": 2, "eps": 1e-5}


@pytest.fixture(scope="module")
def registered():
    from ninfer_amd_mi50_b200 import kernels
    from ninfer_amd_mi50_b200.config import LayerCall, LayerSpec, ModelPlan, PartSpec
    from ninfer_amd_mi50_b200.parts.base import Block, CacheSpec, FeedForward, Mixer, StateSpec, TensorSpec, summed
    from ninfer_amd_mi50_b200.registry import (register_architecture, register_part, unregister_architecture,
                                               unregister_part)

    @register_part("mixer", "toy_latent_attention")
    class ToyLatentAttention(Mixer):
        """c_t = W_c x_t is all that is cached (one row of `latent` numbers a token);
        y_t = W_o sum_j softmax_j(q_t . c_j / sqrt(latent)) c_j over j <= t, q_t = W_q x_t."""

        def __init__(self, hidden_size, latent, prefix):
            self.H, self.R, self.prefix = hidden_size, latent, prefix

        def tensor_specs(self):
            p = self.prefix
            return [TensorSpec(p + "c.weight", (self.R, self.H)), TensorSpec(p + "q.weight", (self.R, self.H)),
                    TensorSpec(p + "o.weight", (self.H, self.R))]

        def load(self, fetch):
            p = self.prefix
            self.wc, self.wq, self.wo = fetch(p + "c.weight"), fetch(p + "q.weight"), fetch(p + "o.weight")

        def cache_spec(self):
            return CacheSpec("full", row_width=self.R)

        def forward(self, x, ctx, cache, state):
            assert cache.pages.shape[1:] == (cache.page_size, self.R)
            c = kernels.linear(x, self.wc)
            q = kernels.linear(x, self.wq, out_dtype=torch.float32)
            out = torch.empty((x.shape[0], self.R), dtype=torch.float32, device=x.device)
            table = cache.block_table.tolist()
            row = 0
            for s, (n, pos0) in enumerate(zip(ctx.seg_len_host, ctx.seg_pos0_host)):
                for i in range(n):                                    # append, then read back through the pages
                    p = pos0 + i
                    cache.pages[table[s][p // cache.page_size], p % cache.page_size] = c[row + i]
                pages = [table[s][lp] for lp in range((pos0 + n + cache.page_size - 1) // cache.page_size)]
                lat = cache.pages[pages].reshape(-1, self.R)[:pos0 + n].float()
                sc = (q[row:row + n] @ lat.T) / math.sqrt(self.R)
                keep = torch.arange(pos0 + n, device=x.device)[None, :] <= (pos0 + torch.arange(n, device=x.device))[:, None]
                out[row:row + n] = torch.softmax(sc.masked_fill(~keep, float("-inf")), dim=-1) @ lat
                row += n
            return kernels.linear(out.to(x.dtype), self.wo)

    @register_part("feed_forward", "toy_running_mean")
    class ToyRunningMean(FeedForward):
        """f_t = W (x_t + mean of x_0 .. x_t): the sum so far and the count live in the request's
        state slot, which the block asks for on this part's behalf."""

        def __init__(self, hidden_size, prefix):
            self.H, self.prefix = hidden_size, prefix

        def tensor_specs(self):
            return [TensorSpec(self.prefix + "w.weight", (self.H, self.H))]

        def load(self, fetch):
            self.w = fetch(self.prefix + "w.weight")

        def state_spec(self):
            return StateSpec((self.H + 1,), torch.float32)

        def forward_with_state(self, x, ctx, state):
            xf = x.float()
            mixed = torch.empty_like(xf)
            row = 0
            for slot, n in zip(ctx.seg_slot.tolist(), ctx.seg_len_host):
                s = state[slot]
                for i in range(row, row + n):
                    s[:self.H] += xf[i]
                    s[self.H] += 1
                    mixed[i] = xf[i] + s[:self.H] / s[self.H]
                row += n
            return kernels.linear(mixed.to(x.dtype), self.w)

    @register_part("block", "toy_stateful_ffn_block")
    class ToyStatefulFfnBlock(Block):
        def __init__(self, norm1, mixer, norm2, feed_forward):
            self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward

        def parts(self):
            return (self.norm1, self.mixer, self.norm2, self.feed_forward)

        def tensor_specs(self):
            return [s for p in self.parts() for s in p.tensor_specs()]

        def load(self, fetch):
            for p in self.parts():
                p.load(fetch)

        def state_spec(self):                       # the feed-forward's, not the mixer's
            return self.feed_forward.state_spec()

        def forward(self, h, pending, ctx, cache, state):
            x1 = self.norm1.add_norm(h, summed(pending), ctx.dtype)
            a = self.mixer.forward(x1, ctx, cache, None)
            x2 = self.norm2.add_norm(h, a, ctx.dtype)
            return self.feed_forward.forward_with_state(x2, ctx, state)

    def build_plan(c):
        norm = PartSpec.make("rms_norm", size=c["hidden_size"], eps=c["eps"])
        mix = PartSpec.make("toy_latent_attention", hidden_size=c["hidden_size"], latent=c["latent"])
        ff = PartSpec.make("toy_running_mean", hidden_size=c["hidden_size"])
        names = (("norm1", "ln1"), ("mixer", "mix"), ("norm2", "ln2"), ("feed_forward", "ff"))
        layers = tuple(LayerSpec("toy_stateful_ffn_block", norm, mix, ff, prefix=f"toy.l{i}.", names=names)
                       for i in range(c["layers"]))
        return ModelPlan(c["vocab_size"], c["hidden_size"], layers, tuple(LayerCall(i, i) for i in range(c["layers"])),
                         norm, True, embedding_name="toy.embed.weight", final_norm_name="toy.norm.")

    register_architecture("ToyLatentForCausalLM", lambda d: d, build_plan)
    yield
    unregister_architecture("ToyLatentForCausalLM")
    unregister_part("mixer", "toy_latent_attention")
    unregister_part("feed_forward", "toy_running_mean")
    unregister_part("block", "toy_stateful_ffn_block")


def toy_plain(cfg, W, tokens):
    T, R = len(tokens), cfg["latent"]
    h = PM.plain_embedding(W["toy.embed.weight"], tokens)
    keep = torch.arange(T)[None, :] <= torch.arange(T)[:, None]
    for i in range(cfg["layers"]):
        p = f"toy.l{i}."
        x = PM.plain_rms_norm(h, W[p + "ln1.weight"], cfg["eps"])
        c, q = x @ W[p + "mix.c.weight"].T, x @ W[p + "mix.q.weight"].T
        att = torch.softmax((q @ c.T / math.sqrt(R)).masked_fill(~keep, float("-inf")), dim=-1) @ c
        h = h + att @ W[p + "mix.o.weight"].T
        x = PM.plain_rms_norm(h, W[p + "ln2.weight"], cfg["eps"])
        mean = torch.cumsum(x, dim=0) / torch.arange(1, T + 1)[:, None]
        h = h + (x + mean) @ W[p + "ff.w.weight"].T
    return PM.plain_rms_norm(h, W["toy.norm.weight"], cfg["eps"]) @ W["toy.embed.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_latent_rows_in_pages_and_a_feed_forward_with_state(registered, tmp_path, dtype):
    from ninfer_amd_mi50_b200.config import EngineOptions
    from ninfer_amd_mi50_b200.engine import load_runner
    from ninfer_amd_mi50_b200.weights import write_random_model
    from test_replay_gpu import check
    d = str(tmp_path / "toy")
    write_random_model(TOY, 9, d)
    cfg, W = PM.read_model_folder(d)
    reqs = {f"r{i}": random_tokens(n, TOY["vocab_size"], 160 + i) for i, n in enumerate([37, 5, 70, 18, 49])}
    want = {r: toy_plain(cfg, W, t) for r, t in reqs.items()}
    for make in (schedules.whole, schedules.portions, lambda r: schedules.mixed(r, page=16, pool_tokens=160)):
        runner = load_runner(d, options=EngineOptions(dtype=dtype, page_size=16, num_sequences=4, max_context=160,
                                                       cache_tokens=160, use_graph=False))
        (group,) = runner.cache.groups
        assert group.pages.shape == (2, 160 // 16 + 1, 16, TOY["latent"])           # rows of latents, no heads
        assert all(s is not None for s in runner.model.state_specs())                # asked for by the blocks
        assert runner.cache.bytes_per_token() == 2 * TOY["latent"] * (4 if dtype == "float32" else 2)
        got = schedules.run_schedule(runner, make(reqs))
        assert runner.cache.pages_free() == [160 // 16]
        for r in reqs:
            check(got[r], want[r], dtype, f"toy latent {r}")
