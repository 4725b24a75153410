"""Each part alone on the GPU against the plain function of the same part, and a toy mixer
with state of its own that is registered, built and stepped without touching the package."""

import math
from types import SimpleNamespace

import pytest
import torch

import plain_model as PM

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)


def fetcher(tensors, dtype):
    from ninfer_amd_mi50_b200.weights import held_dtype

    def fetch_for(specs):
        roles = {s.name: s.role for s in specs}
        return lambda name: tensors[name].to(device="cuda", dtype=held_dtype(roles[name], dtype))
    return fetch_for


def random_tensors(specs, seed):
    g = torch.Generator().manual_seed(seed)
    out = {}
    for s in specs:
        t = torch.randn(s.shape, generator=g)
        out[s.name] = (1 + 0.05 * t if s.init == "norm" else 0.05 * t).to(torch.bfloat16).float()
    return out


def simple_ctx(dtype, seg_lens, page=16):
    """Fresh requests (position 0 onwards), pages handed out in reverse order."""
    T = sum(seg_lens)
    positions, row_seg = [], []
    for s, n in enumerate(seg_lens):
        positions += list(range(n))
        row_seg += [s] * n
    width = max((n + page - 1) // page for n in seg_lens)
    n_pages = sum((n + page - 1) // page for n in seg_lens)
    bt = torch.full((len(seg_lens), width), -1, dtype=torch.int32)
    nxt = n_pages - 1
    for s, n in enumerate(seg_lens):
        for lp in range((n + page - 1) // page):
            bt[s, lp] = nxt
            nxt -= 1
    from ninfer_amd_mi50_b200.parts.base import StepContext
    mk = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    row0 = [0]
    for n in seg_lens:
        row0.append(row0[-1] + n)
    ctx = StepContext(dtype=dtype, device=torch.device("cuda"), T=T, S=len(seg_lens),
                      token_ids=mk([0] * T), positions=mk(positions), row_seg=mk(row_seg),
                      seg_row0=mk(row0), seg_pos0=mk([0] * len(seg_lens)),
                      seg_slot=mk(list(range(len(seg_lens)))), logit_rows=mk([]),
                      seg_len_host=list(seg_lens), seg_pos0_host=[0] * len(seg_lens),
                      max_rows_per_seg=max(seg_lens), max_context=max(seg_lens))
    return ctx, bt.cuda(), n_pages


@pytest.mark.parametrize("dtype", DTYPES)
def test_rms_norm_part(dtype):
    from ninfer_amd_mi50_b200.parts.norm import RmsNorm
    n = RmsNorm(size=200, eps=3e-6, prefix="n.")
    t = random_tensors(n.tensor_specs(), 1)
    n.load(fetcher(t, dtype)(n.tensor_specs()))
    h = torch.randn(9, 200, device="cuda")
    delta = torch.randn(9, 200, device="cuda").to(dtype)
    want_h = h + delta.float()
    out = n.add_norm(h, delta, dtype)
    torch.testing.assert_close(h, want_h)
    torch.testing.assert_close(out.float(), PM.plain_rms_norm(want_h.cpu(), t["n.weight"], 3e-6).cuda(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hq,Hkv,D,window,bias", [(6, 2, 48, None, True), (4, 1, 128, 21, False)])
def test_attention_part(dtype, Hq, Hkv, D, window, bias):
    from ninfer_amd_mi50_b200.config import PartSpec
    from ninfer_amd_mi50_b200.parts.attention import PagedGqaAttention
    from ninfer_amd_mi50_b200.parts.base import CacheView
    H, theta, page = 200, 50000.0, 16
    att = PagedGqaAttention(hidden_size=H, num_heads=Hq, num_kv_heads=Hkv, head_dim=D, qkv_bias=bias,
                            position=PartSpec.make("rotary_half_split", head_dim=D, theta=theta),
                            prefix="a.", window=window)
    t = random_tensors(att.tensor_specs(), 2)
    att.load(fetcher(t, dtype)(att.tensor_specs()))
    seg_lens = [37, 5]
    ctx, bt, n_pages = simple_ctx(dtype, seg_lens, page)
    pages = torch.zeros((n_pages + 1, 2, Hkv, page, D), dtype=dtype, device="cuda")
    x = torch.randn(sum(seg_lens), H).to(torch.bfloat16).float()
    out = att.forward(x.cuda().to(dtype), ctx, CacheView(att.cache_spec(), pages, bt, page, True), None)
    inv = PM.plain_inv_freq(D, theta)
    r0 = 0
    for n in seg_lens:
        xs = x[r0:r0 + n]
        q, k, v = (xs @ t[f"a.{p}_proj.weight"].T + (t[f"a.{p}_proj.bias"] if bias else 0) for p in "qkv")
        pos = torch.arange(n)
        q = PM.plain_rope(q.view(n, Hq, D), pos, inv)
        k = PM.plain_rope(k.view(n, Hkv, D), pos, inv)
        want = PM.plain_attention(q, k, v.view(n, Hkv, D), window) @ t["a.o_proj.weight"].T
        torch.testing.assert_close(out[r0:r0 + n].float().cpu(), want, **tol(dtype))
        r0 += n


@pytest.mark.parametrize("dtype", DTYPES)
def test_dense_and_sparse_feed_forward_parts(dtype):
    from ninfer_amd_mi50_b200.parts.base import summed
    from ninfer_amd_mi50_b200.parts.feedforward import DenseSwiglu, SparseMoeSwiglu
    H = 200
    x = torch.randn(23, H).to(torch.bfloat16).float()
    ctx = SimpleNamespace()
    dense = DenseSwiglu(hidden_size=H, intermediate_size=232, prefix="m.")
    t = random_tensors(dense.tensor_specs(), 3)
    dense.load(fetcher(t, dtype)(dense.tensor_specs()))
    want = PM.plain_swiglu_mlp(x, t["m.gate_proj.weight"], t["m.up_proj.weight"], t["m.down_proj.weight"])
    torch.testing.assert_close(dense.forward(x.cuda().to(dtype), ctx).float().cpu(), want, **tol(dtype))
    for norm_topk, shared in ((True, 104), (False, 0)):
        moe = SparseMoeSwiglu(hidden_size=H, num_experts=6, top_k=3, norm_topk_prob=norm_topk,
                              moe_intermediate_size=72, shared_intermediate_size=shared, prefix="m.")
        t = random_tensors(moe.tensor_specs(), 4)
        moe.load(fetcher(t, dtype)(moe.tensor_specs()))
        cfg = {"num_experts": 6, "num_experts_per_tok": 3, "norm_topk_prob": norm_topk,
               "shared_expert_intermediate_size": shared}
        want = PM.plain_sparse_ffn(x, t, "m.", cfg)
        got = summed(moe.forward(x.cuda().to(dtype), ctx)).float().cpu()
        if dtype == torch.float32:
            torch.testing.assert_close(got, want, **tol(dtype))
        else:
            # a row whose k-th and (k+1)-th experts are within rounding may take the other one
            bad = ((got - want).abs().max(dim=1).values > 3e-2).sum().item()
            assert bad <= 2


@pytest.mark.parametrize("H,k,T", [(200, 3, 23), (2048, 4, 9), (3584, 8, 130), (8192, 2, 3)])
@pytest.mark.parametrize("with_shared", [True, False])
def test_norm_adds_up_the_routed_sum_in_its_own_kernel(H, k, T, with_shared):
    """A routed feed-forward hands its output on unsummed; the RMS norm adds it up, adds it to
    the residual row and normalises in one kernel.  The bits are those of the three steps done
    apart (combine, add, norm), for whole steps (the residual is updated) and for chosen rows
    (it is not)."""
    from ninfer_amd_mi50_b200 import kernels
    from ninfer_amd_mi50_b200.parts.base import RoutedSum
    from ninfer_amd_mi50_b200.parts.norm import RmsNorm
    g = torch.Generator().manual_seed(H + k)
    E = 2 * k + 1
    idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32).cuda()
    plan = kernels.moe_plan(idx, E)
    y = torch.randn(T * k, H, generator=g).to(torch.bfloat16).cuda()
    wts = torch.rand(T, k, generator=g).cuda()
    shared = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda() if with_shared else None
    gate = torch.randn(T, 1, generator=g).cuda() if with_shared else None
    norm = RmsNorm(size=H, eps=1e-6, prefix="n.")
    norm.weight = (1 + 0.05 * torch.randn(H, generator=g)).cuda()
    h0 = torch.randn(T, H, generator=g).cuda()
    delta = RoutedSum(y, plan, wts, shared, gate, torch.bfloat16)
    assert norm._fusable(delta, torch.bfloat16, min(T, 64))
    kernels.TUNING["fuse_combine_norm_max_rows"] = 10 ** 9
    h1, h2 = h0.clone(), h0.clone()
    fused = norm.add_norm(h1, delta, torch.bfloat16)
    apart = norm.add_norm(h2, delta.materialize(), torch.bfloat16)
    assert torch.equal(fused, apart) and torch.equal(h1, h2) and not torch.equal(h1, h0)
    rows = torch.tensor([T - 1, 0, T // 2], dtype=torch.int32).cuda()
    h3 = h0.clone()
    fused = norm.add_norm_rows(h3, delta, rows, torch.bfloat16)
    apart = norm.add_norm_rows(h0.clone(), delta.materialize(), rows, torch.bfloat16)
    assert torch.equal(fused, apart) and torch.equal(h3, h0)
    kernels.TUNING["fuse_combine_norm_max_rows"] = 64
    assert kernels.index_status() == 0
    # a wider row than the kernel keeps in registers, many rows, or float32: the three steps are done apart
    assert not kernels.can_fuse_combine_norm(y, 8192 + 4, 1)
    assert not kernels.can_fuse_combine_norm(y, H, 65)
    assert not norm._fusable(RoutedSum(y.float(), plan, wts, None, None, torch.float32), torch.float32, 1)


def test_rotary_table_follows_single_precision_pow():
    from ninfer_amd_mi50_b200.parts.position import rotary_inverse_frequencies
    for D, theta in ((64, 10000.0), (128, 1e6), (48, 50000.0)):
        assert torch.equal(rotary_inverse_frequencies(D, theta), PM.plain_inv_freq(D, theta))
