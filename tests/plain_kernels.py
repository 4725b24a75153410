"""Plain PyTorch restatements of each kernel operation, with the kernels' signatures.

Two uses.  GPU tests call a CUDA kernel and its plain twin on the same inputs and compare.
CPU tests substitute these for the kernels (`install`) so that the engine's own logic
- cache manager, step function, scheduler - can be exercised without a GPU.  They are test
doubles, not a second implementation of the product: the package never imports this file.

All arithmetic is float32 (or the input's dtype if wider); outputs are rounded to the
dtype the kernel would write.
"""

from __future__ import annotations

import math
from typing import Optional

import torch


def _f(t):
    return t.to(torch.float32) if t.dtype in (torch.bfloat16, torch.float16) else t


def embed_rows(table, ids, out):
    out.copy_(_f(table)[ids.long()])


def add_rmsnorm(h, delta, weight, eps, out):
    if delta is not None:
        h.add_(_f(delta))
    inv = torch.rsqrt((h * h).mean(dim=-1, keepdim=True) + eps)
    out.copy_((h * inv * weight).to(out.dtype))


def add_rmsnorm_rows(h, delta, rows, weight, eps, out):
    v = h[rows.long()]
    if delta is not None:
        v = v + _f(delta[rows.long()])
    inv = torch.rsqrt((v * v).mean(dim=-1, keepdim=True) + eps)
    out.copy_((v * inv * weight).to(out.dtype))


def silu_mul(gate_up):
    inner = gate_up.shape[1] // 2
    g, u = _f(gate_up[:, :inner]), _f(gate_up[:, inner:])
    return (g / (1 + torch.exp(-g)) * u).to(gate_up.dtype)


def linear(x, w, out_dtype=None):
    return (_f(x) @ _f(w).T).to(out_dtype or x.dtype)


def linear_swiglu(x, w_gate_up):
    inner = w_gate_up.shape[0] // 2
    gu = _f(x) @ _f(w_gate_up).T
    g, u = gu[:, :inner], gu[:, inner:]
    return (g / (1 + torch.exp(-g)) * u).to(x.dtype)


def rope_append(qkv, bias, positions, row_seg, inv_freq, rotary_dim, Hq, Hkv, D, pages,
                block_table, page_size, append):
    T = qkv.shape[0]
    x = _f(qkv).clone()
    if bias is not None:
        x = x + bias
    x = x.view(T, Hq + 2 * Hkv, D)
    if inv_freq is not None and rotary_dim > 0:
        half = rotary_dim // 2
        ang = positions.to(torch.float32)[:, None] * inv_freq[None, :]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        qk = x[:, :Hq + Hkv]
        a, b = qk[..., :half].clone(), qk[..., half:rotary_dim].clone()
        qk[..., :half] = a * c - b * s
        qk[..., half:rotary_dim] = a * s + b * c
    qkv[:, :Hq * D] = x[:, :Hq].reshape(T, Hq * D).to(qkv.dtype)
    if not append:
        return
    for t in range(T):
        pos = int(positions[t])
        page = int(block_table[int(row_seg[t]), pos // page_size])
        assert page >= 0, "no page reserved for a position that is written"
        pages[page, 0, :, pos % page_size, :] = x[t, Hq:Hq + Hkv].to(pages.dtype)
        pages[page, 1, :, pos % page_size, :] = x[t, Hq + Hkv:].to(pages.dtype)


def linear_rope_append(x, w_qkv, bias, positions, row_seg, inv_freq, rotary_dim, Hq, Hkv, D, pages,
                       block_table, page_size, append):
    qkv = linear(x, w_qkv)
    rope_append(qkv, bias, positions, row_seg, inv_freq, rotary_dim, Hq, Hkv, D, pages, block_table,
                page_size, append)
    return qkv


def paged_attention(qkv, Hq, Hkv, D, pages, block_table, page_size, ctx, window, scale):
    T = qkv.shape[0]
    out = torch.zeros((T, Hq * D), dtype=torch.float32, device=qkv.device)
    rep = Hq // Hkv
    for t in range(T):
        pos = int(ctx.positions[t])
        seg = int(ctx.row_seg[t])
        lo = max(0, pos - window + 1) if window > 0 else 0
        js = list(range(lo, pos + 1))
        pg = [int(block_table[seg, j // page_size]) for j in js]
        assert all(p >= 0 for p in pg), "attention reads a page that was released"
        k = torch.stack([_f(pages[p, 0, :, j % page_size, :]) for p, j in zip(pg, js)])  # [n, Hkv, D]
        v = torch.stack([_f(pages[p, 1, :, j % page_size, :]) for p, j in zip(pg, js)])
        q = _f(qkv[t, :Hq * D]).view(Hq, D)
        for h in range(Hq):
            s = (k[:, h // rep] @ q[h]) * scale
            p = torch.softmax(s, dim=0)
            out[t, h * D:(h + 1) * D] = p @ v[:, h // rep]
    return out.to(qkv.dtype)


class MoePlan:
    def __init__(self, offsets, order, inv, num_experts, num_tokens, top_k, active=None):
        self.offsets, self.order, self.inv = offsets, order, inv
        self.num_experts, self.num_tokens, self.top_k = num_experts, num_tokens, top_k
        self.active = active


def split_router(w_router):
    return None


def router_topk(x, w_router, E, k, norm_topk, split=None):
    logits = _f(x) @ w_router.T
    extra = logits[:, E:].contiguous() if w_router.shape[0] > E else None
    p = torch.softmax(logits[:, :E], dim=-1)
    T = x.shape[0]
    idx = torch.zeros((T, k), dtype=torch.int32, device=x.device)
    wts = torch.zeros((T, k), dtype=torch.float32, device=x.device)
    pc = p.cpu()
    for t in range(T):
        order = sorted(range(E), key=lambda e: (-float(pc[t, e]), e))[:k]
        idx[t] = torch.tensor(order, dtype=torch.int32)
        wts[t] = p[t, order]
    if norm_topk:
        wts = wts / wts.sum(dim=-1, keepdim=True)
    return idx, wts, extra


def moe_plan(topk_idx, E):
    T, k = topk_idx.shape
    flat = topk_idx.reshape(-1).cpu().tolist()
    order = sorted(range(T * k), key=lambda i: (flat[i], i))       # stable by expert
    inv = [0] * (T * k)
    for p, i in enumerate(order):
        inv[i] = p
    counts = [0] * E
    for e in flat:
        counts[e] += 1
    offsets = [0]
    for c in counts:
        offsets.append(offsets[-1] + c)
    dev = topk_idx.device
    mk = lambda l: torch.tensor(l, dtype=torch.int32, device=dev)
    n_act = min(E, max(T * k, 1))
    act = [e for e in range(E) if counts[e] > 0]
    return MoePlan(mk(offsets), mk(order), mk(inv), E, T, k, mk(act + [-1] * (n_act - len(act))))


def route(x, w_router, E, k, norm_topk, split=None):
    idx, wts, ext = router_topk(x, w_router, E, k, norm_topk)
    return idx, wts, ext, moe_plan(idx, E)


def moe_experts(x, w13, w2, plan, k, gathered=None):
    return moe_gemm2(moe_gemm1(x, w13, plan, k), w2, plan)


def moe_gemm1(x, w13, plan, k, gathered=None):
    T, H = x.shape
    E, two_i, _ = w13.shape
    inner = two_i // 2
    act = torch.zeros((T * k, inner), dtype=torch.float32, device=x.device)
    off = plan.offsets.cpu().tolist()
    order = plan.order.cpu().tolist()
    for e in range(E):
        for p in range(off[e], off[e + 1]):
            xr = _f(x[order[p] // k])
            gu = _f(w13[e]) @ xr
            g, u = gu[:inner], gu[inner:]
            act[p] = g / (1 + torch.exp(-g)) * u
    return act.to(x.dtype)


def moe_gemm2(act, w2, plan, plan_is_older=False):
    n, inner = act.shape
    E, H, _ = w2.shape
    y = torch.zeros((n, H), dtype=torch.float32, device=act.device)
    off = plan.offsets.cpu().tolist()
    for e in range(E):
        if off[e + 1] > off[e]:
            y[off[e]:off[e + 1]] = _f(act[off[e]:off[e + 1]]) @ _f(w2[e]).T
    return y.to(act.dtype)


def moe_combine(y, plan, wts, shared, gate, out_dtype):
    T, k = wts.shape
    inv = plan.inv.view(T, k).long()
    out = torch.zeros((T, y.shape[1]), dtype=torch.float32, device=y.device)
    for j in range(k):
        out += wts[:, j:j + 1] * _f(y[inv[:, j]])
    if shared is not None:
        s = _f(shared)
        if gate is not None:
            s = s * (1 / (1 + torch.exp(-gate[:, :1])))
        out += s
    return out.to(out_dtype)


def argmax_rows(logits):
    return torch.argmax(logits, dim=-1).to(torch.int32)


def can_pack(n_features, K):
    return False


class PackedWeights:
    pass


def chain_break():
    pass


def check_head_dim(head_dim):
    pass


def check_router_sizes(num_experts, top_k):
    pass


NAMES = ["chain_break", "can_pack", "PackedWeights", "split_router", "embed_rows", "add_rmsnorm", "add_rmsnorm_rows", "silu_mul", "linear", "linear_swiglu",
         "rope_append", "linear_rope_append", "paged_attention", "router_topk", "route", "moe_plan", "moe_experts", "moe_gemm1", "moe_gemm2",
         "moe_combine", "argmax_rows"]


def install(monkeypatch) -> None:
    """Substitute the plain twins for the CUDA kernels (CPU tests of the engine's logic)."""
    import ninfer_amd_mi50_b200.kernels as K
    g = globals()
    for n in NAMES:
        monkeypatch.setattr(K, n, g[n], raising=False)
