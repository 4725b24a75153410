"""Each CUDA kernel alone against its plain PyTorch twin, at sizes other than the engine's:
widths that are no power of two, head sizes in steps of 16, odd row counts."""

import math
from types import SimpleNamespace

import pytest
import torch

import plain_kernels as P

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, scale=1.0):
    return dict(rtol=2e-5, atol=2e-5 * scale) if dtype == torch.float32 else dict(rtol=1.6e-2, atol=1.6e-2 * scale)


def close(out, ref, dtype):
    """Sums of many products: the error of float32 accumulation grows with the magnitude of
    the largest result, so the absolute bound is relative to it; a bfloat16 result carries
    its own rounding (2^-9 relative) on top."""
    out, ref = out.float(), ref.float()
    top = ref.abs().max().item()
    if dtype == torch.float32:
        torch.testing.assert_close(out, ref, rtol=1e-5, atol=2e-5 * top)
    else:
        torch.testing.assert_close(out, ref, rtol=2 ** -7, atol=1e-3 * top)


@pytest.fixture(scope="module")
def K():
    from ninfer_amd_mi50_b200 import kernels
    kernels.load()
    return kernels


@pytest.fixture(params=["auto", "simt"])
def bf16_path(request, K):
    """Run a test once with the kernels the engine would pick and once with the plain
    CUDA-core kernels forced, so that both stay covered."""
    old = dict(K.TUNING)
    if request.param == "simt":
        K.TUNING.update(bf16_linear="simt", bf16_moe="simt", bf16_attention="generic")
    yield request.param
    K.TUNING.update(old)


def rnd(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).cuda()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("V,H,T", [(777, 200, 13), (2003, 96, 1)])
def test_embed_rows(K, dtype, V, H, T):
    table = rnd((V, H), dtype, 1)
    ids = torch.randint(0, V, (T,), dtype=torch.int32).cuda()
    out = torch.empty((T, H), dtype=torch.float32, device="cuda")
    K.embed_rows(table, ids, out)
    ref = torch.empty_like(out)
    P.embed_rows(table, ids, ref)
    assert torch.equal(out, ref)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H", [(5, 200), (33, 1000), (1, 7168)])
def test_add_rmsnorm(K, dtype, T, H):
    h = rnd((T, H), torch.float32, 2)
    delta = rnd((T, H), dtype, 3)
    w = 1 + 0.05 * rnd((H,), torch.float32, 4)
    out = torch.empty((T, H), dtype=dtype, device="cuda")
    h2, ref = h.clone(), torch.empty_like(out)
    K.add_rmsnorm(h, delta, w, 1e-5, out)
    P.add_rmsnorm(h2, delta, w, 1e-5, ref)
    torch.testing.assert_close(h, h2, rtol=0, atol=0)
    torch.testing.assert_close(out.float(), ref.float(), **tol(dtype))
    # without a delta, and the gathered form that leaves h alone
    out0, ref0 = torch.empty_like(out), torch.empty_like(out)
    K.add_rmsnorm(h, None, w, 1e-5, out0)
    P.add_rmsnorm(h2, None, w, 1e-5, ref0)
    torch.testing.assert_close(out0.float(), ref0.float(), **tol(dtype))
    rows = torch.tensor([T - 1, 0, T // 2], dtype=torch.int32).cuda()
    outr = torch.empty((3, H), dtype=dtype, device="cuda")
    refr = torch.empty_like(outr)
    before = h.clone()
    K.add_rmsnorm_rows(h, delta, rows, w, 1e-5, outr)
    P.add_rmsnorm_rows(h2, delta, rows, w, 1e-5, refr)
    assert torch.equal(h, before)
    torch.testing.assert_close(outr.float(), refr.float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K_", [(1, 200, 200), (37, 300, 72), (130, 65, 1000), (3, 2003, 96),
                                     (8, 2816, 2048), (64, 48, 1408), (17, 100, 36)])
def test_linear(K, dtype, M, N, K_, bf16_path):
    x, w = rnd((M, K_), dtype, 5), rnd((N, K_), dtype, 6, 0.05)
    for od in (None, torch.float32):
        out = K.linear(x, w, out_dtype=od)
        ref = P.linear(x, w, out_dtype=od)
        close(out, ref, out.dtype)


@pytest.mark.parametrize("M,N,K_", [(1, 2048, 5632), (8, 2048, 2048), (16, 3584, 20480), (3, 200, 1000), (9, 96, 1288)])
def test_dense_product_split_over_k_by_a_cluster(K, M, N, K_):
    """Few features and a long k: clusters of 2 or 4 CTAs share a feature tile, split k and add
    their sums in the first member's shared memory, in member order.  Against the plain twin,
    against the same kernel without the split (another order of the sum: close, not equal), and
    twice (same bits)."""
    dtype = torch.bfloat16
    x, w = rnd((M, K_), dtype, 71), rnd((N, K_), dtype, 72, 0.05)
    lib = K.load()
    split = [K.linear(x, w) for _ in range(2)]
    head = K.linear(x, w, out_dtype=torch.float32)
    try:
        lib.nf_set_skinny_max_split(1)
        whole = K.linear(x, w)
    finally:
        lib.nf_set_skinny_max_split(4)
    assert torch.equal(split[0], split[1])
    close(split[0], P.linear(x, w), dtype)
    close(split[0], whole, dtype)
    close(head, x.float() @ w.float().T, torch.float32 if False else dtype)
    gu = rnd((2 * 104, K_), dtype, 73, 0.05)
    a = K.linear_swiglu(x, gu)
    close(a, P.linear_swiglu(x, gu), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,I,K_", [(1, 72, 200), (37, 100, 96), (70, 33, 300), (9, 1408, 2048)])
def test_linear_swiglu_and_silu_mul(K, dtype, M, I, K_, bf16_path):
    x, w = rnd((M, K_), dtype, 7), rnd((2 * I, K_), dtype, 8, 0.1)
    close(K.linear_swiglu(x, w), P.linear_swiglu(x, w), dtype)
    gu = rnd((M, 2 * I), dtype, 9)
    torch.testing.assert_close(K.silu_mul(gu).float(), P.silu_mul(gu).float(), **tol(dtype))


def make_cache_case(dtype, Hq, Hkv, D, page, seg_lens, pos0s, n_pages, seed):
    """A batch of segments with scattered pages; returns everything the attention ops need."""
    g = torch.Generator().manual_seed(seed)
    S = len(seg_lens)
    width = max((p + n + page - 1) // page for p, n in zip(pos0s, seg_lens))
    perm = torch.randperm(n_pages, generator=g).tolist()
    bt = torch.full((S, width), -1, dtype=torch.int32)
    for s, (p0, n) in enumerate(zip(pos0s, seg_lens)):
        for lp in range((p0 + n + page - 1) // page):
            bt[s, lp] = perm.pop()
    pages = (torch.randn((n_pages, 2, Hkv, page, D), generator=g)).to(dtype).cuda()
    positions, row_seg = [], []
    for s, (p0, n) in enumerate(zip(pos0s, seg_lens)):
        positions += list(range(p0, p0 + n))
        row_seg += [s] * n
    T = len(positions)
    ctx = SimpleNamespace(positions=torch.tensor(positions, dtype=torch.int32).cuda(),
                          row_seg=torch.tensor(row_seg, dtype=torch.int32).cuda())
    qkv = (torch.randn((T, (Hq + 2 * Hkv) * D), generator=g)).to(dtype).cuda()
    return pages, bt.cuda(), ctx, qkv


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hq,Hkv,D,page,rot", [(6, 2, 48, 16, 48), (4, 1, 128, 64, 128), (5, 5, 80, 32, 32)])
def test_rope_append(K, dtype, Hq, Hkv, D, page, rot):
    pages, bt, ctx, qkv = make_cache_case(dtype, Hq, Hkv, D, page, [5, 1, 19], [0, 77, 30], 12, 11)
    bias = 0.1 * rnd(((Hq + 2 * Hkv) * D,), torch.float32, 12)
    inv_freq = torch.tensor([10000.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float32).cuda()
    q1, p1 = qkv.clone(), pages.clone()
    q2, p2 = qkv.clone(), pages.clone()
    K.rope_append(q1, bias, ctx.positions, ctx.row_seg, inv_freq, rot, Hq, Hkv, D, p1, bt, page, True)
    P.rope_append(q2, bias, ctx.positions, ctx.row_seg, inv_freq, rot, Hq, Hkv, D, p2, bt, page, True)
    torch.testing.assert_close(q1[:, :Hq * D].float(), q2[:, :Hq * D].float(), **tol(dtype, 3))
    torch.testing.assert_close(p1.float(), p2.float(), **tol(dtype, 3))
    # without appending the cache stays as it was; without a table nothing rotates
    q3, p3 = qkv.clone(), pages.clone()
    K.rope_append(q3, None, ctx.positions, ctx.row_seg, None, 0, Hq, Hkv, D, p3, bt, page, False)
    assert torch.equal(p3, pages) and torch.equal(q3, qkv)


@pytest.mark.parametrize("Hq,Hkv,D,page,H,rows", [(4, 1, 128, 64, 256, 3), (6, 2, 48, 16, 200, 11), (16, 16, 128, 64, 2048, 8),
                                                  (5, 5, 80, 32, 104, 16), (3, 1, 16, 16, 40, 1)])
@pytest.mark.parametrize("append,with_bias", [(True, True), (False, False)])
def test_projection_with_rotate_and_append_epilogue(K, Hq, Hkv, D, page, H, rows, append, with_bias):
    """Few bfloat16 rows: q/k/v projection, bias, rotation and the write into the cache in one
    kernel, against projection and rotate-and-append done apart by the plain twins (float32
    throughout, rounded once) and by the two separate kernels."""
    dtype = torch.bfloat16
    lens = [0, 63, 64, 129, 5, 700, 31, 1, 2, 300, 17, 64, 65, 127, 128, 9][:rows]
    pages, bt, ctx, _ = make_cache_case(dtype, Hq, Hkv, D, page, [1] * rows, lens, 256, 23)
    N = (Hq + 2 * Hkv) * D
    x, w = rnd((rows, H), dtype, 24), rnd((N, H), dtype, 25, 0.1)
    bias = 0.1 * rnd((N,), torch.float32, 26) if with_bias else None
    inv_freq = torch.tensor([10000.0 ** (-2.0 * i / D) for i in range(D // 2)], dtype=torch.float32).cuda()
    p1, p2, p3 = pages.clone(), pages.clone(), pages.clone()
    q1 = K.linear_rope_append(x, w, bias, ctx.positions, ctx.row_seg, inv_freq, D, Hq, Hkv, D, p1, bt, page, append)
    # plain: the projection kept in float32 until the one rounding at the end
    y = (x.float() @ w.float().T)
    q2 = y.clone()
    pf = p2.float()
    P.rope_append(q2, bias, ctx.positions, ctx.row_seg, inv_freq, D, Hq, Hkv, D, pf, bt, page, append)
    torch.testing.assert_close(q1[:, :Hq * D].float(), q2[:, :Hq * D].to(dtype).float(), **tol(dtype, 3))
    torch.testing.assert_close(p1.float(), pf.to(dtype).float(), **tol(dtype, 3))
    if not append:
        assert torch.equal(p1, pages)
    # the two-kernel path
    old = dict(K.TUNING)
    try:
        K.TUNING.update(qkv_rope_fused=False)
        q3 = K.linear_rope_append(x, w, bias, ctx.positions, ctx.row_seg, inv_freq, D, Hq, Hkv, D, p3, bt, page, append)
    finally:
        K.TUNING.update(old)
    torch.testing.assert_close(q1[:, :Hq * D].float(), q3[:, :Hq * D].float(), **tol(dtype, 4))
    torch.testing.assert_close(p1.float(), p3.float(), **tol(dtype, 4))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hq,Hkv,D,page,window", [(6, 2, 48, 16, 0), (4, 1, 128, 64, 0), (4, 4, 64, 16, 21),
                                                  (8, 2, 256, 32, 0), (3, 1, 16, 16, 40)])
def test_paged_attention(K, dtype, Hq, Hkv, D, page, window):
    pages, bt, ctx, qkv = make_cache_case(dtype, Hq, Hkv, D, page, [37, 1, 2, 1], [0, 130, 61, 0], 24, 13)
    scale = 1 / math.sqrt(D)
    out = K.paged_attention(qkv, Hq, Hkv, D, pages, bt, page, ctx, window, scale)
    ref = P.paged_attention(qkv, Hq, Hkv, D, pages, bt, page, ctx, window, scale)
    torch.testing.assert_close(out.float(), ref.float(), **tol(dtype))


@pytest.mark.parametrize("Hq,Hkv,D,page,window", [(4, 1, 128, 64, 0), (16, 16, 128, 64, 0), (6, 2, 64, 16, 0),
                                                  (6, 1, 32, 16, 150), (2, 2, 256, 32, 0), (10, 2, 16, 16, 0)])
def test_decode_attention_split_kernel(K, Hq, Hkv, D, page, window):
    """Steps of single rows in bfloat16 take the split-key kernel: contexts from 1 key to
    several blocks of 128, against the plain twin and against the any-rows kernel."""
    dtype = torch.bfloat16
    lens = [0, 127, 128, 129, 700, 383, 5]
    pages, bt, ctx, qkv = make_cache_case(dtype, Hq, Hkv, D, page, [1] * len(lens), lens, 128, 41)
    ctx.all_single, ctx.max_context = True, max(lens) + 1
    scale = 1 / math.sqrt(D)
    out = K.paged_attention(qkv, Hq, Hkv, D, pages, bt, page, ctx, window, scale)
    ref = P.paged_attention(qkv, Hq, Hkv, D, pages, bt, page, ctx, window, scale)
    torch.testing.assert_close(out.float(), ref.float(), **tol(dtype))
    ctx.all_single = False
    gen = K.paged_attention(qkv, Hq, Hkv, D, pages, bt, page, ctx, window, scale)
    torch.testing.assert_close(out.float(), gen.float(), **tol(dtype))
    # the one-launch form (one CTA per block of keys; the last CTA of a row merges), twice: its
    # counters must come back to zero.  It rounds differently from the streaming kernel.
    ctx.all_single = True
    old = K.TUNING["decode_merge_fused_max_rows"]
    K.TUNING["decode_merge_fused_max_rows"] = 64
    try:
        ones = [K.paged_attention(qkv, Hq, Hkv, D, pages, bt, page, ctx, window, scale) for _ in range(2)]
    finally:
        K.TUNING["decode_merge_fused_max_rows"] = old
    assert torch.equal(ones[0], ones[1])
    torch.testing.assert_close(ones[0].float(), ref.float(), **tol(dtype))


@pytest.mark.parametrize("Hq,Hkv,D,page,window", [(8, 4, 128, 64, 0), (32, 2, 64, 16, 300), (4, 4, 64, 32, 0),
                                                  (3, 3, 128, 16, 1000)])
def test_decode_attention_streaming_kernel(K, Hq, Hkv, D, page, window):
    """Steps with a thousand and more blocks of keys take the persistent streaming kernel:
    many rows with contexts from one key to seventeen blocks, with and without a window, up to
    16 query heads a group.  Against the any-rows kernel (itself checked against the plain
    twin), against the plain twin on the rows it can afford, and against the one-CTA-per-block
    kernel it replaces."""
    from ninfer_amd_mi50_b200.kernels import lib as klib
    dtype = torch.bfloat16
    lens = [0, 15, 16, 17, 127, 128, 129, 2100, 700, 383, 5, 1, 64, 1023, 1024, 1025, 2047, 2048, 33, 900,
            1500, 1777, 250, 255, 256, 257, 511, 512, 513, 1999, 47, 48, 49, 1200, 1300, 1400, 640, 641, 2, 3]
    n_pages = sum((n + 1 + page - 1) // page for n in lens) + 3
    pages, bt, ctx, qkv = make_cache_case(dtype, Hq, Hkv, D, page, [1] * len(lens), lens, n_pages, 43)
    ctx.all_single, ctx.max_context = True, max(lens) + 1
    assert len(lens) * Hkv * ((ctx.max_context + 127) // 128) >= 1024
    scale = 1 / math.sqrt(D)
    out = K.paged_attention(qkv, Hq, Hkv, D, pages, bt, page, ctx, window, scale)
    lib = klib.load()
    try:
        lib.nf_set_decode_stream(0)
        per_block = K.paged_attention(qkv, Hq, Hkv, D, pages, bt, page, ctx, window, scale)
    finally:
        lib.nf_set_decode_stream(1)
    assert not torch.equal(out, per_block)          # two kernels ran (they round differently)
    torch.testing.assert_close(out.float(), per_block.float(), **tol(dtype))
    ctx.all_single = False
    gen = K.paged_attention(qkv, Hq, Hkv, D, pages, bt, page, ctx, window, scale)
    torch.testing.assert_close(out.float(), gen.float(), **tol(dtype))
    few = [0, 1, 4, 5, 6, 10, 11, 32, 38, 39]       # short rows: the plain twin walks key by key
    sub = SimpleNamespace(positions=ctx.positions[few], row_seg=ctx.row_seg[few])
    ref = P.paged_attention(qkv[few], Hq, Hkv, D, pages, bt, page, sub, window, scale)
    torch.testing.assert_close(out[few].float(), ref.float(), **tol(dtype))
    # a far key that matters: make one early key of the longest row dominate one head's scores
    t_long = lens.index(2100)
    q = qkv.clone()
    seg = int(ctx.row_seg[t_long])
    j = 777 if window == 0 else 2100 - min(window, 2100) + 3
    kpage, slot = int(bt[seg, j // page]), j % page
    q[t_long, :D] = 0
    q[t_long, 0] = 30.0 / scale
    pages[kpage, 0, 0, slot, :] = 0
    pages[kpage, 0, 0, slot, 0] = 8.0                # score 240; the others are 30 * N(0, 1)
    ctx.all_single = True
    hot = K.paged_attention(q, Hq, Hkv, D, pages, bt, page, ctx, window, scale)
    torch.testing.assert_close(hot[t_long, :D].float(), pages[kpage, 1, 0, slot, :].float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("Hq,Hkv,D,page,window", [(4, 1, 128, 64, 0), (6, 2, 48, 16, 0), (4, 4, 64, 32, 37),
                                                  (2, 2, 16, 16, 0), (8, 2, 112, 64, 200)])
def test_prefill_attention_flash_kernel(K, Hq, Hkv, D, page, window):
    """Mixed segments in bfloat16 take the flash kernel: a long portion continuing an earlier
    one, a fresh prompt, single rows, a portion that ends exactly on a tile edge."""
    from ninfer_amd_mi50_b200.parts.base import StepContext
    dtype = torch.bfloat16
    seg_lens, pos0s = [150, 1, 64, 3, 1], [70, 333, 0, 127, 0]
    pages, bt, c, qkv = make_cache_case(dtype, Hq, Hkv, D, page, seg_lens, pos0s, 96, 43)
    row0 = [0]
    for n in seg_lens:
        row0.append(row0[-1] + n)
    mk = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    ctx = StepContext(dtype=dtype, device=torch.device("cuda"), T=row0[-1], S=len(seg_lens), token_ids=mk([0]),
                      positions=c.positions, row_seg=c.row_seg, seg_row0=mk(row0), seg_pos0=mk(pos0s),
                      seg_slot=mk([0] * 5), logit_rows=mk([]), seg_len_host=seg_lens, seg_pos0_host=pos0s,
                      max_rows_per_seg=150, max_context=334)
    scale = 1 / math.sqrt(D)
    out = K.paged_attention(qkv, Hq, Hkv, D, pages, bt, page, ctx, window, scale)
    ref = P.paged_attention(qkv, Hq, Hkv, D, pages, bt, page, ctx, window, scale)
    torch.testing.assert_close(out.float(), ref.float(), **tol(dtype))
    old = K.TUNING["bf16_attention"]
    K.TUNING["bf16_attention"] = "generic"
    gen = K.paged_attention(qkv, Hq, Hkv, D, pages, bt, page, ctx, window, scale)
    K.TUNING["bf16_attention"] = old
    torch.testing.assert_close(out.float(), gen.float(), **tol(dtype))


@pytest.mark.parametrize("Hq,Hkv,D,page,window", [(4, 2, 128, 64, 0), (3, 1, 64, 16, 0), (2, 2, 128, 128, 300),
                                                  (8, 2, 64, 32, 77), (2, 1, 128, 16, 0)])
def test_prefill_attention_on_tensor_cores(K, Hq, Hkv, D, page, window):
    """Steps with many rows take the tcgen05 attention kernel: a long portion that continues an
    earlier one across many blocks of 128 keys, a fresh prompt that ends inside a tile, single
    rows, a portion of exactly one tile.  Against the mma.sync kernel and the any-rows kernel
    (both checked against the plain twin elsewhere), against the plain twin on some rows, and
    with one far key made to dominate; and no bounded wait may have given up."""
    from ninfer_amd_mi50_b200.parts.base import StepContext
    dtype = torch.bfloat16
    seg_lens, pos0s = [700, 1, 300, 128, 1, 5], [450, 333, 0, 128, 0, 1019]
    n_pages = sum((p + n + page - 1) // page for p, n in zip(pos0s, seg_lens)) + 2
    pages, bt, c, qkv = make_cache_case(dtype, Hq, Hkv, D, page, seg_lens, pos0s, n_pages, 47)
    row0 = [0]
    for n in seg_lens:
        row0.append(row0[-1] + n)
    mk = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")

    def context():
        return StepContext(dtype=dtype, device=torch.device("cuda"), T=row0[-1], S=len(seg_lens), token_ids=mk([0]),
                           positions=c.positions, row_seg=c.row_seg, seg_row0=mk(row0), seg_pos0=mk(pos0s),
                           seg_slot=mk([0] * len(seg_lens)), logit_rows=mk([]), seg_len_host=seg_lens,
                           seg_pos0_host=pos0s, max_rows_per_seg=max(seg_lens), max_context=1200)
    scale = 1 / math.sqrt(D)
    # a far key that matters: row 650 of the long portion (position 1100) sees key 40 dominate head 0
    t_hot, j_hot = 650, 40 if window == 0 else 1100 - window + 2
    qkv[t_hot, :D] = 0
    qkv[t_hot, 0] = 30.0 / scale
    kpage, slot = int(bt[0, j_hot // page]), j_hot % page
    pages[kpage, 0, 0, slot, :] = 0
    pages[kpage, 0, 0, slot, 0] = 8.0                # score 240; the others are 30 * N(0, 1)
    out = K.paged_attention(qkv, Hq, Hkv, D, pages, bt, page, context(), window, scale)
    assert K.tensor_core_status() == 0
    old = dict(K.TUNING)
    try:
        K.TUNING.update(prefill_attention_tc_min_rows=10 ** 9)
        flash = K.paged_attention(qkv, Hq, Hkv, D, pages, bt, page, context(), window, scale)
        K.TUNING.update(bf16_attention="generic")
        gen = K.paged_attention(qkv, Hq, Hkv, D, pages, bt, page, context(), window, scale)
    finally:
        K.TUNING.update(old)
    assert not torch.equal(out, flash)               # two kernels ran (they round differently)
    torch.testing.assert_close(out.float(), flash.float(), **tol(dtype))
    torch.testing.assert_close(out.float(), gen.float(), **tol(dtype))
    torch.testing.assert_close(out[t_hot, :D].float(), pages[kpage, 1, 0, slot, :].float(), rtol=2e-2, atol=2e-2)
    few = [0, 1, 699, 700, 701, 702, 1000, 1001, 1128, 1129, 1130, 1134]
    sub = SimpleNamespace(positions=c.positions[few], row_seg=c.row_seg[few])
    ref = P.paged_attention(qkv[few], Hq, Hkv, D, pages, bt, page, sub, window, scale)
    torch.testing.assert_close(out[few].float(), ref.float(), **tol(dtype))


def _step_context(c, seg_lens, pos0s, dtype, max_context):
    from ninfer_amd_mi50_b200.parts.base import StepContext
    row0 = [0]
    for n in seg_lens:
        row0.append(row0[-1] + n)
    mk = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    return StepContext(dtype=dtype, device=torch.device("cuda"), T=row0[-1], S=len(seg_lens), token_ids=mk([0]),
                       positions=c.positions, row_seg=c.row_seg, seg_row0=mk(row0), seg_pos0=mk(pos0s),
                       seg_slot=mk([0] * len(seg_lens)), logit_rows=mk([]), seg_len_host=list(seg_lens),
                       seg_pos0_host=list(pos0s), max_rows_per_seg=max(seg_lens), max_context=max_context)


@pytest.mark.parametrize("keys", [4096, 8192])
@pytest.mark.parametrize("Hq,Hkv", [(16, 16), (28, 4)])
def test_attention_at_the_contexts_that_are_timed(K, Hq, Hkv, keys):
    """Head counts of the two large configurations (16 kv heads for 16 query heads; 4 for 28:
    seven heads a group), head size 128, pages of 64, contexts of 4,096 and 8,192 keys.
    Decode rows through both split-key kernels, a prompt portion through both flash kernels;
    all against the any-rows kernel, and against the plain twin on a few rows."""
    from ninfer_amd_mi50_b200.kernels import lib as klib
    dtype, D, page = torch.bfloat16, 128, 64
    scale = 1 / math.sqrt(D)
    # ---- decode: eight requests near the context length
    lens = [keys - 1, keys - 2, keys - 129, keys // 2, keys - 64, keys - 65, 100, keys - 1000]
    n_pages = sum((n + 1 + page - 1) // page for n in lens) + 1
    pages, bt, ctx, qkv = make_cache_case(dtype, Hq, Hkv, D, page, [1] * len(lens), lens, n_pages, 61)
    ctx.all_single, ctx.max_context = True, keys
    assert len(lens) * Hkv * (keys // 128) >= 1024           # enough blocks for the streaming kernel
    stream = K.paged_attention(qkv, Hq, Hkv, D, pages, bt, page, ctx, 0, scale)
    lib = klib.load()
    try:
        lib.nf_set_decode_stream(0)
        block = K.paged_attention(qkv, Hq, Hkv, D, pages, bt, page, ctx, 0, scale)
    finally:
        lib.nf_set_decode_stream(1)
    ctx.all_single = False
    gen = K.paged_attention(qkv, Hq, Hkv, D, pages, bt, page, ctx, 0, scale)
    assert not torch.equal(stream, block)
    torch.testing.assert_close(stream.float(), gen.float(), **tol(dtype))
    torch.testing.assert_close(block.float(), gen.float(), **tol(dtype))
    few = [0, 6]
    sub = SimpleNamespace(positions=ctx.positions[few], row_seg=ctx.row_seg[few])
    ref = P.paged_attention(qkv[few], Hq, Hkv, D, pages, bt, page, sub, 0, scale)
    torch.testing.assert_close(stream[few].float(), ref.float(), **tol(dtype))
    assert K.index_status() == 0
    del pages, qkv
    # ---- a prompt portion of 384 rows that ends at the context length, beside a short fresh prompt
    seg_lens, pos0s = [384, 130], [keys - 384, 0]
    n_pages = sum((p + n + page - 1) // page for p, n in zip(pos0s, seg_lens)) + 1
    pages, bt, c, qkv = make_cache_case(dtype, Hq, Hkv, D, page, seg_lens, pos0s, n_pages, 62)
    out = K.paged_attention(qkv, Hq, Hkv, D, pages, bt, page, _step_context(c, seg_lens, pos0s, dtype, keys), 0, scale)
    assert K.tensor_core_status() == 0
    old = dict(K.TUNING)
    try:
        K.TUNING.update(prefill_attention_tc_min_rows=10 ** 9)
        flash = K.paged_attention(qkv, Hq, Hkv, D, pages, bt, page, _step_context(c, seg_lens, pos0s, dtype, keys), 0, scale)
        K.TUNING.update(bf16_attention="generic")
        gen = K.paged_attention(qkv, Hq, Hkv, D, pages, bt, page, _step_context(c, seg_lens, pos0s, dtype, keys), 0, scale)
    finally:
        K.TUNING.update(old)
    assert not torch.equal(out, flash)
    torch.testing.assert_close(out.float(), gen.float(), **tol(dtype))
    torch.testing.assert_close(flash.float(), gen.float(), **tol(dtype))
    few = [383, 384 + 129]
    sub = SimpleNamespace(positions=c.positions[few], row_seg=c.row_seg[few])
    ref = P.paged_attention(qkv[few], Hq, Hkv, D, pages, bt, page, sub, 0, scale)
    torch.testing.assert_close(out[few].float(), ref.float(), **tol(dtype))


@pytest.mark.parametrize("Hq,Hkv,D,page,window", [(4, 2, 64, 16, 0), (16, 16, 128, 64, 0), (6, 1, 32, 16, 150)])
def test_single_rows_of_a_mixed_step_take_the_decode_kernel(K, Hq, Hkv, D, page, window):
    """A step that holds prompt portions and single decoded tokens: the single rows are served
    by the split-key kernel through a list of rows and get, bit for bit, what they get in a
    step that holds nothing else; the portions go to a flash kernel."""
    dtype = torch.bfloat16
    seg_lens = [1, 40, 1, 1, 150, 2, 1]
    pos0s = [700, 10, 0, 129, 300, 64, 383]
    n_pages = sum((p + n + page - 1) // page for p, n in zip(pos0s, seg_lens)) + 2
    pages, bt, c, qkv = make_cache_case(dtype, Hq, Hkv, D, page, seg_lens, pos0s, n_pages, 63)
    scale = 1 / math.sqrt(D)
    ctx = _step_context(c, seg_lens, pos0s, dtype, 701)
    rows, n = ctx.single_rows()
    assert n == 4 and rows.tolist() == [0, 41, 42, 195]
    mixed = K.paged_attention(qkv, Hq, Hkv, D, pages, bt, page, ctx, window, scale)
    K.TUNING["bf16_attention"] = "generic"
    try:
        gen = K.paged_attention(qkv, Hq, Hkv, D, pages, bt, page, ctx, window, scale)
    finally:
        K.TUNING["bf16_attention"] = "auto"
    torch.testing.assert_close(mixed.float(), gen.float(), **tol(dtype))
    # the same four rows alone, as a decode-only step over the same cache
    single = rows.tolist()
    alone = SimpleNamespace(positions=c.positions[single].contiguous(), row_seg=c.row_seg[single].contiguous(),
                            all_single=True, max_context=701)
    dec = K.paged_attention(qkv[single].contiguous(), Hq, Hkv, D, pages, bt, page, alone, window, scale)
    assert torch.equal(mixed[single], dec)
    assert K.index_status() == 0


def test_decode_attention_with_too_few_key_blocks_is_cut_and_reported(K):
    """The workspace of the split-key kernels has `nsplit` blocks of 128 keys per row; positions
    live on the device, so a call cannot be refused for a row that needs more.  Such a row is
    computed over the keys the workspace covers, nothing is written outside the workspace (the
    slabs behind it keep their fill), and the status names the row."""
    import ctypes
    dtype, Hq, Hkv, D, page = torch.bfloat16, 4, 2, 64, 16
    lens = [100, 700, 30, 5] * 44              # rows 1, 5, ... need 6 blocks
    pages, bt, ctx, qkv = make_cache_case(dtype, Hq, Hkv, D, page, [1] * len(lens), lens,
                                          sum((n + page) // page for n in lens) + 1, 64)
    T, nsplit = len(lens), 3
    lib = K.load()
    vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    for stream_kernel in (1, 0):
        lib.nf_set_decode_stream(stream_kernel)
        try:
            acc = torch.full((T * Hq * nsplit * D + 4096,), 7.0, dtype=torch.float32, device="cuda")
            ml = torch.full((T * Hq * nsplit * 2 + 4096,), 7.0, dtype=torch.float32, device="cuda")
            out = torch.zeros((T, Hq * D), dtype=dtype, device="cuda")
            assert stream_kernel == 0 or T * Hkv * nsplit >= 1024
            rc = lib.nf_decode_attention(vp(qkv.data_ptr()), ci(qkv.shape[1]), vp(pages.data_ptr()), vp(bt.data_ptr()),
                                         ci(bt.shape[1]), vp(ctx.positions.data_ptr()), vp(ctx.row_seg.data_ptr()),
                                         vp(out.data_ptr()), vp(acc.data_ptr()), vp(ml.data_ptr()), ci(T), ci(Hq),
                                         ci(Hkv), ci(D), ci(page), ci(pages.shape[0]), ci(0), cf(0.125), ci(nsplit),
                                         vp(torch.cuda.current_stream().cuda_stream))
            assert rc == 0
            torch.cuda.synchronize()
        finally:
            lib.nf_set_decode_stream(1)
        assert bool((acc[-4096:] == 7.0).all()) and bool((ml[-4096:] == 7.0).all())
        status = K.index_status()
        assert status > 100000 and (status - 100001) % 4 == 1       # one of the long rows
        assert K.index_status() == 0                                 # reading clears it
        # the rows that fit are right
        ok = [t for t, n in enumerate(lens) if n < nsplit * 128][:12]
        sub = SimpleNamespace(positions=ctx.positions[ok], row_seg=ctx.row_seg[ok])
        ref = P.paged_attention(qkv[ok], Hq, Hkv, D, pages, bt, page, sub, 0, 0.125)
        torch.testing.assert_close(out[ok].float(), ref.float(), **tol(dtype))


def test_a_wait_that_runs_out_reaches_the_host_as_an_error(K):
    """The tensor-core kernels bound every wait on a barrier and record a code when one gives
    up.  A kernel whose only barrier nobody ever arrives at shows the path end to end: it
    returns (the context stays usable), the status carries its code, `check_status` raises,
    and the next check is clean."""
    import ctypes
    from ninfer_amd_mi50_b200.kernels import lib as klib
    assert K.tensor_core_status() == 0
    klib.call("nf_bounded_wait_selftest", ctypes.c_int(2000),
              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    with pytest.raises(klib.KernelError, match="gave up on a wait .code 9."):
        K.check_status("test")
    K.check_status("test")
    x = torch.ones(8, device="cuda")
    assert float(x.sum()) == 8.0


def test_attention_finds_one_far_key(K):
    """One key among hundreds is made to dominate; the output must be its value row."""
    Hq, Hkv, D, page = 2, 1, 64, 16
    for dtype in DTYPES:
        pages, bt, ctx, qkv = make_cache_case(dtype, Hq, Hkv, D, page, [1], [700], 48, 17)
        far = 3          # a key in the very first page, 697 positions back
        qkv[0, :Hq * D] = 0
        qkv[0, 5] = 8.0
        qkv[0, D + 5] = 8.0
        pg = int(bt[0, far // page])
        pages[:, 0, :, :, 5] = 0
        pages[pg, 0, 0, far % page, 5] = 40.0
        want = pages[pg, 1, 0, far % page].float()
        for single in (False, True):
            ctx.all_single, ctx.max_context = single, 701
            out = K.paged_attention(qkv, Hq, Hkv, D, pages, bt, page, ctx, 0, 1 / math.sqrt(D))
            for h in range(Hq):
                torch.testing.assert_close(out[0, h * D:(h + 1) * D].float(), want, rtol=1e-2, atol=1e-2)


def test_attention_window_edge(K):
    """The key just outside the window is made huge: it must not be seen; the one just
    inside must."""
    Hq, Hkv, D, page, window = 1, 1, 32, 16, 24
    pages, bt, ctx, qkv = make_cache_case(torch.float32, Hq, Hkv, D, page, [1], [100], 16, 19)
    qkv[0, :D] = 0
    qkv[0, 0] = 10.0
    pages[:, 0, :, :, 0] = 0
    outside, inside = 100 - window, 100 - window + 1
    pages[int(bt[0, outside // page]), 0, 0, outside % page, 0] = 50.0
    out = K.paged_attention(qkv, Hq, Hkv, D, pages, bt, page, ctx, window, 1.0)
    ref = P.paged_attention(qkv, Hq, Hkv, D, pages, bt, page, ctx, window, 1.0)
    torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-5)
    pages[int(bt[0, inside // page]), 0, 0, inside % page, 0] = 50.0
    out = K.paged_attention(qkv, Hq, Hkv, D, pages, bt, page, ctx, window, 1.0)
    torch.testing.assert_close(out[0], pages[int(bt[0, inside // page]), 1, 0, inside % page], rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H,E,k,norm,extra", [(9, 200, 6, 3, True, 1), (64, 96, 60, 4, False, 1),
                                                (1, 512, 16, 4, True, 0), (5, 1000, 130, 8, False, 1)])
def test_router_topk(K, dtype, T, H, E, k, norm, extra):
    x = rnd((T, H), dtype, 21)
    w = rnd((E + extra, H), torch.float32, 22, 0.1)
    idx, wts, ext = K.router_topk(x, w, E, k, norm)
    ridx, rwts, rext = P.router_topk(x, w, E, k, norm)
    assert torch.equal(idx, ridx)
    torch.testing.assert_close(wts, rwts, rtol=1e-4, atol=1e-6)
    if extra:
        torch.testing.assert_close(ext, rext, rtol=1e-4, atol=1e-5)
    else:
        assert ext is None


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H,E,k,norm,extra", [(1, 200, 6, 3, True, 1), (8, 2048, 60, 4, False, 1),
                                                (16, 96, 16, 4, True, 0), (13, 1000, 130, 8, False, 1),
                                                (64, 96, 16, 4, True, 0), (5, 3000, 70, 2, True, 2)])
def test_route_in_one_launch(K, dtype, T, H, E, k, norm, extra):
    """Few rows: logits, selection and plan come from one launch - by one thread-block cluster,
    or by a grid whose last block finishes the work; each twice in a row, since the second
    form must leave its ticket counter as it found it.  Both give the same bits."""
    x = rnd((T, H), dtype, 71)
    w = rnd((E + extra, H), torch.float32, 72, 0.1)
    ridx, rwts, rext = P.router_topk(x, w, E, k, norm)
    rplan = P.moe_plan(ridx, E)
    old = dict(K.TUNING)
    seen = []
    try:
        for cluster in (True, False):
            K.TUNING.update(router_cluster_max_rows=32 if cluster else 0)
            for _ in range(2):
                idx, wts, ext, plan = K.route(x, w, E, k, norm)
                assert torch.equal(idx, ridx)
                torch.testing.assert_close(wts, rwts, rtol=1e-4, atol=1e-6)
                if extra:
                    torch.testing.assert_close(ext, rext, rtol=1e-4, atol=1e-5)
                assert torch.equal(plan.offsets, rplan.offsets) and torch.equal(plan.order, rplan.order)
                assert torch.equal(plan.inv, rplan.inv) and torch.equal(plan.active, rplan.active)
            seen.append((wts, ext))
    finally:
        K.TUNING.update(old)
    assert torch.equal(seen[0][0], seen[1][0])
    if extra:
        assert torch.equal(seen[0][1], seen[1][1])


def test_router_ties_go_to_lower_index(K):
    x = torch.ones((2, 64), dtype=torch.float32, device="cuda")
    w = torch.zeros((8, 64), dtype=torch.float32, device="cuda")
    w[5] = 0.01
    idx, wts, _ = K.router_topk(x, w, 8, 3, False)
    assert idx.tolist() == [[5, 0, 1], [5, 0, 1]]


@pytest.mark.parametrize("T,k,E", [(1, 2, 8), (37, 4, 60), (700, 3, 6), (2048, 4, 60)])
def test_moe_plan(K, T, k, E):
    g = torch.Generator().manual_seed(23)
    idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32).cuda()
    plan = K.moe_plan(idx, E)
    ref = P.moe_plan(idx, E)
    assert torch.equal(plan.offsets, ref.offsets)
    assert torch.equal(plan.order, ref.order)
    assert torch.equal(plan.inv, ref.inv)
    assert torch.equal(plan.active, ref.active)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H,I,E,k", [(1, 200, 72, 6, 3), (50, 96, 100, 16, 4), (130, 256, 33, 8, 2),
                                       (64, 512, 136, 60, 4), (8, 2048, 1408, 60, 4)])
def test_moe_gemms_and_combine(K, dtype, T, H, I, E, k, bf16_path):
    g = torch.Generator().manual_seed(29)
    x = rnd((T, H), dtype, 31)
    w13, w2 = rnd((E, 2 * I, H), dtype, 32, 0.1), rnd((E, H, I), dtype, 33, 0.1)
    idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32).cuda()
    wts = torch.rand((T, k), generator=g).cuda()
    plan = K.moe_plan(idx, E)
    act = K.moe_gemm1(x, w13, plan, k)
    ract = P.moe_gemm1(x, w13, plan, k)
    close(act, ract, dtype)
    y = K.moe_gemm2(ract, w2, plan)
    ry = P.moe_gemm2(ract, w2, plan)
    close(y, ry, dtype)
    shared, gate = rnd((T, H), dtype, 34), rnd((T, 1), torch.float32, 35)
    out = K.moe_combine(ry, plan, wts, shared, gate, dtype)
    rout = P.moe_combine(ry, plan, wts, shared, gate, dtype)
    torch.testing.assert_close(out.float(), rout.float(), **tol(dtype, 2))
    out = K.moe_combine(ry, plan, wts, None, None, dtype)
    rout = P.moe_combine(ry, plan, wts, None, None, dtype)
    torch.testing.assert_close(out.float(), rout.float(), **tol(dtype, 2))


def test_refusals_are_clear(K):
    with pytest.raises(ValueError, match="head_dim"):
        K.check_head_dim(40)
    with pytest.raises(Exception, match="CUDA tensor"):
        K.linear(torch.zeros(2, 4), torch.zeros(3, 4))


@pytest.mark.parametrize("T,H,I,E,k", [(64, 256, 128, 4, 2), (300, 200, 136, 6, 3), (700, 512, 264, 3, 2),
                                       (2048, 2048, 1408, 60, 4), (400, 328, 72, 5, 2), (1024, 3584, 2560, 64, 8)])
def test_grouped_gemm_on_tensor_cores(K, T, H, I, E, k):
    """The tcgen05 / TMEM / TMA grouped product that serves routed experts at prefill: ragged
    groups (empty, one row, more than one pass of 256 rows), feature counts and k that are not
    multiples of the tile, against the plain twin; and no bounded wait may have given up."""
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(T + I)
    x = rnd((T, H), dtype, 51)
    w13, w2 = rnd((E, 2 * I, H), dtype, 52, 0.1), rnd((E, H, I), dtype, 53, 0.1)
    # skewed routing: expert 0 gets nearly every token, the last expert none
    idx = torch.stack([torch.cat([torch.zeros(1, dtype=torch.long),
                                  1 + torch.randperm(max(E - 2, 1), generator=g)[:k - 1]]) if t % 7 else
                       torch.randperm(E - 1, generator=g)[:k] for t in range(T)]).to(torch.int32).cuda()
    plan = K.moe_plan(idx, E)
    pw13, pw2 = K.pack_weights(w13, swiglu=True), K.pack_weights(w2, swiglu=False)
    big = T > 700
    if big:        # the plain twin loops in Python: use the CUDA-core kernel as the yardstick
        old = dict(K.TUNING)
        K.TUNING.update(bf16_moe="simt")
        ract = K.moe_gemm1(x, w13, plan, k)
        ry = K.moe_gemm2(ract, w2, plan)
        K.TUNING.update(old)
    else:
        ract = P.moe_gemm1(x, w13, plan, k)
        ry = P.moe_gemm2(ract, w2, plan)
    old = dict(K.TUNING)
    try:
        for limit in (0, 10 ** 9):       # tensor-core kernel, then the streaming kernel, on packed weights
            if limit and big:
                continue
            K.TUNING.update(skinny_moe_max_tokens=limit)
            close(K.moe_gemm1(x, pw13, plan, k), ract, dtype)
            close(K.moe_gemm2(ract, pw2, plan), ry, dtype)
        # the second product with two feature tiles an item (many rows an expert; an odd number
        # of tiles leaves the last one alone) and with one: the same products in the same order
        K.TUNING.update(skinny_moe_max_tokens=0)
        lib = K.load()
        try:
            lib.nf_set_grouped_gemm_pair(1, 1)
            paired = K.moe_gemm2(ract, pw2, plan)
            lib.nf_set_grouped_gemm_pair(0, 0)
            single = K.moe_gemm2(ract, pw2, plan)
        finally:
            lib.nf_set_grouped_gemm_pair(1, 64)
        assert torch.equal(paired, single)
        close(paired, ry, dtype)
    finally:
        K.TUNING.update(old)
    assert K.tensor_core_status() == 0


@pytest.mark.parametrize("T,H,I,E,k", [(1, 256, 128, 4, 2), (5, 200, 136, 6, 3), (8, 2048, 1408, 60, 4),
                                       (13, 512, 264, 7, 2), (3, 40, 24, 3, 1)])
def test_streaming_experts_with_an_early_start(K, T, H, I, E, k):
    """The experts' second product may start fetching weights before the first has finished,
    when the caller vouches that the plan is older than that kernel: same bits either way, on
    packed and on plain weights, and close to the plain twin."""
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(T * 31 + H)
    x = rnd((T, H), dtype, 71)
    w13, w2 = rnd((E, 2 * I, H), dtype, 72, 0.1), rnd((E, H, I), dtype, 73, 0.1)
    idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32).cuda()
    plan = K.moe_plan(idx, E)
    pw13, pw2 = K.pack_weights(w13, swiglu=True), K.pack_weights(w2, swiglu=False)
    old = dict(K.TUNING)
    try:
        K.TUNING.update(skinny_moe_max_tokens=10 ** 9)
        act = K.moe_gemm1(x, pw13, plan, k)
        y0 = K.moe_gemm2(act, pw2, plan)
        act_b = K.moe_gemm1(x, pw13, plan, k)
        y1 = K.moe_gemm2(act_b, pw2, plan, plan_is_older=True)
        act_c = K.moe_gemm1(x, w13, plan, k)
        y2 = K.moe_gemm2(act_c, w2, plan, plan_is_older=True)
    finally:
        K.TUNING.update(old)
    assert torch.equal(act, act_b) and torch.equal(act, act_c)
    assert torch.equal(y0, y1) and torch.equal(y0, y2)
    ract = P.moe_gemm1(x, w13, plan, k)
    close(act, ract, dtype)
    close(y0, P.moe_gemm2(ract, w2, plan), dtype)


@pytest.mark.parametrize("T,H,I,E,k", [(1, 256, 128, 4, 2), (2, 2048, 1408, 60, 4), (5, 200, 136, 6, 3),
                                       (8, 2048, 1408, 60, 4), (13, 512, 264, 7, 2), (3, 40, 24, 3, 1),
                                       (16, 2048, 1408, 60, 4), (8, 3584, 2560, 64, 8), (4, 2048, 1408, 60, 4),
                                       (1, 2048, 1408, 60, 4), (24, 512, 264, 3, 2), (64, 2048, 1408, 60, 4),
                                       (33, 200, 136, 6, 3)])
def test_experts_in_one_persistent_launch(K, T, H, I, E, k):
    """Decode steps run both products of the routed experts in one persistent launch that streams
    the packed weights through a ring of shared memory: close to the plain twin, the same bits
    when run again, a token's rows the same bits whatever else is in the batch (as long as the
    item size is the same), its counters back at zero, and no wait given up.  Experts with more
    than eight rows are served eight rows at a time."""
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(T * 17 + I)
    x = rnd((T, H), dtype, 81)
    w13, w2 = rnd((E, 2 * I, H), dtype, 82, 0.1), rnd((E, H, I), dtype, 83, 0.1)
    idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32).cuda()
    plan = K.moe_plan(idx, E)
    pw13, pw2 = K.pack_weights(w13, swiglu=True), K.pack_weights(w2, swiglu=False)
    old = dict(K.TUNING)
    K.TUNING.update(moe_stream_min_tokens=1, moe_stream_max_tokens=64)
    try:
        _persistent_experts_case(K, x, w13, w2, pw13, pw2, idx, plan, T, E, k, dtype)
    finally:
        K.TUNING.update(old)


def _persistent_experts_case(K, x, w13, w2, pw13, pw2, idx, plan, T, E, k, dtype):
    assert K.moe_experts_fit_stream(x, pw13, pw2, plan, k)
    y = K.moe_experts(x, pw13, pw2, plan, k)
    again = K.moe_experts(x, pw13, pw2, plan, k)
    assert torch.equal(y, again)
    ry = P.moe_gemm2(P.moe_gemm1(x, w13, plan, k), w2, plan)
    close(y, ry, dtype)
    K.TUNING.update(moe_stream_max_tokens=0)
    assert not K.moe_experts_fit_stream(x, pw13, pw2, plan, k)
    close(K.moe_experts(x, pw13, pw2, plan, k), ry, dtype)      # the two-launch path, same answer
    K.TUNING.update(moe_stream_max_tokens=64)
    from ninfer_amd_mi50_b200.kernels import ops
    half = T // 2
    if half:
        # the first half of the batch alone: where the item size is the same, every row must come out the same
        xh, plan_h = x[:half].contiguous(), K.moe_plan(idx[:half].contiguous(), E)
        yh = K.moe_experts(xh, pw13, pw2, plan_h, k)
        pairs = torch.arange(half * k, device="cuda")
        if ops._stream_items(xh, pw13, pw2, E, k) == ops._stream_items(x, pw13, pw2, E, k):
            assert torch.equal(yh[plan_h.inv.long()[pairs]], y[plan.inv.long()[pairs]])
        else:
            close(yh[plan_h.inv.long()[pairs]], y[plan.inv.long()[pairs]], dtype)
    assert K.tensor_core_status() == 0 and K.index_status() == 0
    assert int(ops._STREAM_WORK[str(x.device)][:K.load().nf_moe_stream_counter_ints()].abs().sum()) == 0


@pytest.mark.parametrize("T,H,I,E,k,extra", [(8, 2048, 1408, 60, 4, 1), (1, 256, 128, 4, 2, 0), (5, 200, 136, 6, 3, 1),
                                             (16, 512, 264, 7, 2, 1), (64, 2048, 1408, 60, 4, 1), (33, 328, 72, 70, 8, 2)])
def test_persistent_launch_that_routes_as_well(K, T, H, I, E, k, extra):
    """The same launch with the routing inside: its CTAs compute the logits, the last one to
    finish selects and writes the plan, all go on to the products.  Selection, weights, raw
    logits of the further rows, plan and outputs have the bits of `route` followed by
    `moe_experts`; run twice, the same again; counters back at zero."""
    dtype = torch.bfloat16
    x = rnd((T, H), dtype, 87)
    wr = rnd((E + extra, H), torch.float32, 88, 0.05)
    w13, w2 = rnd((E, 2 * I, H), dtype, 82, 0.1), rnd((E, H, I), dtype, 83, 0.1)
    pw13, pw2 = K.pack_weights(w13, swiglu=True), K.pack_weights(w2, swiglu=False)
    old = dict(K.TUNING)
    K.TUNING.update(moe_stream_min_tokens=1, moe_stream_max_tokens=64, moe_stream_route_max_tokens=64)
    try:
        assert K.can_route_and_run_experts(x, wr, pw13, pw2, E, k)
        idx, wts, ext, plan, y = K.route_and_run_experts(x, wr, E, k, True, pw13, pw2)
        idx2, wts2, ext2, plan2, y2 = K.route_and_run_experts(x, wr, E, k, True, pw13, pw2)
        ridx, rwts, rext, rplan = K.route(x, wr, E, k, True)
        ry = K.moe_experts(x, pw13, pw2, rplan, k)
    finally:
        K.TUNING.update(old)
    for a, b, c in ((idx, idx2, ridx), (wts, wts2, rwts), (plan.offsets, plan2.offsets, rplan.offsets),
                    (plan.order, plan2.order, rplan.order), (plan.inv, plan2.inv, rplan.inv),
                    (plan.active, plan2.active, rplan.active), (y, y2, ry)):
        assert torch.equal(a, b) and torch.equal(a, c)
    if extra:
        assert torch.equal(ext, ext2) and torch.equal(ext, rext)
    pidx, pwts, pext = P.router_topk(x, wr, E, k, True)
    same = (idx == pidx).all(dim=1)
    assert same.float().mean() > 0.97
    torch.testing.assert_close(wts[same], pwts[same], rtol=2e-4, atol=1e-6)
    assert K.tensor_core_status() == 0 and K.index_status() == 0
    from ninfer_amd_mi50_b200.kernels import ops
    assert int(ops._STREAM_WORK[str(x.device)][:K.load().nf_moe_stream_counter_ints()].abs().sum()) == 0


@pytest.mark.parametrize("T,H,I,E,k,Is", [(8, 2048, 1408, 60, 4, 5632), (1, 256, 128, 4, 2, 256), (5, 200, 136, 6, 3, 104),
                                          (16, 512, 264, 7, 2, 600), (64, 2048, 1408, 60, 4, 5632), (2, 2048, 1408, 60, 4, 5632)])
def test_persistent_launch_with_the_shared_expert_inside(K, T, H, I, E, k, Is):
    """Routing, the experts' products and the shared expert's (cut into chunks of the experts'
    width, also where that does not divide it) in the one launch: the sum over the rows and
    weights it names is the plain feed-forward, the routed part has the bits of the launch
    without the shared expert, and a second run gives the same bits."""
    dtype = torch.bfloat16
    x = rnd((T, H), dtype, 87)
    wr = rnd((E + 1, H), torch.float32, 88, 0.05)
    w13, w2 = rnd((E, 2 * I, H), dtype, 82, 0.1), rnd((E, H, I), dtype, 83, 0.1)
    ws13, ws2 = rnd((2 * Is, H), dtype, 84, 0.1), rnd((H, Is), dtype, 85, 0.1)
    pw13, pw2 = K.pack_weights(w13, swiglu=True), K.pack_weights(w2, swiglu=False)
    shared = K.pack_shared_expert(ws13, ws2, I)
    chunks = shared[0].groups
    assert chunks == (Is + I - 1) // I
    old = dict(K.TUNING)
    K.TUNING.update(moe_stream_min_tokens=1, moe_stream_max_tokens=64, moe_stream_route_max_tokens=64,
                    moe_stream_shared_max_tokens=64)
    try:
        assert K.can_route_and_run_experts(x, wr, pw13, pw2, E, k, shared=shared)
        idx, wts, ext, plan, y, cw, cplan = K.route_and_run_experts(x, wr, E, k, True, pw13, pw2, shared=shared)
        again = K.route_and_run_experts(x, wr, E, k, True, pw13, pw2, shared=shared)
        ridx, rwts, rext, rplan, ry = K.route_and_run_experts(x, wr, E, k, True, pw13, pw2)
    finally:
        K.TUNING.update(old)
    assert torch.equal(y, again[4]) and torch.equal(cw, again[5]) and torch.equal(cplan.inv, again[6].inv)
    assert torch.equal(idx, ridx) and torch.equal(wts, rwts) and torch.equal(plan.inv, rplan.inv)
    assert torch.equal(y[:T * k], ry)
    assert torch.equal(cw[:, :k], wts) and torch.equal(cplan.inv.view(T, k + chunks)[:, :k], plan.inv.view(T, k))
    torch.testing.assert_close(cw[:, k:], torch.sigmoid(ext[:, :1]).expand(T, chunks), rtol=1e-6, atol=1e-7)
    got = K.moe_combine(y, cplan, cw, None, None, dtype)
    # the plain twin, chunk by chunk as the launch does it (every chunk's output is rounded to bfloat16) ...
    parts = [P.moe_gemm2(P.moe_gemm1(x, w13, plan, k), w2, plan)]
    for c in range(chunks):
        lo, hi = c * I, min(Is, (c + 1) * I)
        gu = torch.cat([ws13[lo:hi], ws13[Is + lo:Is + hi]])
        parts.append(P.linear(P.linear_swiglu(x, gu), ws2[:, lo:hi].contiguous()))
    close(y, torch.cat(parts), dtype)
    # ... and in one piece: the chunks' roundings add up to a few bfloat16 steps of the largest value
    pshared = P.linear(P.linear_swiglu(x, ws13), ws2)
    want = P.moe_combine(parts[0], plan, wts, pshared, ext, dtype).float()
    assert (got.float() - want).abs().max().item() <= 2 ** -7 * want.abs().max().item()
    assert K.tensor_core_status() == 0 and K.index_status() == 0
    from ninfer_amd_mi50_b200.kernels import ops
    assert int(ops._STREAM_WORK[str(x.device)][:K.load().nf_moe_stream_counter_ints()].abs().sum()) == 0


def test_persistent_launch_gives_up_cleanly_when_activations_never_complete(K):
    """The second product waits for a count that the first product raises.  With the counters
    set so that the count can never be reached, every wait of the launch runs out (within about
    a second), its three kinds of warps leave, the copies in flight land, the launch returns, the
    status names the wait, the counters are back at zero, and the next launch is right."""
    from ninfer_amd_mi50_b200.kernels import lib as klib, ops
    T, H, I, E, k = 8, 512, 264, 7, 2
    dtype = torch.bfloat16
    x = rnd((T, H), dtype, 87)
    w13, w2 = rnd((E, 2 * I, H), dtype, 82, 0.1), rnd((E, H, I), dtype, 83, 0.1)
    pw13, pw2 = K.pack_weights(w13, swiglu=True), K.pack_weights(w2, swiglu=False)
    g = torch.Generator().manual_seed(5)
    idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32).cuda()
    plan = K.moe_plan(idx, E)
    good = K.moe_experts(x, pw13, pw2, plan, k)
    assert K.moe_experts_fit_stream(x, pw13, pw2, plan, k) and K.tensor_core_status() == 0
    work = ops._STREAM_WORK[str(x.device)]
    counters = K.load().nf_moe_stream_counter_ints()
    work[8:counters] = -(1 << 20)                      # the row groups' counters: no count will reach its mark
    K.moe_experts(x, pw13, pw2, plan, k)
    torch.cuda.synchronize()
    with pytest.raises(klib.KernelError, match="gave up on a wait .code 4(04|12)."):
        K.check_status("test")
    K.check_status("test")
    assert int(work[:counters].abs().sum()) == 0
    assert torch.equal(K.moe_experts(x, pw13, pw2, plan, k), good)
    assert K.tensor_core_status() == 0


def test_persistent_experts_launch_is_refused_where_it_does_not_fit(K):
    """Eight rows of a very wide model leave too little shared memory for the ring: the
    two-launch path serves the step, with the same answer."""
    T, H, I, E, k = 8, 8192, 512, 8, 2
    x = rnd((T, H), torch.bfloat16, 84)
    w13, w2 = rnd((E, 2 * I, H), torch.bfloat16, 85, 0.1), rnd((E, H, I), torch.bfloat16, 86, 0.1)
    g = torch.Generator().manual_seed(3)
    idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32).cuda()
    plan = K.moe_plan(idx, E)
    pw13, pw2 = K.pack_weights(w13, swiglu=True), K.pack_weights(w2, swiglu=False)
    old = dict(K.TUNING)
    K.TUNING.update(moe_stream_min_tokens=1)
    try:
        assert not K.moe_experts_fit_stream(x, pw13, pw2, plan, k)
        assert K.moe_experts_fit_stream(x[:, :4096].contiguous(), K.pack_weights(w13[:, :, :4096].contiguous(), swiglu=True),
                                        K.pack_weights(w2[:, :4096].contiguous(), swiglu=False), plan, k)
    finally:
        K.TUNING.update(old)
    close(K.moe_experts(x, pw13, pw2, plan, k), P.moe_gemm2(P.moe_gemm1(x, w13, plan, k), w2, plan), torch.bfloat16)


@pytest.mark.parametrize("exact_bf16", [True, False])
def test_router_many_rows_through_split_matrix(K, exact_bf16):
    """More than 128 bfloat16 rows: the logits come from library products over the routing
    matrix split into two bfloat16 halves (one half when the matrix is bfloat16 already)."""
    T, H, E, k = 700, 512, 60, 4
    x = rnd((T, H), torch.bfloat16, 61)
    w = rnd((E + 1, H), torch.float32, 62, 0.1)
    if exact_bf16:
        w = w.to(torch.bfloat16).float()
    split = K.split_router(w)
    assert (split[1] is None) == exact_bf16
    idx, wts, ext = K.router_topk(x, w, E, k, True, split=split)
    ridx, rwts, rext = P.router_topk(x, w, E, k, True)
    same = (idx == ridx).all(dim=1)
    assert same.float().mean() > 0.995          # a tie within 2^-17 may fall the other way
    torch.testing.assert_close(wts[same], rwts[same], rtol=2e-4, atol=1e-6)
    torch.testing.assert_close(ext, rext, rtol=2e-4, atol=2e-5)


@pytest.mark.parametrize("dtype", DTYPES)
def test_router_with_logits_that_are_not_numbers_still_names_valid_experts(K, dtype):
    """A row of NaN (a broken checkpoint, an overflow upstream) must not become an expert index:
    the selection still names k distinct valid experts, the plan stays inside its arrays, and the
    row's weights are NaN so that its output shows the fault.  Other rows are untouched."""
    T, H, E, k = 6, 256, 8, 2
    x = rnd((T, H), dtype, 91)
    x[2] = float("nan")
    x[4, 7] = float("inf")
    wr = rnd((E + 1, H), torch.float32, 92, 0.05)
    clean = x.clone()
    clean[2] = 0
    clean[4] = 0
    for fn in (K.route, lambda *a: K.router_topk(*a) + (None,)):
        idx, wts, ext, plan = fn(x, wr, E, k, False)
        ref_idx, ref_wts, _, _ = fn(clean, wr, E, k, False)
        assert int(idx.min()) >= 0 and int(idx.max()) < E
        assert all(len(set(row)) == k for row in idx.tolist())
        assert bool(torch.isnan(wts[2]).all()) and bool(torch.isnan(wts[4]).all())
        ok = [0, 1, 3, 5]
        assert torch.equal(idx[ok], ref_idx[ok]) and torch.equal(wts[ok], ref_wts[ok])
        if plan is not None:
            assert int(plan.offsets[-1]) == T * k and sorted(plan.order.tolist()) == list(range(T * k))
    assert K.index_status() == 0
