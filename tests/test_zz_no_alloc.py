"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory themselves: a plug-in inside
an application that owns the whole device budget, a loop that cannot afford the
synchronisation an allocation may cause, a sandbox that forbids allocations after start-up.
`nf_decode_attention_static` serves them from a fixed scratch array inside the library.
This test calls it twice in a row (the scratch keeps the first call's contents when the
second runs) and lays each result beside the ordinary entry point's, and checks that a call
too large for the fixed array is refused rather than run.

The file's name makes pytest collect it last, so that a run which stops at the first failure
has already run everything else.
"""

import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(T, Hq, Hkv, D, page, lens, seed):
    g = torch.Generator().manual_seed(seed)
    n_pages = sum((n + 1 + page - 1) // page for n in lens)
    width = max((n + 1 + page - 1) // page for n in lens)
    perm = torch.randperm(n_pages, generator=g).tolist()
    bt = torch.full((T, width), -1, dtype=torch.int32)
    for s, n in enumerate(lens):
        for lp in range((n + 1 + page - 1) // page):
            bt[s, lp] = perm.pop()
    pages = torch.randn((n_pages, 2, Hkv, page, D), generator=g).to(torch.bfloat16).cuda()
    qkv = torch.randn((T, (Hq + 2 * Hkv) * D), generator=g).to(torch.bfloat16).cuda()
    positions = torch.tensor(lens, dtype=torch.int32).cuda()
    row_seg = torch.arange(T, dtype=torch.int32).cuda()
    return pages, bt.cuda(), positions, row_seg, qkv


def test_static_scratch_entry_point_matches_the_ordinary_one():
    from ninfer_amd_mi50_b200 import kernels
    lib = kernels.load()
    lib.nf_decode_attention_static_scratch_bytes.restype = ctypes.c_longlong
    lib.nf_last_error.restype = ctypes.c_char_p
    assert lib.nf_decode_attention_static_scratch_bytes() == 8 << 20
    vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    stream = vp(torch.cuda.current_stream().cuda_stream)
    for seed, (Hq, Hkv, D, page, lens) in enumerate([(4, 2, 64, 16, [0, 130, 517, 255]),
                                                     (16, 16, 128, 64, [2047, 900, 64])]):
        T = len(lens)
        pages, bt, positions, row_seg, qkv = _case(T, Hq, Hkv, D, page, lens, 70 + seed)
        nsplit = (max(lens) + 1 + 127) // 128
        scale = 1 / math.sqrt(D)
        ws_acc = torch.empty((T, Hq, nsplit, D), dtype=torch.float32, device="cuda")
        ws_ml = torch.empty((T, Hq, nsplit, 2), dtype=torch.float32, device="cuda")
        want = torch.empty((T, Hq * D), dtype=torch.bfloat16, device="cuda")
        rc = lib.nf_decode_attention(vp(qkv.data_ptr()), ci(qkv.shape[1]), vp(pages.data_ptr()), vp(bt.data_ptr()),
                                     ci(bt.shape[1]), vp(positions.data_ptr()), vp(row_seg.data_ptr()),
                                     vp(want.data_ptr()), vp(ws_acc.data_ptr()), vp(ws_ml.data_ptr()), ci(T), ci(Hq),
                                     ci(Hkv), ci(D), ci(page), ci(pages.shape[0]), ci(0), cf(scale), ci(nsplit), stream)
        assert rc == 0, lib.nf_last_error()
        for call in range(2):                     # two calls in a row share the fixed scratch
            got = torch.full((T, Hq * D), float("nan"), dtype=torch.bfloat16, device="cuda")
            rc = lib.nf_decode_attention_static(vp(qkv.data_ptr()), ci(qkv.shape[1]), vp(pages.data_ptr()),
                                                vp(bt.data_ptr()), ci(bt.shape[1]), vp(positions.data_ptr()),
                                                vp(row_seg.data_ptr()), vp(got.data_ptr()), ci(T), ci(Hq), ci(Hkv),
                                                ci(D), ci(page), ci(pages.shape[0]), ci(0), cf(scale), ci(nsplit), stream)
            assert rc == 0, lib.nf_last_error()
            torch.cuda.synchronize()
            torch.testing.assert_close(got.float(), want.float(), rtol=1.6e-2, atol=1.6e-2)
            # same kernels, same order of sums, other scratch: the bits are the same too
            assert torch.equal(got, want)
    # beyond the fixed array: refused with a message, nothing launched
    rc = lib.nf_decode_attention_static(vp(qkv.data_ptr()), ci(qkv.shape[1]), vp(pages.data_ptr()), vp(bt.data_ptr()),
                                        ci(bt.shape[1]), vp(positions.data_ptr()), vp(row_seg.data_ptr()),
                                        vp(got.data_ptr()), ci(4096), ci(64), ci(8), ci(128), ci(64),
                                        ci(pages.shape[0]), ci(0), cf(0.1), ci(64), stream)
    assert rc != 0 and b"fixed array" in lib.nf_last_error()
    torch.cuda.synchronize()
