"""Python faces of the CUDA kernels.  Every function launches on torch's current stream.

One function per operation of the step (reference: the free functions of
src/ops/ops.h:19-234).  Which kernel serves a call is decided by the dtype and by the
number of rows only, never by what the rows are (prompt or decode), so that a row's
result does not depend on its neighbours.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import lib as _lib

c_int, c_float, c_void_p, c_longlong = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong

_DT = {torch.float32: 0, torch.bfloat16: 1}

# Library products of the bfloat16 path must add up in float32: no split-k partial sums
# rounded to bfloat16, and never TF32 for float32 operands.
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
torch.backends.cuda.matmul.allow_tf32 = False

# Tunables that tests may override to force a particular kernel.
TUNING = {
    "bf16_linear": "auto",        # "simt" | "auto"
    "bf16_attention": "auto",     # "generic" | "auto"
    "bf16_moe": "auto",           # "simt" | "auto"
    "skinny_max_rows": 16,        # dense products with more rows go to the library
    # routed experts: up to this many tokens the streaming kernel serves, beyond it the
    # tensor-core kernel (measured decode steps: 4 % slower at 16 tokens, 7 % faster at 32,
    # 10 % faster at 64)
    "skinny_moe_max_tokens": 16,
    # prompt portions: steps with at least this many rows use the tcgen05 attention kernel (head
    # size 64 or 128), fewer the mma.sync one; a huge number turns the tensor-core kernel off
    "prefill_attention_tc_min_rows": 128,
    "qkv_rope_fused": True,       # few bfloat16 rows: rotation and cache append in the projection's epilogue
    "router_tensor_min_rows": 128,   # router logits of more rows than this use tensor cores
    # up to this many rows, routing is a single launch (whole decode steps at 24 and 32 tokens:
    # 0.5 % faster than logits, selection and plan apart; at 64 tokens 1 % slower)
    "router_fused_max_rows": 32,
    # ... by one cluster of 8 CTAs up to this many rows (measured: 6.6 against 10.5 us at 1 row,
    # 10.1 against 11.5 at 8, 17.2 against 15.5 at 16); 0 turns the cluster kernel off
    "router_cluster_max_rows": 8,
    # decode attention can merge its key blocks in the same launch (the last CTA of a row does
    # it); measured slower than the separate merge kernel at every batch size, so it is off
    "decode_merge_fused_max_rows": 0,
    # the routed experts' weighted sum joins the residual add and the next norm in one kernel, up
    # to this many rows (same bits either way; measured on B200: no difference to a decode step,
    # which only loses a launch, and a prompt of 2,048 tokens 2 % slower fused, because the
    # separate combine reads 16 bytes a lane and spreads a row over more CTAs); 0 turns it off
    "fuse_combine_norm_max_rows": 64,
    # a shared expert runs beside the routed path, on a second stream, in steps of up to
    # `shared_fork_max_rows` rows (larger steps fill the device with either alone); it is started
    # beside the router up to `shared_fork_late_rows` rows and after it beyond.  (With the
    # experts as two launches, starting after the router was 3 % faster at 48 and 64 rows; with
    # their persistent launch, starting beside the router is 2 % faster at 40 to 64 rows too, so
    # the second threshold now equals the first.)
    "shared_fork_max_rows": 64,
    "shared_fork_late_rows": 64,
    # in steps of at least this many rows (and more than `shared_fork_max_rows`) the routing
    # (logits, selection, plan, gather: short kernels of a few CTAs, one waiting for the other)
    # runs on a second stream of higher priority while the shared expert's products fill the
    # device; 0 turns it off.  (A prompt of 2,048 tokens: 3 % faster; decode steps of 72 to 128
    # tokens: 1.3 %.)
    "route_beside_shared_min_rows": 65,
    # steps of `moe_stream_min_tokens` to `moe_stream_max_tokens` tokens run both products of the
    # routed experts in one persistent launch (packed bfloat16 weights); a max of 0: always two
    # launches.  Measured at A2.7B sizes, whole decode steps against the two launches (the
    # streaming product up to 16 tokens, the tensor-core grouped product beyond): the same at 4
    # tokens, 3 % faster at 6, 6 % at 8, 16 % at 16, 10 % at 32, 3.5 % at 64, 2 % slower at 96 and
    # 128 (experts with more than eight rows are served eight at a time and stream their weights
    # again).  `moe_stream_smem_kb`: shared memory that launch takes on every SM - what is left
    # stays free for the shared expert's kernels, which run beside it on a second stream (160
    # instead of 192: the same up to 16 tokens, 2 % slower at 32 and 64)
    "moe_stream_min_tokens": 6,
    "moe_stream_max_tokens": 64,
    # ... and up to this many tokens that launch routes as well (logits, selection and plan by
    # its own CTAs before the products); 0: the router's kernels run before it
    "moe_stream_route_max_tokens": 64,
    # ... and up to `moe_stream_shared_max_tokens` tokens it serves a shared expert as well (a
    # second, packed copy of its matrices is then kept: `pack_shared_expert`; 0: no such copy, the
    # shared expert always runs beside the launch on a second stream).  Measured at A2.7B sizes,
    # whole decode steps against the router's kernels + the launch + the second stream: 3 % faster
    # at 6 tokens, 2 % at 8, the same at 16, 3 % slower at 32, 6 % at 64 (the routing inside the
    # launch takes 15 us, and only the CTAs that hold an item of the shared expert have work
    # until it is done); with fewer than 6 tokens the separate kernels win as well
    "moe_stream_shared": 1,
    "moe_stream_shared_max_tokens": 16,
    "moe_stream_smem_kb": 192,
}

SUPPORTED_HEAD_DIMS = tuple(range(16, 257, 16))
DECODE_HEAD_DIMS = (16, 32, 64, 128, 256)   # head sizes of the split-key decode kernel
DECODE_SPLIT = 128                          # keys per block of that kernel
PREFILL_HEAD_DIMS = tuple(range(16, 129, 16))   # head sizes of the flash prefill kernel
PREFILL_TILE_ROWS = 64                      # query rows per tile of that kernel
PREFILL_KEY_BLOCK = 64                      # keys per block of that kernel
MAX_EXPERTS = 3072


def check_head_dim(head_dim: int) -> None:
    if head_dim not in SUPPORTED_HEAD_DIMS:
        raise ValueError(f"head_dim={head_dim} is not supported by the attention kernels "
                         f"(multiples of 16 from 16 to 256)")


DECODE_MAX_SPLITS = 1024                    # key blocks one row's merge takes


def check_attention_limits(dtype: torch.dtype, head_dim: int, max_context: int, page_size: int) -> None:
    """What the attention kernels cannot serve, said at start-up: the bfloat16 decode kernels
    merge at most `DECODE_MAX_SPLITS` blocks of `DECODE_SPLIT` keys per row."""
    check_head_dim(head_dim)
    if dtype == torch.bfloat16 and head_dim in DECODE_HEAD_DIMS:
        most = DECODE_MAX_SPLITS * DECODE_SPLIT
        if max_context > most:
            raise ValueError(f"max_context={max_context} is beyond the {most} keys a request may hold "
                             f"in bfloat16 mode (decode attention merges at most {DECODE_MAX_SPLITS} "
                             f"blocks of {DECODE_SPLIT} keys)")


def check_router_sizes(num_experts: int, top_k: int) -> None:
    if not 1 <= num_experts <= MAX_EXPERTS:
        raise ValueError(f"num_experts={num_experts} is not supported (1..{MAX_EXPERTS})")
    if not 1 <= top_k <= num_experts:
        raise ValueError(f"top_k={top_k} must lie in [1, {num_experts}]")


def _p(t: Optional[torch.Tensor]):
    return None if t is None else c_void_p(t.data_ptr())


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}") from None


def _chk(t: torch.Tensor, name: str, dtype=None, contiguous=True) -> None:
    if not t.is_cuda:
        raise _lib.KernelError(f"{name} must be a CUDA tensor; there is no CPU implementation")
    if contiguous and not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")


# ---------------------------------------------------------------------------------------
# rows
# ---------------------------------------------------------------------------------------

def embed_rows(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = float32(table[ids[t]])."""
    _chk(table, "table"); _chk(ids, "ids", torch.int32); _chk(out, "out", torch.float32)
    _lib.call("nf_embed_rows", _p(table), _p(ids), _p(out), c_int(ids.numel()),
              c_int(table.shape[1]), c_int(table.shape[0]), c_int(_dt(table)), _stream())


def add_rmsnorm(h: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor) -> None:
    """h += delta (float32, in place); out = h * rsqrt(mean(h^2) + eps) * weight."""
    _chk(h, "h", torch.float32); _chk(weight, "weight", torch.float32); _chk(out, "out")
    if delta is not None:
        _chk(delta, "delta", out.dtype)
    _lib.call("nf_add_rmsnorm", _p(h), _p(delta), None, _p(weight), c_float(eps), _p(out),
              c_int(h.shape[0]), c_int(h.shape[1]), c_int(_dt(out)), _stream())


def add_rmsnorm_rows(h: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor,
                     weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """out[r] = norm(h[rows[r]] + delta[rows[r]]); h is left as it is."""
    _chk(h, "h", torch.float32); _chk(rows, "rows", torch.int32); _chk(out, "out")
    _chk(weight, "weight", torch.float32)
    if delta is not None:
        _chk(delta, "delta", out.dtype)
    _lib.call("nf_add_rmsnorm", _p(h), _p(delta), _p(rows), _p(weight), c_float(eps), _p(out),
              c_int(rows.numel()), c_int(h.shape[1]), c_int(_dt(out)), _stream())


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """[M, 2I] -> [M, I]: silu(first half) * second half."""
    _chk(gate_up, "gate_up")
    M, two_i = gate_up.shape
    out = torch.empty((M, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    _lib.call("nf_silu_mul", _p(gate_up), _p(out), c_int(M), c_int(two_i // 2), c_int(_dt(gate_up)),
              _stream())
    return out


# ---------------------------------------------------------------------------------------
# matrix products
# ---------------------------------------------------------------------------------------

def _gemm_simt(a, lda, b, b_group_stride, c, M, N, K, groups, max_rows, offsets, a_rows, a_div,
               swiglu) -> None:
    _lib.call("nf_gemm_simt", _p(a), c_int(lda), _p(b), c_longlong(b_group_stride), _p(c),
              c_int(c.shape[1]), c_int(M), c_int(N), c_int(K), c_int(groups), c_int(max_rows),
              _p(offsets), _p(a_rows), c_int(a_div), c_int(1 if swiglu else 0), c_int(_dt(a)),
              c_int(_dt(c)), _stream())


def _skinny(x, ldx, w, w_group_stride, out, M, N, K, groups, max_rows, offsets, x_rows, x_div, swiglu,
            packed=False, group_map=None, early_index=False) -> None:
    _lib.call("nf_skinny_gemm", _p(x), c_int(ldx), _p(w), c_longlong(w_group_stride), _p(out),
              c_int(out.shape[1]), c_int(M), c_int(N), c_int(K), c_int(groups), c_int(max_rows),
              _p(offsets), _p(x_rows), c_int(x_div), c_int(1 if swiglu else 0), c_int(_dt(out)),
              c_int(1 if packed else 0), _p(group_map),
              c_int(group_map.numel() if group_map is not None else 0), c_int(1 if early_index else 0),
              _stream())


class PackedWeights:
    """Grouped bfloat16 weights [G, rows, K] in the tile layout the streaming kernels read.

    Tiles of 128 rows x 64 k (SwiGLU: 128 gate rows followed by the 128 matching up rows),
    stored contiguously as [group][feature tile][k tile][tile rows][64], each tile in the
    128-byte-swizzled image (the 16-byte piece j of tile row r is stored at piece j ^ (r & 7)),
    zero-padded to whole tiles.  A CTA that owns 128 features reads one contiguous slab."""

    def __init__(self, data: torch.Tensor, groups: int, n_features: int, K: int, swiglu: bool):
        self.data, self.groups, self.n_features, self.K, self.swiglu = data, groups, n_features, K, swiglu
        self.dtype, self.device = data.dtype, data.device

    @property
    def group_stride(self) -> int:
        return self.data[0].numel()

    def nbytes(self) -> int:
        return self.data.numel() * self.data.element_size()

    def group_nbytes(self) -> int:
        return self.group_stride * self.data.element_size()


def can_pack(n_features: int, K: int) -> bool:
    return K % 8 == 0


def pack_weights(w: torch.Tensor, swiglu: bool, chunk: int = 4) -> PackedWeights:
    """[G, rows, K] bfloat16 (rows = 2 * features with gate rows first when `swiglu`) -> packed."""
    _chk(w, "w", torch.bfloat16)
    G, R, K = w.shape
    N = R // 2 if swiglu else R
    NT, KT = (N + 127) // 128, (K + 63) // 64
    rows = 256 if swiglu else 128
    out = torch.empty((G, NT, KT, rows, 64), dtype=w.dtype, device=w.device)
    r = torch.arange(rows, device=w.device)
    src_piece = (torch.arange(8, device=w.device)[None, :] ^ (r[:, None] & 7))       # [rows, 8]
    for g0 in range(0, G, chunk):
        blk = w[g0:g0 + chunk]
        n = blk.shape[0]
        halves = [blk[:, :N], blk[:, N:]] if swiglu else [blk]
        tiles = []
        for h in halves:
            p = torch.zeros((n, NT * 128, KT * 64), dtype=w.dtype, device=w.device)
            p[:, :N, :K] = h
            tiles.append(p.view(n, NT, 128, KT, 64).permute(0, 1, 3, 2, 4))             # [n, NT, KT, 128, 64]
        t = torch.cat(tiles, dim=3) if swiglu else tiles[0]                            # [n, NT, KT, rows, 64]
        t = t.reshape(n, NT, KT, rows, 8, 8)
        idx = src_piece.view(1, 1, 1, rows, 8, 1).expand(n, NT, KT, rows, 8, 8)
        out[g0:g0 + n] = torch.gather(t, 4, idx).reshape(n, NT, KT, rows, 64)
    return PackedWeights(out, G, N, K, swiglu)


def _bf16_path(rows: int, K: int, key: str) -> str:
    """Which bfloat16 product serves `rows` rows: decided by the row count and K only."""
    if TUNING[key] == "simt":
        return "simt"
    limit = TUNING["skinny_max_rows"] if key == "bf16_linear" else TUNING["skinny_moe_max_tokens"]
    if rows <= limit and K % 8 == 0:
        return "skinny"
    if key == "bf16_moe":
        return "simt"          # unpacked expert weights and many tokens: the CUDA-core product
    return "large"


def chain_break() -> None:
    """The next kernel launched (by this thread) waits for everything before it in its stream
    in the ordinary way.  To be called after making a stream wait for another stream's event:
    the kernel that follows must not be chained to the kernel before it in its own stream."""
    _lib.load().nf_chain_break()


def tensor_core_status() -> int:
    """0, or the code of the first bounded wait that a kernel with a shared-memory ring gave up on
    since the last call (synchronises the device): 1-4 from the grouped GEMM, 101-110 from
    attention, 401-413 from the persistent experts' kernel (405-407: a plan that does not fit it)."""
    lib = _lib.load()
    gemm, attn = int(lib.nf_grouped_gemm_tc_status()), int(lib.nf_prefill_attention_tc_status())
    ms = int(lib.nf_moe_stream_status())
    return gemm if gemm else (100 + attn if attn else (400 + ms if ms else 0))


def index_status() -> int:
    """0, or what a kernel that follows device-side indices found outside its operands since the
    last call (it skips such an access): 201-203 the streaming product (group, row range, row
    index), 300 + token + 1 the combine, 100000 + row + 1 a decode-attention row whose position
    lay beyond the key blocks its call allowed for.  Synchronises the device."""
    lib = _lib.load()
    sk, cb = int(lib.nf_skinny_index_status()), int(lib.nf_combine_index_status())
    da = int(lib.nf_decode_attention_status())
    return 200 + sk if sk else (300 + cb if cb else (100000 + da if da else 0))


def check_status(where: str = "") -> None:
    """Raise `KernelError` if a kernel gave up on a bounded wait or skipped an access outside
    its operands since the last check: its output is then not to be used.  Synchronises the
    device, so it is called where the host waits anyway (after a step's logits or tokens have
    been read) and every so many decode steps."""
    tc = tensor_core_status()
    ix = index_status()
    if tc or ix:
        what = []
        if tc:
            what.append(f"a tensor-core kernel gave up on a wait (code {tc})")
        if ix:
            what.append(f"a kernel met an index outside its operands (code {ix})")
        raise _lib.KernelError((where + ": " if where else "") + "; ".join(what)
                               + "; the results of the steps since the last check are invalid")


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """x [M, K] times w [N, K] transposed -> [M, N]; float32 accumulation."""
    _chk(x, "x"); _chk(w, "w", x.dtype)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise ValueError(f"linear: x has {K} columns, w has {w.shape[1]}")
    out_dtype = out_dtype or x.dtype
    if M == 0:
        return torch.empty((M, N), dtype=out_dtype, device=x.device)
    path = "simt" if x.dtype == torch.float32 else _bf16_path(M, K, "bf16_linear")
    if path == "large":
        # a plain library product, as the reference uses rocBLAS for M > 1 (src/ops/linear.hip)
        if out_dtype == torch.bfloat16:
            return torch.mm(x, w.t())
        try:
            return torch.mm(x, w.t(), out_dtype=torch.float32)
        except (TypeError, RuntimeError):
            path = "simt"
    out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    if path == "skinny":
        _skinny(x, K, w, 0, out, M, N, K, 1, M, None, None, 1, False)
    else:
        _gemm_simt(x, K, w, 0, out, M, N, K, 1, M, None, None, 1, False)
    return out


def linear_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    """x [M, K], w [2I, K] (gate rows first) -> silu(x gate^T) * (x up^T)  [M, I]."""
    _chk(x, "x"); _chk(w_gate_up, "w_gate_up", x.dtype)
    M, K = x.shape
    inner = w_gate_up.shape[0] // 2
    if M == 0:
        return torch.empty((M, inner), dtype=x.dtype, device=x.device)
    path = "simt" if x.dtype == torch.float32 else _bf16_path(M, K, "bf16_linear")
    if path == "large":
        return silu_mul(torch.mm(x, w_gate_up.t()))
    out = torch.empty((M, inner), dtype=x.dtype, device=x.device)
    if path == "skinny":
        _skinny(x, K, w_gate_up, 0, out, M, inner, K, 1, M, None, None, 1, True)
    else:
        _gemm_simt(x, K, w_gate_up, 0, out, M, inner, K, 1, M, None, None, 1, True)
    return out


# ---------------------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------------------

def rope_append(qkv: torch.Tensor, bias: Optional[torch.Tensor], positions: torch.Tensor,
                row_seg: torch.Tensor, inv_freq: Optional[torch.Tensor], rotary_dim: int,
                Hq: int, Hkv: int, D: int, pages: torch.Tensor, block_table: torch.Tensor,
                page_size: int, append: bool) -> None:
    """In place: qkv += bias; rotate q and k heads; write k, v to the cache pages."""
    _chk(qkv, "qkv"); _chk(pages, "pages", qkv.dtype); _chk(block_table, "block_table", torch.int32)
    _chk(positions, "positions", torch.int32); _chk(row_seg, "row_seg", torch.int32)
    if bias is not None:
        _chk(bias, "bias", torch.float32)
    if inv_freq is not None:
        _chk(inv_freq, "inv_freq", torch.float32)
    if qkv.shape[1] != (Hq + 2 * Hkv) * D:
        raise ValueError("rope_append: qkv width does not match the head counts")
    _lib.call("nf_rope_append", _p(qkv), _p(bias), _p(positions), _p(row_seg), _p(inv_freq),
              c_int(rotary_dim if inv_freq is not None else 0), c_int(qkv.shape[0]), c_int(Hq),
              c_int(Hkv), c_int(D), _p(pages), _p(block_table), c_int(block_table.shape[1]),
              c_int(page_size), c_int(pages.shape[0]), c_int(1 if append else 0), c_int(_dt(qkv)),
              _stream())


def linear_rope_append(x: torch.Tensor, w_qkv: torch.Tensor, bias: Optional[torch.Tensor],
                       positions: torch.Tensor, row_seg: torch.Tensor, inv_freq: torch.Tensor,
                       rotary_dim: int, Hq: int, Hkv: int, D: int, pages: torch.Tensor,
                       block_table: torch.Tensor, page_size: int, append: bool) -> torch.Tensor:
    """qkv = x w_qkv^T, then `rope_append` on it -> [T, (Hq + 2 Hkv) D] whose query columns hold
    the rotated queries (the key and value columns are not meant to be read: they went to the
    cache).  A bfloat16 step of few rows does both in one kernel: the streaming product's
    epilogue adds the bias, rotates and writes keys and values into their cache page."""
    T, K = x.shape
    if (TUNING["qkv_rope_fused"] and x.is_cuda and x.dtype == torch.bfloat16 and 0 < T <= min(16, TUNING["skinny_max_rows"])
            and TUNING["bf16_linear"] == "auto" and K % 8 == 0 and D % 16 == 0 and rotary_dim == D
            and inv_freq is not None):
        _chk(x, "x"); _chk(w_qkv, "w_qkv", x.dtype); _chk(pages, "pages", x.dtype)
        _chk(block_table, "block_table", torch.int32); _chk(positions, "positions", torch.int32)
        _chk(row_seg, "row_seg", torch.int32); _chk(inv_freq, "inv_freq", torch.float32)
        if bias is not None:
            _chk(bias, "bias", torch.float32)
        N = (Hq + 2 * Hkv) * D
        if w_qkv.shape != (N, K):
            raise ValueError("linear_rope_append: the projection does not match the head counts")
        qkv = torch.empty((T, N), dtype=x.dtype, device=x.device)
        _lib.call("nf_skinny_qkv_rope", _p(x), c_int(K), _p(w_qkv), _p(qkv), c_int(N), c_int(T), c_int(K),
                  _p(bias), _p(positions), _p(row_seg), _p(inv_freq), c_int(Hq), c_int(Hkv), c_int(D),
                  _p(pages), _p(block_table), c_int(block_table.shape[1]), c_int(page_size),
                  c_int(pages.shape[0]), c_int(1 if append else 0), _stream())
        return qkv
    qkv = linear(x, w_qkv)
    rope_append(qkv, bias, positions, row_seg, inv_freq, rotary_dim, Hq, Hkv, D, pages, block_table,
                page_size, append)
    return qkv


_COUNTERS = {}


def _zeroed_counters(device, n: int) -> torch.Tensor:
    """Ints that kernels find zero and leave zero (completion counters of one-launch
    reductions).  Kept for the life of the process, so that captured graphs may refer to them."""
    key = str(device)
    bufs = _COUNTERS.setdefault(key, [])
    if not bufs or bufs[-1].numel() < n:
        # earlier, smaller buffers stay alive: a captured graph may still point at them
        bufs.append(torch.zeros((max(n, 4096),), dtype=torch.int32, device=device))
    return bufs[-1]


def _tiles(ctx, rows_per_tile, window, keys_per_block, pair, min_rows):
    if min_rows > 1:
        return ctx.paired_query_tiles(rows_per_tile, window, keys_per_block, pair=pair, min_rows=min_rows)
    return ctx.paired_query_tiles(rows_per_tile, window, keys_per_block, pair=pair)


def _decode_attention(qkv, Hq, Hkv, D, pages, block_table, page_size, ctx, window, scale, out,
                      rows: Optional[torch.Tensor], n: int) -> None:
    """The split-key decode kernels on all rows of the step (`rows` None) or on the `n` rows
    listed in `rows` (int32 on the device); writes those rows of `out`."""
    nsplit = max(1, (int(ctx.max_context) + DECODE_SPLIT - 1) // DECODE_SPLIT)
    ws_acc = torch.empty((n, Hq, nsplit, D), dtype=torch.float32, device=qkv.device)
    ws_ml = torch.empty((n, Hq, nsplit, 2), dtype=torch.float32, device=qkv.device)
    if rows is not None:
        _lib.call("nf_decode_attention_rows", _p(qkv), c_int(qkv.shape[1]), _p(pages), _p(block_table),
                  c_int(block_table.shape[1]), _p(ctx.positions), _p(ctx.row_seg), _p(out),
                  _p(ws_acc), _p(ws_ml), _p(rows), c_int(n), c_int(Hq), c_int(Hkv), c_int(D), c_int(page_size),
                  c_int(pages.shape[0]), c_int(window), c_float(scale), c_int(nsplit), _stream())
    elif n > TUNING["decode_merge_fused_max_rows"]:
        _lib.call("nf_decode_attention", _p(qkv), c_int(qkv.shape[1]), _p(pages), _p(block_table),
                  c_int(block_table.shape[1]), _p(ctx.positions), _p(ctx.row_seg), _p(out),
                  _p(ws_acc), _p(ws_ml), c_int(n), c_int(Hq), c_int(Hkv), c_int(D), c_int(page_size),
                  c_int(pages.shape[0]), c_int(window), c_float(scale), c_int(nsplit), _stream())
    else:
        counters = _zeroed_counters(qkv.device, n * Hkv)
        _lib.call("nf_decode_attention_fused", _p(qkv), c_int(qkv.shape[1]), _p(pages), _p(block_table),
                  c_int(block_table.shape[1]), _p(ctx.positions), _p(ctx.row_seg), _p(out),
                  _p(ws_acc), _p(ws_ml), _p(counters), c_int(n), c_int(Hq), c_int(Hkv), c_int(D),
                  c_int(page_size), c_int(pages.shape[0]), c_int(window), c_float(scale), c_int(nsplit),
                  _stream())


def paged_attention(qkv: torch.Tensor, Hq: int, Hkv: int, D: int, pages: torch.Tensor,
                    block_table: torch.Tensor, page_size: int, ctx, window: int, scale: float
                    ) -> torch.Tensor:
    """Causal attention of the rows' (rotated) queries in `qkv` over the cache -> [T, Hq*D].

    In bfloat16 a row is served according to its own segment: a segment of one row (a decoded
    token) by the split-key decode kernel, a segment of several rows (a prompt portion) by a
    flash kernel - whatever else the step holds.  A mixed step is therefore two launches."""
    _chk(qkv, "qkv"); _chk(pages, "pages", qkv.dtype)
    T = qkv.shape[0]
    out = torch.empty((T, Hq * D), dtype=qkv.dtype, device=qkv.device)
    if T == 0:
        return out
    fast = qkv.dtype == torch.bfloat16 and TUNING["bf16_attention"] != "generic"
    if fast and getattr(ctx, "all_single", False) and D in DECODE_HEAD_DIMS:
        _decode_attention(qkv, Hq, Hkv, D, pages, block_table, page_size, ctx, window, scale, out, None, T)
        return out
    if (fast and D in PREFILL_HEAD_DIMS and getattr(ctx, "seg_len_host", None) is not None
            and getattr(ctx, "seg_pos0_host", None) is not None and qkv.shape[1] % 8 == 0):
        min_rows = 1
        if D in DECODE_HEAD_DIMS and hasattr(ctx, "single_rows"):
            rows, n_single = ctx.single_rows()
            if n_single:
                _decode_attention(qkv, Hq, Hkv, D, pages, block_table, page_size, ctx, window, scale, out,
                                  rows, n_single)
                min_rows = 2
        if (T >= TUNING["prefill_attention_tc_min_rows"] and qkv.is_contiguous() and pages.is_contiguous()
                and _lib.load().nf_prefill_attention_tc_fits(c_int(Hq), c_int(Hkv), c_int(D), c_int(page_size),
                                                            c_longlong(pages.shape[0]))):
            # tcgen05 / TMEM / TMA: tiles of 128 rows, blocks of 128 keys
            tiles, n_tiles = _tiles(ctx, 128, window, 128, False, min_rows)
            _lib.call("nf_prefill_attention_tc", _p(qkv), c_longlong(T), c_int(qkv.shape[1]), _p(pages),
                      _p(block_table), c_int(block_table.shape[1]), _p(ctx.positions), _p(ctx.seg_row0),
                      _p(tiles), c_int(n_tiles), _p(out), c_int(Hq), c_int(Hkv), c_int(D), c_int(page_size),
                      c_int(pages.shape[0]), c_int(window), c_float(scale), _stream())
            return out
        tiles, n_tiles = _tiles(ctx, PREFILL_TILE_ROWS, window, PREFILL_KEY_BLOCK, True, min_rows)
        _lib.call("nf_prefill_attention", _p(qkv), c_int(qkv.shape[1]), _p(pages), _p(block_table),
                  c_int(block_table.shape[1]), _p(ctx.positions), _p(ctx.seg_row0), _p(tiles),
                  c_int(n_tiles), _p(out), c_int(Hq), c_int(Hkv), c_int(D), c_int(page_size),
                  c_int(pages.shape[0]), c_int(window), c_float(scale), _stream())
        return out
    _lib.call("nf_paged_attention_generic", _p(qkv), c_int(qkv.shape[1]), _p(pages),
              _p(block_table), c_int(block_table.shape[1]), _p(ctx.positions), _p(ctx.row_seg),
              _p(out), c_int(T), c_int(Hq), c_int(Hkv), c_int(D), c_int(page_size),
              c_int(pages.shape[0]), c_int(window), c_float(scale), c_int(_dt(qkv)), _stream())
    return out


# ---------------------------------------------------------------------------------------
# routed experts
# ---------------------------------------------------------------------------------------

@dataclass
class MoePlan:
    offsets: torch.Tensor   # int32 [E + 1] rows of each expert in sorted order
    order: torch.Tensor     # int32 [T * k] pair (t * k + j) at each sorted position
    inv: torch.Tensor       # int32 [T * k] sorted position of each pair
    num_experts: int
    num_tokens: int
    top_k: int
    active: Optional[torch.Tensor] = None   # int32 [min(E, T * k)] experts that have pairs, -1 padded


def split_router(w_router: torch.Tensor) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """A float32 routing matrix as bfloat16 `hi` plus bfloat16 `lo` with hi + lo = w to 16 bits
    of mantissa; `lo` is None when the matrix is exactly bfloat16 (the usual checkpoint).
    With them, router logits of many rows are tensor-core products whose every partial
    product is exact and whose sums are float32."""
    hi = w_router.to(torch.bfloat16)
    rest = w_router - hi.to(torch.float32)
    lo = rest.to(torch.bfloat16) if bool((rest != 0).any()) else None
    return hi, lo


def router_topk(x: torch.Tensor, w_router: torch.Tensor, E: int, k: int, norm_topk: bool,
                split: Optional[Tuple[torch.Tensor, Optional[torch.Tensor]]] = None
                ) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """Router logits (float32), softmax, top-k.  Rows of `w_router` beyond E give raw
    logits back (`extra`, [T, rows - E]).  Returns (idx int32 [T, k], weights float32 [T, k], extra).

    With many bfloat16 rows and a `split` of the matrix (see `split_router`) the logits come
    from tensor-core products with float32 sums; otherwise from the float32 CUDA-core kernel."""
    _chk(x, "x"); _chk(w_router, "w_router", torch.float32)
    T, H = x.shape
    extra = w_router.shape[0] - E
    idx = torch.empty((T, k), dtype=torch.int32, device=x.device)
    wts = torch.empty((T, k), dtype=torch.float32, device=x.device)
    ext = torch.empty((T, extra), dtype=torch.float32, device=x.device) if extra > 0 else None
    if (split is not None and x.dtype == torch.bfloat16 and T > TUNING["router_tensor_min_rows"]
            and TUNING["bf16_linear"] != "simt" and H % 8 == 0):
        # logits^T [E + extra, T] = W_r x^T with the streaming tensor-core kernel: the routing
        # matrix (at most a few dozen rows) plays the part of the batch, the tokens that of the
        # weights.  Products of bfloat16 values are exact, sums are float32.
        rows = E + extra
        logits_t = torch.empty((rows, T), dtype=torch.float32, device=x.device)
        _skinny(split[0], H, x, 0, logits_t, rows, T, H, 1, rows, None, None, 1, False)
        if split[1] is not None:
            low = torch.empty_like(logits_t)
            _skinny(split[1], H, x, 0, low, rows, T, H, 1, rows, None, None, 1, False)
            logits_t += low
        _lib.call("nf_router_select", _p(logits_t), c_longlong(1), c_longlong(T), c_int(T), c_int(E),
                  c_int(extra), c_int(k), c_int(1 if norm_topk else 0), _p(idx), _p(wts), _p(ext), _stream())
        return idx, wts, ext
    logits = torch.empty((T, E + extra), dtype=torch.float32, device=x.device)
    _lib.call("nf_router_topk", _p(x), _p(w_router), c_int(T), c_int(H), c_int(E), c_int(extra),
              c_int(k), c_int(1 if norm_topk else 0), _p(logits), _p(idx), _p(wts), _p(ext),
              c_int(_dt(x)), _stream())
    return idx, wts, ext


def moe_plan(topk_idx: torch.Tensor, E: int) -> MoePlan:
    _chk(topk_idx, "topk_idx", torch.int32)
    T, k = topk_idx.shape
    dev = topk_idx.device
    offsets = torch.empty((E + 1,), dtype=torch.int32, device=dev)
    order = torch.empty((T * k,), dtype=torch.int32, device=dev)
    inv = torch.empty((T * k,), dtype=torch.int32, device=dev)
    counts = torch.empty((E,), dtype=torch.int32, device=dev)
    active = torch.empty((min(E, max(T * k, 1)),), dtype=torch.int32, device=dev)
    _lib.call("nf_moe_plan", _p(topk_idx), c_int(T * k), c_int(E), _p(offsets), _p(order), _p(inv),
              _p(counts), _p(active), c_int(active.numel()), _stream())
    return MoePlan(offsets, order, inv, E, T, k, active)


_TICKETS = {}


def route(x: torch.Tensor, w_router: torch.Tensor, E: int, k: int, norm_topk: bool,
          split: Optional[Tuple[torch.Tensor, Optional[torch.Tensor]]] = None):
    """Routing of a step: `router_topk` and `moe_plan` together -> (idx, weights, extra, plan).

    Up to `TUNING["router_fused_max_rows"]` rows this is one launch: blocks compute the
    logits, and the block that finishes last selects for every row and builds the plan."""
    _chk(x, "x"); _chk(w_router, "w_router", torch.float32)
    T, H = x.shape
    if T == 0 or T > TUNING["router_fused_max_rows"]:
        idx, wts, ext = router_topk(x, w_router, E, k, norm_topk, split=split)
        return idx, wts, ext, moe_plan(idx, E)
    dev = x.device
    extra = w_router.shape[0] - E
    idx = torch.empty((T, k), dtype=torch.int32, device=dev)
    wts = torch.empty((T, k), dtype=torch.float32, device=dev)
    ext = torch.empty((T, extra), dtype=torch.float32, device=dev) if extra > 0 else None
    logits = torch.empty((T, E + extra), dtype=torch.float32, device=dev)
    offsets = torch.empty((E + 1,), dtype=torch.int32, device=dev)
    order = torch.empty((T * k,), dtype=torch.int32, device=dev)
    inv = torch.empty((T * k,), dtype=torch.int32, device=dev)
    active = torch.empty((min(E, T * k),), dtype=torch.int32, device=dev)
    if (T <= TUNING["router_cluster_max_rows"] and x.is_contiguous()
            and _lib.load().nf_router_cluster_fits(T, H, E, extra, k)):
        # one thread-block cluster: logits meet selection and plan in distributed shared memory
        _lib.call("nf_router_cluster", _p(x), _p(w_router), c_int(T), c_int(H), c_int(E), c_int(extra), c_int(k),
                  c_int(1 if norm_topk else 0), None, _p(idx), _p(wts), _p(ext), _p(offsets), _p(order),
                  _p(inv), _p(active), c_int(active.numel()), c_int(_dt(x)), _stream())
        return idx, wts, ext, MoePlan(offsets, order, inv, E, T, k, active)
    key = str(dev)
    if key not in _TICKETS:
        _TICKETS[key] = torch.zeros((1,), dtype=torch.int32, device=dev)
    _lib.call("nf_router_fused", _p(x), _p(w_router), c_int(T), c_int(H), c_int(E), c_int(extra), c_int(k),
              c_int(1 if norm_topk else 0), _p(logits), _p(idx), _p(wts), _p(ext), _p(offsets), _p(order),
              _p(inv), _p(active), c_int(active.numel()), _p(_TICKETS[key]), c_int(_dt(x)), _stream())
    return idx, wts, ext, MoePlan(offsets, order, inv, E, T, k, active)


def moe_uses_gathered_rows(x: torch.Tensor, w13) -> bool:
    """Whether `moe_gemm1` would first copy the rows of `x` into sorted order (`moe_gather`)."""
    return isinstance(w13, PackedWeights) and x.shape[0] > TUNING["skinny_moe_max_tokens"]


def moe_gather(x: torch.Tensor, plan: MoePlan, k: int) -> torch.Tensor:
    """Row p of the result is row order[p] // k of `x`: the tokens in the experts' order."""
    _chk(x, "x")
    T, H = x.shape
    xp = torch.empty((T * k, H), dtype=x.dtype, device=x.device)
    if T:
        _lib.call("nf_gather_rows", _p(x), _p(plan.order), c_int(k), _p(xp), c_int(T * k),
                  c_int(H * x.element_size()), _stream())
    return xp


def moe_gemm1(x: torch.Tensor, w13, plan: MoePlan, k: int, gathered: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Sorted pair p (token order[p] // k, expert e) -> silu(x Wgate_e^T) * (x Wup_e^T)  [T*k, I].

    `w13` is [E, 2I, H] (gate rows first), or `PackedWeights` of it for the bfloat16 kernels.
    `gathered`: `moe_gather(x, plan, k)` if the caller has it already."""
    _chk(x, "x")
    T, H = x.shape
    packed = isinstance(w13, PackedWeights)
    if packed:
        E, inner = w13.groups, w13.n_features
        if x.dtype != torch.bfloat16 or w13.K != H or not w13.swiglu:
            raise ValueError("moe_gemm1: packed weights do not fit the activations")
    else:
        _chk(w13, "w13", x.dtype)
        E, two_i, _ = w13.shape
        inner = two_i // 2
    act = torch.empty((T * k, inner), dtype=x.dtype, device=x.device)
    if T == 0:
        return act
    if packed:
        if T <= TUNING["skinny_moe_max_tokens"]:
            _skinny(x, H, w13.data, w13.group_stride, act, T * k, inner, H, E, T, plan.offsets, plan.order,
                    k, True, packed=True, group_map=plan.active)
        else:
            # rows in sorted order, then one tensor-core launch over all experts
            xp = gathered if gathered is not None else moe_gather(x, plan, k)
            _lib.call("nf_grouped_gemm_tc", _p(xp), c_longlong(T * k), _p(w13.data), c_int(E),
                      c_int(inner), c_int(H), _p(plan.offsets), _p(act), c_int(inner), c_int(1), _stream())
        return act
    path = "simt" if x.dtype == torch.float32 else _bf16_path(T, H, "bf16_moe")
    if path == "skinny":
        _skinny(x, H, w13, two_i * H, act, T * k, inner, H, E, T, plan.offsets, plan.order, k, True,
                group_map=plan.active)
    else:
        _gemm_simt(x, H, w13, two_i * H, act, T * k, inner, H, E, T, plan.offsets, plan.order, k, True)
    return act


def moe_gemm2(act: torch.Tensor, w2, plan: MoePlan, plan_is_older: bool = False) -> torch.Tensor:
    """Sorted pair p of expert e -> act[p] Wdown_e^T  [T*k, H].  `w2` is [E, H, I] or packed.

    `plan_is_older`: the plan was complete before the kernel that produced `act` was launched
    (the usual order: router, first product, this).  The streaming kernel then starts fetching
    weights while that kernel is still finishing."""
    _chk(act, "act")
    n, inner = act.shape
    packed = isinstance(w2, PackedWeights)
    if packed:
        E, H = w2.groups, w2.n_features
        if act.dtype != torch.bfloat16 or w2.K != inner or w2.swiglu:
            raise ValueError("moe_gemm2: packed weights do not fit the activations")
    else:
        _chk(w2, "w2", act.dtype)
        E, H, _ = w2.shape
    y = torch.empty((n, H), dtype=act.dtype, device=act.device)
    if n == 0:
        return y
    if packed:
        if plan.num_tokens <= TUNING["skinny_moe_max_tokens"]:
            _skinny(act, inner, w2.data, w2.group_stride, y, n, H, inner, E, plan.num_tokens, plan.offsets,
                    None, 1, False, packed=True, group_map=plan.active, early_index=plan_is_older)
        else:
            _lib.call("nf_grouped_gemm_tc", _p(act), c_longlong(n), _p(w2.data), c_int(E), c_int(H),
                      c_int(inner), _p(plan.offsets), _p(y), c_int(H), c_int(0), _stream())
        return y
    path = "simt" if act.dtype == torch.float32 else _bf16_path(plan.num_tokens, inner, "bf16_moe")
    if path == "skinny":
        _skinny(act, inner, w2, H * inner, y, n, H, inner, E, plan.num_tokens, plan.offsets, None, 1, False,
                group_map=plan.active, early_index=plan_is_older)
    else:
        _gemm_simt(act, inner, w2, H * inner, y, n, H, inner, E, plan.num_tokens, plan.offsets, None, 1, False)
    return y


_STREAM_WORK = {}


def _stream_items(x: torch.Tensor, w13, w2, E: int, k: int, routes: bool = False, shared_chunks: int = 0) -> int:
    """Sixteen-feature groups an item of the persistent experts' kernel covers (8, 4 or 2), or 0 if
    the step does not fit the kernel.  The fewer experts a step selects, the finer the items, so
    that every SM has some; a finer item also needs a smaller ring.  `routes`: the launch is to
    route as well."""
    T, H = x.shape
    if not (isinstance(w13, PackedWeights) and isinstance(w2, PackedWeights) and x.is_cuda):
        return 0
    if T < max(TUNING["moe_stream_min_tokens"], 1) or T > TUNING["moe_stream_max_tokens"] or x.dtype != torch.bfloat16 or not x.is_contiguous():
        return 0
    if routes and T > TUNING["moe_stream_route_max_tokens"]:
        return 0
    if w13.K != H or w2.n_features != H or w2.K != w13.n_features or not w13.swiglu or w2.swiglu:
        return 0
    pairs = T * k
    q = 8 if pairs >= 16 else (4 if pairs >= 8 else 2)
    fits = _lib.load().nf_moe_stream_fits
    while q >= 2 and not fits(H, w13.n_features, pairs, min(E, pairs), q, TUNING["moe_stream_smem_kb"] * 1024,
                              E if routes else 0, shared_chunks * T):
        q //= 2
    return q if q >= 2 else 0


def moe_experts_fit_stream(x: torch.Tensor, w13, w2, plan: MoePlan, k: int) -> bool:
    """Whether `moe_experts` serves this step with the one persistent launch."""
    return plan.active is not None and _stream_items(x, w13, w2, plan.num_experts, k) > 0


def _stream_work(device: torch.device) -> torch.Tensor:
    """The persistent launch's counters and tables: one buffer a device, so its launches must not
    overlap one another - they are issued to one stream (the step's), eagerly or inside its
    graphs, and each leaves the counters at zero."""
    key = str(device)
    if key not in _STREAM_WORK:
        _STREAM_WORK[key] = torch.zeros((int(_lib.load().nf_moe_stream_work_ints()),), dtype=torch.int32, device=device)
    return _STREAM_WORK[key]


def moe_experts(x: torch.Tensor, w13, w2, plan: MoePlan, k: int,
                gathered: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Both products of the routed experts: sorted pair p of expert e ->
    (silu(x Wgate_e^T) * (x Wup_e^T)) Wdown_e^T  [T*k, H].

    A decode step with packed bfloat16 weights is one persistent launch that streams the weights
    of both products through one ring (`moe_stream.cu`); everything else is `moe_gemm1` followed
    by `moe_gemm2`."""
    q = _stream_items(x, w13, w2, plan.num_experts, k) if plan.active is not None else 0
    if not q:
        return moe_gemm2(moe_gemm1(x, w13, plan, k, gathered=gathered), w2, plan, plan_is_older=True)
    T, H = x.shape
    inner = w13.n_features
    act = torch.empty((T * k, inner), dtype=x.dtype, device=x.device)
    y = torch.empty((T * k, H), dtype=x.dtype, device=x.device)
    _lib.call("nf_moe_stream", _p(x), c_int(x.stride(0)), _p(w13.data), c_longlong(w13.group_stride), _p(w2.data),
              c_longlong(w2.group_stride), _p(act), _p(y), c_int(T * k), c_int(T), c_int(H), c_int(inner),
              c_int(w13.groups), c_int(k), _p(plan.offsets), _p(plan.order), _p(plan.active),
              c_int(plan.active.numel()), _p(_stream_work(x.device)), c_int(q),
              c_int(TUNING["moe_stream_smem_kb"] * 1024), None, c_int(0), c_int(0), None, None, None, None, None,
              None, c_longlong(0), None, c_longlong(0), c_int(0), None, None, _stream())
    return y


def pack_shared_expert(w_gate_up: torch.Tensor, w_down: torch.Tensor, chunk: int) -> Tuple[PackedWeights, PackedWeights]:
    """A shared expert's matrices ([2 Is, H] gate rows first, and [H, Is]) as ceil(Is / chunk)
    experts of `chunk` intermediate features each, packed like the routed ones (the last chunk
    padded with zero features, which contribute nothing).  Its output is then the sum of the
    chunks' outputs, and the persistent experts' launch can serve it."""
    _chk(w_gate_up, "w_gate_up", torch.bfloat16); _chk(w_down, "w_down", torch.bfloat16)
    two_is, H = w_gate_up.shape
    inner = two_is // 2
    n = (inner + chunk - 1) // chunk
    g = torch.zeros((n, 2 * chunk, H), dtype=w_gate_up.dtype, device=w_gate_up.device)
    d = torch.zeros((n, H, chunk), dtype=w_down.dtype, device=w_down.device)
    for c in range(n):
        lo, hi = c * chunk, min(inner, (c + 1) * chunk)
        g[c, :hi - lo] = w_gate_up[lo:hi]
        g[c, chunk:chunk + hi - lo] = w_gate_up[inner + lo:inner + hi]
        d[c, :, :hi - lo] = w_down[:, lo:hi]
    return pack_weights(g, swiglu=True), pack_weights(d, swiglu=False)


def can_route_and_run_experts(x: torch.Tensor, w_router: torch.Tensor, w13, w2, E: int, k: int,
                              shared: Optional[Tuple[PackedWeights, PackedWeights]] = None) -> bool:
    """Whether `route_and_run_experts` serves this step (else: `route`, then `moe_experts`)."""
    if not (w_router.dtype == torch.float32 and w_router.is_contiguous() and w_router.shape[1] == x.shape[1]):
        return False
    chunks = 0
    if shared is not None:
        s13, s2 = shared
        if not (isinstance(w13, PackedWeights) and s13.n_features == w13.n_features and s13.K == w13.K
                and s2.n_features == x.shape[1] and s2.K == w13.n_features and k + s13.groups <= 32):
            return False
        chunks = s13.groups
        if x.shape[0] > TUNING["moe_stream_shared_max_tokens"]:
            return False
    return _stream_items(x, w13, w2, E, k, routes=True, shared_chunks=chunks) > 0


def route_and_run_experts(x: torch.Tensor, w_router: torch.Tensor, E: int, k: int, norm_topk: bool, w13, w2,
                          shared: Optional[Tuple[PackedWeights, PackedWeights]] = None):
    """`route` and `moe_experts` in the one persistent launch: its CTAs compute the router logits
    between them, the one that finishes last selects and writes the plan, and all go on to the
    experts' products.  Returns (idx, weights, extra, plan, y) as the two calls would.

    With `shared` (`pack_shared_expert`) the launch serves the shared expert too, as further
    experts that every token has - their weights are on their way while the routing is still
    being computed.  Then y has T * (k + chunks) rows, and two more values are returned: the
    weights [T, k + chunks] (the k experts', then sigmoid of the first further logit for every
    chunk, or 1 without one) and a plan whose `inv` [T * (k + chunks)] names the rows of y to add
    up for every token - what `moe_combine` and the fused norm take."""
    chunks = shared[0].groups if shared is not None else 0
    q = _stream_items(x, w13, w2, E, k, routes=True, shared_chunks=chunks)
    if not q:
        raise ValueError("route_and_run_experts: the step does not fit the launch")
    T, H = x.shape
    dev = x.device
    inner = w13.n_features
    extra = w_router.shape[0] - E
    rows = T * (k + chunks)
    idx = torch.empty((T, k), dtype=torch.int32, device=dev)
    wts = torch.empty((T, k), dtype=torch.float32, device=dev)
    ext = torch.empty((T, extra), dtype=torch.float32, device=dev) if extra > 0 else None
    logits = torch.empty((T, E + extra), dtype=torch.float32, device=dev)
    offsets = torch.empty((E + 1,), dtype=torch.int32, device=dev)
    order = torch.empty((T * k,), dtype=torch.int32, device=dev)
    inv = torch.empty((T * k,), dtype=torch.int32, device=dev)
    active = torch.empty((min(E, T * k),), dtype=torch.int32, device=dev)
    act = torch.empty((rows, inner), dtype=x.dtype, device=dev)
    y = torch.empty((rows, H), dtype=x.dtype, device=dev)
    cw = torch.empty((T, k + chunks), dtype=torch.float32, device=dev) if chunks else None
    cinv = torch.empty((rows,), dtype=torch.int32, device=dev) if chunks else None
    s13, s2 = shared if shared is not None else (None, None)
    _lib.call("nf_moe_stream", _p(x), c_int(x.stride(0)), _p(w13.data), c_longlong(w13.group_stride), _p(w2.data),
              c_longlong(w2.group_stride), _p(act), _p(y), c_int(T * k), c_int(T), c_int(H), c_int(inner),
              c_int(E), c_int(k), _p(offsets), _p(order), _p(active), c_int(active.numel()),
              _p(_stream_work(dev)), c_int(q), c_int(TUNING["moe_stream_smem_kb"] * 1024), _p(w_router),
              c_int(extra), c_int(1 if norm_topk else 0), _p(logits), _p(idx), _p(wts), _p(ext), _p(inv),
              _p(s13.data) if chunks else None, c_longlong(s13.group_stride if chunks else 0),
              _p(s2.data) if chunks else None, c_longlong(s2.group_stride if chunks else 0), c_int(chunks),
              _p(cw), _p(cinv), _stream())
    plan = MoePlan(offsets, order, inv, E, T, k, active)
    if not chunks:
        return idx, wts, ext, plan, y
    return idx, wts, ext, plan, y, cw, MoePlan(offsets, order, cinv, E, T, k + chunks, active)


def moe_combine(y: torch.Tensor, plan: MoePlan, wts: torch.Tensor, shared: Optional[torch.Tensor],
                gate: Optional[torch.Tensor], out_dtype: torch.dtype) -> torch.Tensor:
    """out[t] = sum_j wts[t, j] * y[inv[t, j]] (j ascending) + sigmoid(gate[t]) * shared[t]."""
    _chk(y, "y"); _chk(wts, "wts", torch.float32)
    T, k = wts.shape
    H = y.shape[1]
    out = torch.empty((T, H), dtype=out_dtype, device=y.device)
    _lib.call("nf_moe_combine", _p(y), _p(plan.inv), _p(wts), _p(shared), _p(gate),
              c_int(gate.shape[1] if gate is not None else 0), _p(out), c_int(T), c_int(H), c_int(k),
              c_int(_dt(y)), _stream())
    return out


FUSED_COMBINE_MAX_K = 32


def can_fuse_combine_norm(y: torch.Tensor, hidden: int, rows: int, k: int = 1) -> bool:
    """Whether `moe_combine_add_rmsnorm` serves these operands (bfloat16 on the device, a row that
    the kernel's threads can keep in registers, few enough rows)."""
    return (y.is_cuda and y.dtype == torch.bfloat16 and rows <= TUNING["fuse_combine_norm_max_rows"]
            and k <= FUSED_COMBINE_MAX_K and bool(_lib.load().nf_moe_combine_add_rmsnorm_fits(c_int(hidden))))


def moe_combine_add_rmsnorm(y: torch.Tensor, plan: MoePlan, wts: torch.Tensor, shared: Optional[torch.Tensor],
                            gate: Optional[torch.Tensor], h: torch.Tensor, rows: Optional[torch.Tensor],
                            weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """`moe_combine` and `add_rmsnorm` (`rows` None: h updated in place) or `add_rmsnorm_rows` in
    one launch, bit for bit what the two give one after the other."""
    _chk(y, "y", torch.bfloat16); _chk(wts, "wts", torch.float32); _chk(h, "h", torch.float32)
    _chk(weight, "weight", torch.float32); _chk(out, "out", torch.bfloat16)
    T, k = wts.shape
    R = T if rows is None else rows.numel()
    _lib.call("nf_moe_combine_add_rmsnorm", _p(y), _p(plan.inv), _p(wts), _p(shared), _p(gate),
              c_int(gate.shape[1] if gate is not None else 0), _p(h), _p(rows), _p(weight), c_float(eps),
              _p(out), c_int(T), c_int(R), c_int(h.shape[1]), c_int(k), _stream())


# ---------------------------------------------------------------------------------------
# sampling
# ---------------------------------------------------------------------------------------

SAMPLE_MAX_TOP_K = 1024


def argmax_rows(logits: torch.Tensor) -> torch.Tensor:
    """First maximum of each row of float32 logits [R, V] -> int32 [R]."""
    _chk(logits, "logits", torch.float32)
    R, V = logits.shape
    out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    chunks = int(_lib.load().nf_argmax_chunks(c_int(R), c_int(V))) if R else 1
    if chunks > 1:
        # a long row is cut into pieces so that the whole device reads it
        sv = torch.empty((R, chunks), dtype=torch.float32, device=logits.device)
        si = torch.empty((R, chunks), dtype=torch.int32, device=logits.device)
        _lib.call("nf_argmax_rows_split", _p(logits), c_int(R), c_int(V), c_int(chunks), _p(sv), _p(si),
                  _p(out), _stream())
        return out
    _lib.call("nf_argmax_rows", _p(logits), c_int(R), c_int(V), _p(out), _stream())
    return out


def repetition_penalty(logits: torch.Tensor, ids: torch.Tensor, counts: torch.Tensor,
                       row_of: torch.Tensor, penalty: torch.Tensor) -> None:
    """In place: for pair i, logits[row_of[i], ids[i]] is divided (if positive) or multiplied
    (if not) by penalty[row] `counts[i]` times."""
    _chk(logits, "logits", torch.float32); _chk(ids, "ids", torch.int32)
    _chk(counts, "counts", torch.int32); _chk(row_of, "row_of", torch.int32)
    _chk(penalty, "penalty", torch.float32)
    _lib.call("nf_repetition_penalty", _p(logits), c_int(logits.shape[1]), _p(ids), _p(counts),
              _p(row_of), _p(penalty), c_int(ids.numel()), _stream())


def sample_rows(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
                top_p: torch.Tensor, draw: torch.Tensor) -> torch.Tensor:
    """One token per row from softmax(logits / temperature) limited by top-k and top-p,
    using the uniform draws `draw` in [0, 1).  The caller has checked the parameters."""
    _chk(logits, "logits", torch.float32); _chk(temperature, "temperature", torch.float32)
    _chk(top_k, "top_k", torch.int32); _chk(top_p, "top_p", torch.float32)
    _chk(draw, "draw", torch.float32)
    R, V = logits.shape
    out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    _lib.call("nf_sample_rows", _p(logits), c_int(R), c_int(V), _p(temperature), _p(top_k),
              _p(top_p), _p(draw), _p(out), _stream())
    return out
