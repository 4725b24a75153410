"""Counter-based random weights: the same value for (seed, tensor name, element index) on
the host and on the device.

A model drawn in place on the GPU (tens of gigabytes that never pass through a file) must be
reproducible elsewhere from its seed alone, e.g. by a plain implementation that checks the
engine at full layer sizes.  A library generator cannot give that: CPU and CUDA streams of
the same seed differ.  So an element's value is a pure function of its tensor's key and its
index, built from 32-bit integer arithmetic and two IEEE single-precision operations, which
every machine evaluates to the same bits: the CUDA kernel of ``csrc/random_fill.cu`` and the
torch integer operations below (which run on any torch device).  The reference has no
random-weights mode.

    s   = mix(mix(lo32(i) ^ k1) ^ hi32(i) ^ k2)
    w_j = mix(s ^ C_j), j = 0..3
    n   = (sum of the twelve 10-bit fields of w_0..w_3) - 6138       mean 0, variance 1048575
    z   = float32(n) * float32(1 / sqrt(1048575))                    ~ N(0, 1), |z| < 6
    linear weights and biases: 0.02 * z;   norm weights: 1 + 0.05 * z;   rounded to bfloat16

(k1, k2) are the first eight bytes of SHA-256 of "<seed>:<tensor name>".
"""

from __future__ import annotations

import ctypes
import hashlib
from typing import Tuple

import torch

M32 = 0xFFFFFFFF
STREAMS = (0x9E3779B9, 0x85EBCA6B, 0xC2B2AE35, 0x27D4EB2F)
INV_STD = 9.765629656612873e-4        # float32(1 / sqrt(1048575))
INITS = {"linear": 0, "norm": 1}
_CHUNK = 1 << 24


def tensor_keys(seed: int, name: str) -> Tuple[int, int]:
    d = hashlib.sha256(f"{int(seed)}:{name}".encode()).digest()
    return int.from_bytes(d[:4], "little"), int.from_bytes(d[4:8], "little")


def _mul32(x: torch.Tensor, c: int) -> torch.Tensor:
    """(x * c) mod 2^32 for int64 `x` in [0, 2^32) without leaving 63 bits."""
    lo = (x & 0xFFFF) * c
    hi = ((x >> 16) * c) & 0xFFFF
    return (lo + (hi << 16)) & M32


def _mix(x: torch.Tensor) -> torch.Tensor:
    x = x ^ (x >> 16)
    x = _mul32(x, 0x7FEB352D)
    x = x ^ (x >> 15)
    x = _mul32(x, 0x846CA68B)
    return x ^ (x >> 16)


def draw(first: int, n: int, keys: Tuple[int, int], init: str, device="cpu") -> torch.Tensor:
    """Elements first .. first + n - 1 as float32 holding bfloat16 values (torch integer ops)."""
    k1, k2 = keys
    i = torch.arange(first, first + n, dtype=torch.int64, device=device)
    s = _mix(_mix((i & M32) ^ k1) ^ (i >> 32) ^ k2)
    total = torch.full_like(s, -6138)
    for c in STREAMS:
        w = _mix(s ^ c)
        total += (w & 1023) + ((w >> 10) & 1023) + ((w >> 20) & 1023)
    z = total.to(torch.float32) * torch.tensor(INV_STD, dtype=torch.float32, device=device)
    if INITS[init] == 1:
        v = 1.0 + torch.tensor(0.05, dtype=torch.float32, device=device) * z
    else:
        v = torch.tensor(0.02, dtype=torch.float32, device=device) * z
    return v.to(torch.bfloat16).to(torch.float32)


def fill(out: torch.Tensor, keys: Tuple[int, int], init: str) -> torch.Tensor:
    """Fill the contiguous float32 or bfloat16 tensor `out` (element index = flat index).  On a
    CUDA device the kernel does it in place; elsewhere the torch twin, chunk by chunk."""
    if not out.is_contiguous() or out.dtype not in (torch.float32, torch.bfloat16):
        raise ValueError("fill takes a contiguous float32 or bfloat16 tensor")
    n = out.numel()
    if out.is_cuda:
        from ..kernels import lib as _lib
        with torch.cuda.device(out.device):
            _lib.call("nf_random_fill", ctypes.c_void_p(out.data_ptr()), ctypes.c_longlong(n),
                      ctypes.c_longlong(0), ctypes.c_uint(keys[0]), ctypes.c_uint(keys[1]),
                      ctypes.c_int(INITS[init]), ctypes.c_int(0 if out.dtype == torch.float32 else 1),
                      ctypes.c_void_p(torch.cuda.current_stream(out.device).cuda_stream))
        return out
    flat = out.view(-1)
    for a in range(0, n, _CHUNK):
        b = min(n, a + _CHUNK)
        flat[a:b] = draw(a, b - a, keys, init, out.device).to(out.dtype)
    return out
