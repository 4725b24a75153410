"""Loading the kernel library and calling into it.

The library is plain C ABI (``extern "C" int nf_*``), loaded with ctypes like the
reference's Python wrapper loads ``libninfer.so`` (tools/ninfer_ctypes.py:20-33).  There is
no other implementation behind these calls: if the library cannot be built or loaded,
the first call raises.
"""

from __future__ import annotations

import ctypes
import os
import threading
from typing import Optional

from . import build as _build

_lib: Optional[ctypes.CDLL] = None
_lock = threading.Lock()


class KernelError(RuntimeError):
    pass


def load() -> ctypes.CDLL:
    """Build if needed, then load.  Raises if there is no CUDA library to call."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            path = _build.build(verbose=True)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelError(f"cannot load the CUDA kernel library {path}: {e}") from None
            lib.nf_last_error.restype = ctypes.c_char_p
            mask = os.environ.get("NINFER_CHAINED_LAUNCH")
            if mask is not None:
                # 0: plain launches (every kernel waits for the one before); otherwise a mask of the
                # kernel classes that keep the attribute: 1 streaming products, 2 norm and combine,
                # 4 rotary, 8 decode attention, 16 router
                lib.nf_set_chained_launch(int(mask))
            if os.environ.get("NINFER_SKINNY_MAX_SPLIT"):
                lib.nf_set_skinny_max_split(int(os.environ["NINFER_SKINNY_MAX_SPLIT"]))   # 1: no split over k
            if os.environ.get("NINFER_CHAINED_OUTSIDE_CAPTURE") == "0":
                lib.nf_set_chained_launch_outside_capture(0)     # chained launches only inside a stream capture
            _lib = lib
    return _lib


_launches = 0


def launch_count() -> int:
    """Kernel launches made through this library so far (one per successful call)."""
    return _launches


def count_launches(n: int) -> None:
    """Account for launches made outside `call` (a replayed CUDA graph's kernels)."""
    global _launches
    _launches += n


def call(name: str, *args) -> None:
    global _launches
    lib = load()
    _launches += 1
    rc = getattr(lib, name)(*args)
    if rc != 0:
        raise KernelError(f"{name}: {lib.nf_last_error().decode(errors='replace')}")


def is_loaded() -> bool:
    return _lib is not None
