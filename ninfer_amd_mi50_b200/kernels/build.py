"""Compiling the CUDA sources of `csrc/` into one shared library, in the tree.

The reference builds with CMake for exactly one architecture and refuses any other
(CMakeLists.txt:7-14); this build does the same for sm_100a, but at first use, so that a
fresh checkout needs no build step.  Objects and the library live in
``<package>/_build`` (or, if the package folder is read-only, in a per-user folder under
the system's temporary directory).  A content hash of the sources and flags decides
whether anything has to be rebuilt, so copied trees with fresh timestamps do not
recompile.  While it compiles it prints a line per file on stderr.
"""

from __future__ import annotations

import concurrent.futures
import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
import time
from typing import List, Optional

PKG_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC_DIR = os.path.join(PKG_DIR, "csrc")
LIB_NAME = "libninfer_b200.so"
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    sys.stderr.write(f"[ninfer build] {msg}\n")
    sys.stderr.flush()


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                 shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("nvcc not found (set NVCC or CUDA_HOME); the CUDA kernels cannot be built "
                     "and there is no other implementation")


def sources() -> List[str]:
    return sorted(f for f in os.listdir(SRC_DIR) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(SRC_DIR) if f.endswith((".cuh", ".h")))


def _digest(paths: List[str], extra: str = "") -> str:
    h = hashlib.sha256(extra.encode())
    for p in paths:
        h.update(p.encode())
        with open(os.path.join(SRC_DIR, p), "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()[:20]


def build_dir() -> str:
    d = os.environ.get("NINFER_BUILD_DIR") or os.path.join(PKG_DIR, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"ninfer_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def library_path() -> str:
    return os.path.join(build_dir(), LIB_NAME)


def is_current() -> bool:
    d = build_dir()
    meta = os.path.join(d, "build.json")
    if not (os.path.exists(meta) and os.path.exists(os.path.join(d, LIB_NAME))):
        return False
    try:
        with open(meta) as fh:
            return json.load(fh).get("digest") == _digest(sources() + _headers(), " ".join(NVCC_FLAGS))
    except (OSError, ValueError):
        return False


def build(verbose: bool = True, force: bool = False, ptxas_info: bool = False) -> str:
    """Compile what is stale and link; return the library's path."""
    d = build_dir()
    lib = os.path.join(d, LIB_NAME)
    if not force and is_current():
        return lib
    nvcc = find_nvcc()
    hdr_digest = _digest(_headers(), " ".join(NVCC_FLAGS))
    srcs = sources()
    todo = []
    objs = []
    for s in srcs:
        obj = os.path.join(d, s[:-3] + ".o")
        stamp = obj + ".digest"
        want = _digest([s], hdr_digest)
        objs.append(obj)
        have = open(stamp).read() if os.path.exists(stamp) and os.path.exists(obj) else ""
        if force or have != want:
            todo.append((s, obj, stamp, want))
    t0 = time.time()
    if verbose and todo:
        _say(f"compiling {len(todo)} of {len(srcs)} CUDA files for sm_100a into {d}")

    def compile_one(item):
        s, obj, stamp, want = item
        cmd = [nvcc, *NVCC_FLAGS, "-I", SRC_DIR, "-c", os.path.join(SRC_DIR, s), "-o", obj]
        if ptxas_info:
            cmd[1:1] = ["-Xptxas", "-v"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"nvcc failed on {s}:\n{r.stderr[-4000:]}")
        with open(stamp, "w") as fh:
            fh.write(want)
        if verbose:
            _say(f"  {s} done ({time.time() - t0:.0f}s)")
        return r.stderr

    logs = []
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(todo)))) as ex:
        for out in ex.map(compile_one, todo):
            logs.append(out)
    tmp = lib + f".{os.getpid()}.tmp"
    r = subprocess.run([nvcc, "-shared", "-o", tmp, *objs], capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"linking {LIB_NAME} failed:\n{r.stderr[-4000:]}")
    os.replace(tmp, lib)
    with open(os.path.join(d, "build.json"), "w") as fh:
        json.dump({"digest": _digest(srcs + _headers(), " ".join(NVCC_FLAGS)), "sources": srcs}, fh)
    if verbose:
        _say(f"built {lib} in {time.time() - t0:.0f}s")
    if ptxas_info:
        return "\n".join(logs)
    return lib


if __name__ == "__main__":
    out = build(force="--force" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(out)
