"""A small reader and writer of the safetensors file format.

Layout, as the reference reads it (src/core/safetensors.cpp:11-56): an 8-byte
little-endian header length, a JSON header mapping tensor name to
``{dtype, shape, data_offsets: [begin, end]}`` (offsets relative to the first byte
after the header; the ``__metadata__`` entry is skipped), then the raw little-endian
data.  The reference rejects a header longer than 1 GiB and malformed entries; so does
this reader, and it also rejects a file shorter than its offsets claim.

Tensors are memory-mapped and handed out as torch views, so a 30 GB checkpoint costs no
host copy before the host-to-device transfer.
"""

from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Tuple

import torch


class SafetensorsError(RuntimeError):
    pass


_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16,
    "BF16": torch.bfloat16, "I64": torch.int64, "I32": torch.int32,
    "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}
MAX_HEADER = 1 << 30


class TensorInfo:
    __slots__ = ("name", "dtype", "shape", "begin", "end")

    def __init__(self, name: str, dtype: str, shape: Tuple[int, ...], begin: int, end: int):
        self.name, self.dtype, self.shape, self.begin, self.end = name, dtype, shape, begin, end

    @property
    def torch_dtype(self) -> torch.dtype:
        if self.dtype not in _DTYPES:
            raise SafetensorsError(
                f"tensor {self.name!r}: unsupported safetensors dtype {self.dtype!r}")
        return _DTYPES[self.dtype]


class SafetensorsFile:
    """One ``.safetensors`` file, header parsed, data mapped read-only."""

    def __init__(self, path: str):
        self.path = path
        if not os.path.exists(path):
            raise SafetensorsError(f"safetensors file not found: {path}")
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to hold a safetensors header")
        self._fh = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen <= 0 or hlen > MAX_HEADER or 8 + hlen > size:
            raise SafetensorsError(f"{path}: bad safetensors header length {hlen}")
        try:
            header = json.loads(self._fh.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self.data_start = 8 + hlen
        self.metadata = header.pop("__metadata__", None)
        self.tensors: Dict[str, TensorInfo] = {}
        for name, ent in header.items():
            try:
                dtype = ent["dtype"]
                shape = tuple(int(x) for x in ent["shape"])
                begin, end = (int(x) for x in ent["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed entry for tensor {name!r}") from None
            info = TensorInfo(name, dtype, shape, begin, end)
            if begin < 0 or end < begin or self.data_start + end > size:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} claims bytes [{begin}, {end}) but the file holds "
                    f"only {size - self.data_start} data bytes (truncated file?)")
            if dtype in _DTYPES:
                n = 1
                for s in shape:
                    n *= s
                want = n * torch.empty((), dtype=_DTYPES[dtype]).element_size()
                if want != end - begin:
                    raise SafetensorsError(
                        f"{path}: tensor {name!r} of shape {list(shape)} and dtype {dtype} needs "
                        f"{want} bytes, entry gives {end - begin}")
            self.tensors[name] = info
        self._map = None

    def names(self) -> List[str]:
        return list(self.tensors)

    def _mapping(self):
        if self._map is None:
            self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        return self._map

    def read(self, name: str) -> torch.Tensor:
        """The tensor as a read-only view of the mapped file (stored dtype, stored shape)."""
        if name not in self.tensors:
            raise SafetensorsError(f"tensor not found in {self.path}: {name}")
        info = self.tensors[name]
        dt = info.torch_dtype
        count = 1
        for s in info.shape:
            count *= s
        if count == 0:
            return torch.empty(info.shape, dtype=dt)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the buffer is read-only; it is never written
            t = torch.frombuffer(self._mapping(), dtype=dt, count=count,
                                 offset=self.data_start + info.begin)
        return t.reshape(info.shape)

    def close(self) -> None:
        # views handed out keep the mapping alive; dropping our references is enough
        self._map = None
        if self._fh is not None:
            self._fh.close()
            self._fh = None


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]],
                      metadata: Dict[str, str] | None = None) -> None:
    """Write ``(name, tensor)`` pairs in the given order.  Tensors are taken on the CPU."""
    items = [(n, t.detach().cpu().contiguous()) for n, t in tensors]
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    off = 0
    for name, t in items:
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} of tensor {name!r}")
        if name in header:
            raise SafetensorsError(f"tensor name written twice: {name!r}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [off, off + nbytes]}
        off += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)    # keep the data 8-byte aligned
    tmp = path + ".tmp"
    with open(tmp, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for _, t in items:
            if t.numel():
                fh.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else
                         t.reshape(1).view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)
