"""Reading and writing of safetensors files: an 8-byte little-endian header
length, a JSON header {name: {dtype, shape, data_offsets}}, then the raw
little-endian tensor bytes.  Tensors are memory-mapped, not copied, on read."""
from __future__ import annotations

import json
import mmap
import os
import struct

import numpy as np
import torch


class SafetensorsError(ValueError):
    pass


_DTYPES = {
    "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2), "F32": (torch.float32, 4), "F64": (torch.float64, 8),
    "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "I16": (torch.int16, 2), "I32": (torch.int32, 4),
    "I64": (torch.int64, 8), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """One opened file; `tensor(name)` gives a read-only view into the mapping."""

    def __init__(self, path: str):
        self.path = path
        try:
            size = os.path.getsize(path)
            self._f = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"{path}: cannot open ({e.strerror})") from None
        if size < 8:
            raise SafetensorsError(f"{path}: too short for a safetensors header ({size} bytes)")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > size - 8 or hlen > (100 << 20):
            raise SafetensorsError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(hlen))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        self.metadata = header.pop("__metadata__", {})
        self._base = 8 + hlen
        self._size = size
        self.entries: dict[str, dict] = {}
        for name, e in header.items():
            dt = e.get("dtype")
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {dt!r}")
            shape = e.get("shape")
            b, end = e.get("data_offsets", (None, None))
            n = int(np.prod(shape, dtype=np.int64)) if shape else 1
            if b is None or end - b != n * _DTYPES[dt][1] or self._base + end > size or b < 0:
                raise SafetensorsError(f"{path}: tensor '{name}' ({dt} {shape}) does not fit its byte range "
                                       f"[{b}, {end}) in a file of {size} bytes (truncated file?)")
            self.entries[name] = {"dtype": dt, "shape": tuple(shape), "begin": b, "end": end}
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self):
        return list(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        dtype, _ = _DTYPES[e["dtype"]]
        n = int(np.prod(e["shape"], dtype=np.int64)) if e["shape"] else 1
        if n == 0:
            return torch.empty(e["shape"], dtype=dtype)
        buf = memoryview(self._map)[self._base + e["begin"]: self._base + e["end"]]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the mapping is read-only; the tensor is only read
            t = torch.frombuffer(buf, dtype=dtype, count=n)
        return t.reshape(e["shape"])


def write_safetensors(path: str, tensors: dict[str, torch.Tensor], metadata: dict | None = None) -> None:
    header = {}
    offset = 0
    order = list(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}': dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-len(blob) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    os.replace(tmp, path)
