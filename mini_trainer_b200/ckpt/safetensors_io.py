"""Minimal safetensors reader/writer (no dependency on the ``safetensors`` package).

File format: 8-byte little-endian header length ``N``; ``N`` bytes of JSON mapping each tensor name
to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the end of the header)
plus an optional ``"__metadata__"`` string map; then the raw little-endian tensor bytes. The
header is space-padded so the data section starts on an 8-byte boundary, as the upstream writer
does. Files written here load with ``safetensors.torch.load_file`` and with HF
``from_pretrained``, and vice versa.
"""
from __future__ import annotations

import json
import mmap
import struct
from typing import Iterable

import numpy as np
import torch

_DTYPES = {
    torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16", torch.float64: "F64",
    torch.int64: "I64", torch.int32: "I32", torch.int16: "I16", torch.int8: "I8", torch.uint8: "U8",
    torch.bool: "BOOL",
}
_FROM = {v: k for k, v in _DTYPES.items()}


def _raw_bytes(t: torch.Tensor) -> memoryview:
    t = t.detach().contiguous().cpu().reshape(-1)   # flat first: a 0-dim tensor has no last dimension to reinterpret
    return memoryview(t.view(torch.uint8).numpy()) if t.numel() else memoryview(b"")


def save_file(tensors: dict, path: str, metadata: dict | None = None) -> None:
    header, off = {}, 0
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    names = sorted(tensors, key=lambda k: (-tensors[k].element_size(), k))  # upstream order: by alignment, then name
    for k in names:
        t = tensors[k]
        n = t.numel() * t.element_size()
        header[k] = {"dtype": _DTYPES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + n]}
        off += n
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for k in names:
            f.write(_raw_bytes(tensors[k]))


def read_header(path: str) -> tuple[dict, int]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n).decode("utf-8"))
    return header, 8 + n


class SafeTensorsFile:
    """Lazy reader: tensors are materialised one at a time from a memory map."""

    def __init__(self, path: str):
        self.path = path
        self.header, self.base = read_header(path)
        self.metadata = self.header.pop("__metadata__", {})
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)

    def keys(self) -> Iterable[str]:
        return self.header.keys()

    def get_tensor(self, name: str) -> torch.Tensor:
        e = self.header[name]
        a, b = e["data_offsets"]
        dt = _FROM[e["dtype"]]
        if b == a:   # an empty tensor has no bytes to reinterpret
            return torch.empty(e["shape"], dtype=dt)
        buf = np.frombuffer(self._mm, dtype=np.uint8, count=b - a, offset=self.base + a).copy()
        return torch.from_numpy(buf).view(dt).reshape(e["shape"])

    def get_slice(self, name: str, lo: int, hi: int) -> torch.Tensor:
        """Elements [lo, hi) of a stored tensor taken as flat, reading only those bytes."""
        e = self.header[name]
        a, b = e["data_offsets"]
        dt = _FROM[e["dtype"]]
        es = torch.empty(0, dtype=dt).element_size()
        lo, hi = max(0, lo), min(hi, (b - a) // es)
        if hi <= lo:
            return torch.empty(0, dtype=dt)
        buf = np.frombuffer(self._mm, dtype=np.uint8, count=(hi - lo) * es, offset=self.base + a + lo * es).copy()
        return torch.from_numpy(buf).view(dt)

    def close(self) -> None:
        self._mm.close()
        self._f.close()


def load_file(path: str) -> dict:
    f = SafeTensorsFile(path)
    try:
        return {k: f.get_tensor(k) for k in f.keys()}
    finally:
        f.close()
