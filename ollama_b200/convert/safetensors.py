"""safetensors container: 8-byte little-endian header length, a JSON header, raw little-endian tensor data.

The reader memory-maps the file and hands out zero-copy torch views; the writer exists for tests and for
exporting fine-tuned weights.  Counterpart of the reference's x/safetensors reader and of the safetensors
branch of convert/reader.go.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Iterator

import numpy as np
import torch

_DTYPES = {"F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "I64": torch.int64,
           "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
           "F8_E4M3": getattr(torch, "float8_e4m3fn", None), "F8_E5M2": getattr(torch, "float8_e5m2", None)}
_NAMES = {v: k for k, v in _DTYPES.items() if v is not None}
MAX_HEADER = 100 << 20


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    def __init__(self, path: str | os.PathLike):
        self.path = str(path)
        self._f = open(self.path, "rb")
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: truncated header")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n > MAX_HEADER or 8 + n > size:
            raise SafetensorsError(f"{self.path}: header length {n} is out of range")
        try:
            hdr = json.loads(self._f.read(n))
        except ValueError as e:
            raise SafetensorsError(f"{self.path}: header is not JSON: {e}") from None
        self.metadata: dict[str, str] = hdr.pop("__metadata__", {}) or {}
        self.data_start = 8 + n
        self.entries: dict[str, tuple[str, tuple[int, ...], int, int]] = {}
        if not isinstance(hdr, dict) or not isinstance(self.metadata, dict):
            raise SafetensorsError(f"{self.path}: header is not a JSON object")
        for name, e in hdr.items():
            try:
                b, end = (int(v) for v in e["data_offsets"])
                dtype, shape = e["dtype"], tuple(int(d) for d in e["shape"])
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{self.path}: tensor {name} has a malformed header entry") from None
            if dtype not in _DTYPES or _DTYPES[dtype] is None:
                raise SafetensorsError(f"{self.path}: tensor {name} has unsupported dtype {dtype}")
            if not 0 <= b <= end <= size - self.data_start or any(d < 0 for d in shape):
                raise SafetensorsError(f"{self.path}: tensor {name} lies outside the file")
            self.entries[name] = (dtype, shape, b, end)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def keys(self) -> Iterator[str]:
        return iter(self.entries)

    def __contains__(self, name: str) -> bool:
        return name in self.entries

    def shape(self, name: str) -> tuple[int, ...]:
        return self.entries[name][1]

    def tensor(self, name: str) -> torch.Tensor:
        dt, shape, b, e = self.entries[name]
        td = _DTYPES[dt]
        n = int(np.prod(shape)) if shape else 1
        if (e - b) != n * torch.empty((), dtype=td).element_size():
            raise SafetensorsError(f"{self.path}: tensor {name}: {e - b} bytes do not match shape {shape} of {dt}")
        buf = np.frombuffer(self._mm, dtype=np.uint8, count=e - b, offset=self.data_start + b)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            t = torch.from_numpy(buf)
        return t.view(td).view(*shape) if shape else t.view(td).reshape(())

    def close(self) -> None:
        if self._mm is not None:
            try:
                self._mm.close()
            except BufferError:        # tensor views of the mapping are still alive: the mapping goes away with the last of them
                pass
            self._mm = None
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def save_file(tensors: dict[str, torch.Tensor], path: str | os.PathLike, metadata: dict[str, str] | None = None) -> None:
    hdr: dict = {}
    if metadata:
        hdr["__metadata__"] = metadata
    off = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        hdr[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    h = json.dumps(hdr, separators=(",", ":")).encode()
    h += b" " * (-len(h) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for raw in blobs:
            f.write(raw)


class ModelDir:
    """All ``*.safetensors`` shards of a checkpoint directory behind one name -> tensor mapping."""

    def __init__(self, path: str | os.PathLike):
        self.files = [SafetensorsFile(os.path.join(path, n)) for n in sorted(os.listdir(path)) if n.endswith(".safetensors")]
        if not self.files:
            raise SafetensorsError(f"{path}: no .safetensors files")
        self.index = {name: f for f in self.files for name in f.keys()}

    def keys(self):
        return self.index.keys()

    def __contains__(self, name: str) -> bool:
        return name in self.index

    def tensor(self, name: str) -> torch.Tensor:
        return self.index[name].tensor(name)

    def close(self) -> None:
        for f in self.files:
            f.close()
