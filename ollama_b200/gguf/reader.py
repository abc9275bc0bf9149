"""GGUF container reader (versions 1-3, little- and big-endian).

Behavioural parity targets in the reference:
  * eager decoder fs/ggml/gguf.go:146-311 (KV decode, tensor table, bounds and
    overflow checks, alignment handling at :253-267),
  * lazy reader fs/gguf/gguf.go:16-101 (limits: 16 MiB strings, 64 Mi array
    elements, 4 tensor dims).

The file is memory-mapped; tensor payloads are returned as zero-copy numpy
``uint8`` views so that a 40 GB checkpoint can be opened without reading it.
"""
from __future__ import annotations

import mmap
import os
import struct
from dataclasses import dataclass, field
from typing import Any, BinaryIO, Iterator

import numpy as np

from .types import GGMLType, tensor_bytes, _LAYOUT

GGUF_MAGIC = b"GGUF"
MAX_STRING_LENGTH = 16 << 20
MAX_ARRAY_SIZE = 64 << 20
MAX_TENSOR_DIMS = 4
DEFAULT_ALIGNMENT = 32

# value type ids
T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64 = range(13)

_SCALAR = {
    T_U8: ("B", 1), T_I8: ("b", 1), T_U16: ("H", 2), T_I16: ("h", 2), T_U32: ("I", 4), T_I32: ("i", 4),
    T_F32: ("f", 4), T_BOOL: ("?", 1), T_U64: ("Q", 8), T_I64: ("q", 8), T_F64: ("d", 8),
}
_NP = {
    T_U8: "u1", T_I8: "i1", T_U16: "u2", T_I16: "i2", T_U32: "u4", T_I32: "i4",
    T_F32: "f4", T_BOOL: "?", T_U64: "u8", T_I64: "i8", T_F64: "f8",
}


class GGUFError(ValueError):
    pass


@dataclass
class TensorInfo:
    name: str
    shape: tuple[int, ...]          # GGUF order: shape[0] is the contiguous (innermost) dimension
    dtype: GGMLType
    offset: int                      # relative to the start of the tensor-data section
    nbytes: int = 0

    @property
    def n_elements(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n

    @property
    def torch_shape(self) -> tuple[int, ...]:
        """Row-major shape (outermost first), i.e. the GGUF dims reversed."""
        return tuple(reversed(self.shape))


@dataclass
class GGUFFile:
    path: str
    version: int
    byte_order: str
    kv: dict[str, Any]
    kv_types: dict[str, Any]
    tensors: dict[str, TensorInfo]
    data_offset: int
    alignment: int
    _mm: Any = field(default=None, repr=False)
    _buf: Any = field(default=None, repr=False)

    # -- metadata helpers (fs/ggml/ggml.go:33-304 style accessors) -------------------
    @property
    def architecture(self) -> str:
        return str(self.kv.get("general.architecture", "unknown"))

    def key(self, k: str) -> str:
        if k.startswith(("general.", "tokenizer.", "adapter.")) or k.startswith(self.architecture + "."):
            return k
        return f"{self.architecture}.{k}"

    def get(self, k: str, default: Any = None) -> Any:
        return self.kv.get(self.key(k), default)

    def uint(self, k: str, default: int = 0) -> int:
        v = self.get(k)
        if v is None:
            return default
        if isinstance(v, (list, np.ndarray)):
            return int(v[0]) if len(v) else default
        return int(v)

    def float(self, k: str, default: float = 0.0) -> float:
        v = self.get(k)
        return default if v is None else float(v)

    def string(self, k: str, default: str = "") -> str:
        v = self.get(k)
        return default if v is None else str(v)

    def bool(self, k: str, default: bool = False) -> bool:
        v = self.get(k)
        return default if v is None else bool(v)

    def array(self, k: str, default: Any = None) -> Any:
        v = self.get(k)
        return default if v is None else v

    def per_layer(self, k: str, n_layers: int, default: int = 0) -> list[int]:
        """A KV that may be a scalar or a per-layer array (e.g. ``attention.head_count_kv``)."""
        v = self.get(k)
        if v is None:
            return [default] * n_layers
        if isinstance(v, (list, np.ndarray)):
            out = [int(x) for x in v]
            if len(out) < n_layers:
                out += [out[-1] if out else default] * (n_layers - len(out))
            return out[:n_layers]
        return [int(v)] * n_layers

    # -- tensor payload access -------------------------------------------------------
    def tensor_bytes(self, name: str) -> np.ndarray:
        info = self.tensors[name]
        start = self.data_offset + info.offset
        return np.frombuffer(self._buf, dtype=np.uint8, count=info.nbytes, offset=start)

    def has(self, name: str) -> bool:
        return name in self.tensors

    def close(self) -> None:
        self._buf = None
        if self._mm is not None:
            try:
                self._mm.close()
            except BufferError:
                pass  # outstanding numpy views keep the mapping alive; the OS reclaims it later
            self._mm = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


class _Cursor:
    def __init__(self, buf, size: int):
        self.buf = buf
        self.size = size
        self.pos = 0
        self.bo = "<"
        self.v1 = False

    def need(self, n: int) -> None:
        if n < 0 or self.pos + n > self.size:
            raise GGUFError("unexpected end of file")

    def unpack(self, fmt: str, n: int):
        self.need(n)
        v = struct.unpack_from(self.bo + fmt, self.buf, self.pos)[0]
        self.pos += n
        return v

    def u32(self) -> int:
        return self.unpack("I", 4)

    def u64(self) -> int:
        return self.unpack("Q", 8)

    def length(self) -> int:
        return self.u32() if self.v1 else self.u64()

    def string(self) -> str:
        n = self.length()
        if n > MAX_STRING_LENGTH:
            raise GGUFError(f"string length {n} exceeds the {MAX_STRING_LENGTH} byte limit")
        self.need(n)
        s = bytes(self.buf[self.pos:self.pos + n])
        self.pos += n
        return s.decode("utf-8", errors="replace")

    def value(self, t: int, max_array: int) -> Any:
        if t in _SCALAR:
            fmt, n = _SCALAR[t]
            return self.unpack(fmt, n)
        if t == T_STR:
            return self.string()
        if t == T_ARR:
            et = self.u32()
            n = self.length()
            if n > MAX_ARRAY_SIZE:
                raise GGUFError(f"array size {n} exceeds the {MAX_ARRAY_SIZE} element limit")
            if et in _NP:
                width = _SCALAR[et][1]
                self.need(n * width)
                arr = np.frombuffer(self.buf, dtype=np.dtype(_NP[et]).newbyteorder(self.bo), count=n, offset=self.pos)
                self.pos += n * width
                if max_array >= 0 and n > max_array:
                    return _ElidedArray(et, n)
                return arr
            if et == T_STR:
                if max_array >= 0 and n > max_array:
                    for _ in range(n):  # skip without materialising
                        ln = self.length()
                        if ln > MAX_STRING_LENGTH:
                            raise GGUFError("string length exceeds limit")
                        self.need(ln)
                        self.pos += ln
                    return _ElidedArray(et, n)
                return [self.string() for _ in range(n)]
            if et == T_ARR:
                return [self.value(T_ARR, max_array) for _ in range(n)]
            raise GGUFError(f"invalid array element type {et}")
        raise GGUFError(f"invalid value type {t}")


class _ElidedArray:
    """Placeholder for an array longer than ``max_array`` (``/api/show`` elides long arrays)."""

    def __init__(self, elem_type: int, n: int):
        self.elem_type = elem_type
        self.n = n

    def __len__(self) -> int:
        return self.n

    def __repr__(self) -> str:
        return f"<array of {self.n}>"


def _padding(offset: int, align: int) -> int:
    return (align - offset % align) % align


def open_gguf(path: str | os.PathLike, max_array: int = -1, metadata_only: bool = False) -> GGUFFile:
    """Open ``path``; ``max_array`` >= 0 elides KV arrays longer than that (metadata browsing)."""
    path = os.fspath(path)
    f = open(path, "rb")
    try:
        size = os.fstat(f.fileno()).st_size
        if size < 8:
            raise GGUFError("file too small to be GGUF")
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
    finally:
        f.close()
    buf = memoryview(mm)
    c = _Cursor(buf, size)
    if bytes(buf[:4]) != GGUF_MAGIC:
        raise GGUFError("invalid file magic")
    c.pos = 4
    version = c.u32()
    if version & 0xFFFF == 0 and version != 0:  # byte-swapped version -> big-endian file
        c.bo = ">"
        version = struct.unpack(">I", struct.pack("<I", version))[0]
    if version not in (1, 2, 3):
        raise GGUFError(f"unsupported GGUF version {version}")
    c.v1 = version == 1
    n_tensors = c.length()
    n_kv = c.length()
    if n_kv > size or n_tensors > size:
        raise GGUFError("implausible header counts")

    kv: dict[str, Any] = {}
    kv_types: dict[str, Any] = {}
    for _ in range(n_kv):
        k = c.string()
        t = c.u32()
        kv_types[k] = t
        kv[k] = c.value(t, max_array)

    tensors: dict[str, TensorInfo] = {}
    for _ in range(n_tensors):
        name = c.string()
        nd = c.u32()
        if nd > MAX_TENSOR_DIMS:
            raise GGUFError(f"tensor {name!r} has {nd} dimensions (max {MAX_TENSOR_DIMS})")
        shape = tuple(c.u64() for _ in range(nd))
        tt = c.u32()
        try:
            gt = GGMLType(tt)
        except ValueError:
            raise GGUFError(f"tensor {name!r} has unknown type {tt}") from None
        off = c.u64()
        n = 1
        for d in shape:
            if d == 0 or d > 1 << 40:
                raise GGUFError(f"tensor {name!r} has an invalid dimension {d}")
            n *= d
            if n > 1 << 62:
                raise GGUFError(f"tensor {name!r} element count overflows")
        bs = _LAYOUT[gt][0]
        if shape and shape[0] % bs:
            raise GGUFError(f"tensor {name!r}: row length {shape[0]} is not a multiple of block size {bs}")
        tensors[name] = TensorInfo(name, shape, gt, off, tensor_bytes(gt, shape))

    alignment = int(kv.get("general.alignment", DEFAULT_ALIGNMENT)) or DEFAULT_ALIGNMENT
    data_offset = c.pos + _padding(c.pos, alignment)
    if not metadata_only:
        for ti in tensors.values():
            if ti.offset % alignment:
                raise GGUFError(f"tensor {ti.name!r} offset {ti.offset} is not {alignment}-byte aligned")
            if data_offset + ti.offset + ti.nbytes > size:
                raise GGUFError(f"tensor {ti.name!r} data exceeds the file size")
    return GGUFFile(path, version, c.bo, kv, kv_types, tensors, data_offset, alignment, mm, buf)


def iter_kv(path: str, max_array: int = 0) -> Iterator[tuple[str, Any]]:
    """Streaming-style metadata walk used by `/api/show` (long arrays elided)."""
    g = open_gguf(path, max_array=max_array, metadata_only=True)
    try:
        yield from g.kv.items()
    finally:
        g.close()


def is_gguf(fh: BinaryIO) -> bool:
    pos = fh.tell()
    try:
        return fh.read(4) == GGUF_MAGIC
    finally:
        fh.seek(pos)
