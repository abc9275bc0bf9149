"""GGUF v3 writer.

Same observable layout as the reference writer (fs/ggml/gguf.go:620-782): keys sorted,
keys without an ``<arch>.``/``general.``/``tokenizer.``/``adapter.`` prefix get the architecture
prefix, tensors ordered by block index then name, tensor data aligned to ``general.alignment``
(default 32).
"""
from __future__ import annotations

import os
import re
import struct
from dataclasses import dataclass
from typing import Any, Iterable

import numpy as np

from .reader import (DEFAULT_ALIGNMENT, GGUF_MAGIC, T_ARR, T_BOOL, T_F32, T_F64, T_I32, T_I64, T_STR, T_U32, T_U64,
                     T_I8, T_U8, T_I16, T_U16, _NP, _SCALAR, _padding)
from .types import GGMLType, tensor_bytes


@dataclass
class WriteTensor:
    name: str
    shape: tuple[int, ...]   # GGUF order (innermost first)
    dtype: GGMLType
    data: Any                # bytes-like / numpy array holding the encoded payload, or a callable returning one

    @property
    def nbytes(self) -> int:
        return tensor_bytes(self.dtype, self.shape)

    def block(self) -> int:
        m = re.match(r"^(?:[a-z]+\.)?blk\.(\d+)\.", self.name)
        return int(m.group(1)) if m else -1


class Typed:
    """Force a GGUF value type: ``Typed(T_U32, 5)`` or ``Typed((T_ARR, T_I32), [...])``."""

    def __init__(self, t, v):
        self.t, self.v = t, v


def _infer(v: Any):
    if isinstance(v, Typed):
        return v.t, v.v
    if isinstance(v, bool) or isinstance(v, np.bool_):
        return T_BOOL, bool(v)
    if isinstance(v, (int, np.integer)):
        if isinstance(v, np.integer):
            m = {np.uint8: T_U8, np.int8: T_I8, np.uint16: T_U16, np.int16: T_I16, np.uint32: T_U32,
                 np.int32: T_I32, np.uint64: T_U64, np.int64: T_I64}
            return m.get(type(v), T_I64), int(v)
        if 0 <= v < 1 << 32:
            return T_U32, v
        if v < 0 and v >= -(1 << 31):
            return T_I32, v
        return (T_U64 if v >= 0 else T_I64), v
    if isinstance(v, (float, np.floating)):
        return (T_F64 if isinstance(v, np.float64) else T_F32), float(v)
    if isinstance(v, str):
        return T_STR, v
    if isinstance(v, np.ndarray):
        for t, code in _NP.items():
            if np.dtype(code) == v.dtype.newbyteorder("="):
                return (T_ARR, t), v
        raise TypeError(f"unsupported array dtype {v.dtype}")
    if isinstance(v, (list, tuple)):
        if not v:
            return (T_ARR, T_I32), []
        e = v[0]
        if isinstance(e, str):
            return (T_ARR, T_STR), list(v)
        if isinstance(e, bool):
            return (T_ARR, T_BOOL), list(v)
        if isinstance(e, int):
            if all(0 <= x < 1 << 32 for x in v):
                return (T_ARR, T_U32), list(v)
            return (T_ARR, T_I32 if all(-(1 << 31) <= x < 1 << 31 for x in v) else T_I64), list(v)
        if isinstance(e, float):
            return (T_ARR, T_F32), list(v)
    raise TypeError(f"unsupported GGUF value {type(v)}")


def _pack_str(s: str) -> bytes:
    b = s.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def _pack_value(t, v) -> bytes:
    if isinstance(t, tuple):
        _, et = t
        out = [struct.pack("<IIQ", T_ARR, et, len(v))]
        if et == T_STR:
            out += [_pack_str(s) for s in v]
        else:
            out.append(np.asarray(v, dtype=np.dtype(_NP[et]).newbyteorder("<")).tobytes())
        return b"".join(out)
    if t == T_STR:
        return struct.pack("<I", t) + _pack_str(v)
    fmt, _ = _SCALAR[t]
    return struct.pack("<I", t) + struct.pack("<" + fmt, v)


def _payload(data: Any) -> memoryview:
    if callable(data):
        data = data()
    if hasattr(data, "detach"):  # torch tensor
        data = data.detach().cpu().contiguous().view(-1).view(dtype=__import__("torch").uint8).numpy()
    if isinstance(data, np.ndarray):
        return memoryview(np.ascontiguousarray(data).view(np.uint8).reshape(-1))
    return memoryview(data)


def write_gguf(path: str | os.PathLike, kv: dict[str, Any], tensors: Iterable[WriteTensor]) -> None:
    arch = kv.get("general.architecture")
    if not arch:
        raise ValueError("architecture not set")
    ts = sorted(tensors, key=lambda t: (t.block(), t.name))
    items = []
    for k in sorted(kv):
        key = k
        if not key.startswith((arch + ".", "general.", "adapter.", "tokenizer.")):
            key = f"{arch}.{key}"
        items.append((key, kv[k]))
    alignment = int(kv.get("general.alignment", DEFAULT_ALIGNMENT))

    with open(path, "wb") as f:
        f.write(GGUF_MAGIC)
        f.write(struct.pack("<IQQ", 3, len(ts), len(items)))
        for key, v in items:
            t, val = _infer(v)
            f.write(_pack_str(key))
            f.write(_pack_value(t, val))
        off = 0
        offsets = []
        for t in ts:
            offsets.append(off)
            f.write(_pack_str(t.name))
            f.write(struct.pack("<I", len(t.shape)))
            f.write(struct.pack(f"<{len(t.shape)}Q", *t.shape))
            f.write(struct.pack("<IQ", int(t.dtype), off))
            off += t.nbytes
            off += _padding(off, alignment)
        pos = f.tell()
        base = pos + _padding(pos, alignment)
        f.write(b"\0" * (base - pos))
        for t, o in zip(ts, offsets):
            f.seek(base + o)
            mv = _payload(t.data)
            if len(mv) != t.nbytes:
                raise ValueError(f"tensor {t.name}: payload has {len(mv)} bytes, expected {t.nbytes}")
            f.write(mv)
        end = base + off
        f.seek(0, os.SEEK_END)
        if f.tell() < end:
            f.write(b"\0" * (end - f.tell()))
