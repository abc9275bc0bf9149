"""Quantised weight containers and GGUF -> tensor loading."""
from __future__ import annotations

import warnings
from dataclasses import dataclass

import numpy as np
import torch

from ..gguf import quants
from ..gguf.reader import GGUFFile
from ..gguf.types import GGMLType, block_size, row_bytes


@dataclass
class QWeight:
    """A tensor kept in its on-disk GGML encoding.

    ``shape`` is row-major (outermost first); rows (the last dimension) are the quantisation axis,
    so any leading-dimension slice is a contiguous byte range.
    """

    name: str
    dtype: GGMLType
    shape: tuple[int, ...]
    raw: torch.Tensor            # flat uint8

    @property
    def row_nbytes(self) -> int:
        return row_bytes(self.dtype, self.shape[-1])

    @property
    def nbytes(self) -> int:
        return self.raw.numel()

    def dequant(self, dtype=torch.float32) -> torch.Tensor:
        return quants.dequantize_tensor(self.raw, self.dtype, self.shape).to(dtype)

    def rows(self, start: int, stop: int) -> "QWeight":
        """Slice of the outermost dimension."""
        inner = self.raw.numel() // self.shape[0]
        return QWeight(self.name, self.dtype, (stop - start,) + tuple(self.shape[1:]), self.raw[start * inner: stop * inner])

    def cols(self, start: int, stop: int) -> "QWeight":
        """Slice of the innermost (quantisation) dimension; both ends must fall on block boundaries."""
        bs = block_size(self.dtype)
        if start % bs or stop % bs or not 0 <= start < stop <= self.shape[-1]:
            raise ValueError(f"{self.name}: columns [{start}, {stop}) do not fall on {bs}-element block boundaries")
        rb = self.row_nbytes
        per = rb // (self.shape[-1] // bs)
        raw = self.raw.view(-1, rb)[:, start // bs * per: stop // bs * per].contiguous().view(-1)
        return QWeight(self.name, self.dtype, tuple(self.shape[:-1]) + (stop - start,), raw)

    def expert(self, e: int) -> "QWeight":
        inner = self.raw.numel() // self.shape[0]
        return QWeight(f"{self.name}[{e}]", self.dtype, tuple(self.shape[1:]), self.raw[e * inner:(e + 1) * inner])

    def to(self, device) -> "QWeight":
        return QWeight(self.name, self.dtype, self.shape, self.raw.to(device))

    @staticmethod
    def from_float(name: str, w: torch.Tensor, dtype: int) -> "QWeight":
        return QWeight(name, GGMLType(dtype), tuple(w.shape), quants.quantize(w, dtype))


def _np_to_torch(a: np.ndarray) -> torch.Tensor:
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        return torch.from_numpy(a)


def load_tensor(g: GGUFFile, name: str, device="cpu") -> QWeight:
    info = g.tensors[name]
    raw = _np_to_torch(g.tensor_bytes(name))
    if str(device) != "cpu":
        raw = raw.to(device, non_blocking=False)
    return QWeight(name, info.dtype, info.torch_shape, raw)


def load_all(g: GGUFFile, device="cpu", skip_prefixes: tuple[str, ...] = ("v.", "mm.", "a.")) -> dict[str, QWeight]:
    """Load every text-model tensor (vision / audio towers embedded in the same blob are skipped)."""
    out = {}
    for name in g.tensors:
        if name.startswith(skip_prefixes):
            continue
        out[name] = load_tensor(g, name, device)
    return out
