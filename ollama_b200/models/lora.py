"""LoRA adapters (Modelfile ADAPTER): GGUF files that add a low-rank update to matrices of the base model.

The reference hands adapter files to its engine process (``--lora``, llm/llama_server.go) which applies them at run
time.  Here they are merged when the model is loaded: for every base matrix ``W`` [out, in] with a pair
``<name>.lora_a`` [r, in] and ``<name>.lora_b`` [out, r] the weight becomes ``W + (alpha / r) B A``.  A merged matrix is
kept as F16 (a quantised base matrix cannot absorb the update without a second quantisation error), every other tensor
keeps its encoding.  Adapter metadata: ``general.type = adapter``, ``adapter.type = lora``, ``adapter.lora.alpha``.
"""
from __future__ import annotations

from typing import Iterable

import torch

from ..gguf.reader import GGUFFile, open_gguf
from ..gguf.types import GGMLType
from .weights import QWeight, load_tensor


class LoraError(ValueError):
    pass


class LoraAdapter:
    def __init__(self, path: str):
        self.path = path
        self.g: GGUFFile = open_gguf(path)
        kv = self.g.kv
        if kv.get("general.type", "adapter") != "adapter" or kv.get("adapter.type", "lora") != "lora":
            self.g.close()
            raise LoraError(f"{path} is not a LoRA adapter (general.type={kv.get('general.type')!r}, adapter.type={kv.get('adapter.type')!r})")
        self.alpha = float(kv.get("adapter.lora.alpha", 0.0))
        self.pairs: dict[str, tuple[str, str]] = {}
        for name in self.g.tensors:
            if name.endswith(".lora_a"):
                base = name[:-len(".lora_a")]
                if base + ".lora_b" in self.g.tensors:
                    self.pairs[base] = (name, base + ".lora_b")

    def delta(self, base: str, shape: tuple[int, ...]) -> torch.Tensor | None:
        """(alpha / r) B A for ``base`` as fp32 [out, in], or None when the adapter does not touch it."""
        p = self.pairs.get(base)
        if p is None:
            return None
        a = load_tensor(self.g, p[0]).dequant()          # [r, in]
        b = load_tensor(self.g, p[1]).dequant()          # [out, r]
        if a.dim() != 2 or b.dim() != 2 or a.shape[0] != b.shape[1] or (b.shape[0], a.shape[1]) != tuple(shape):
            raise LoraError(f"{base}: adapter shapes {tuple(b.shape)} x {tuple(a.shape)} do not fit the base matrix {tuple(shape)}")
        r = a.shape[0]
        scale = self.alpha / r if self.alpha else 1.0
        return (b @ a) * scale

    def close(self) -> None:
        self.g.close()


def merge(w: QWeight, adapters: Iterable[LoraAdapter]) -> QWeight:
    """``w`` with the updates of every adapter that names it (F16), or ``w`` itself when none does."""
    total = None
    for ad in adapters:
        d = ad.delta(w.name, w.shape) if len(w.shape) == 2 else None
        if d is not None:
            total = d if total is None else total + d
    if total is None:
        return w
    return QWeight.from_float(w.name, w.dequant() + total, GGMLType.F16)


class LoraTensors:
    """name -> QWeight over an opened base GGUF with adapters merged in on access (the tensor source of the engines)."""

    def __init__(self, g: GGUFFile, adapter_paths: Iterable[str]):
        self.g = g
        self.adapters = [LoraAdapter(p) for p in adapter_paths]
        touched = {b for ad in self.adapters for b in ad.pairs}
        unknown = sorted(b for b in touched if not g.has(b))
        if unknown:
            self.close()
            raise LoraError(f"adapter names tensors the base model does not have: {', '.join(unknown[:4])}")
        self.touched = touched

    def __contains__(self, name: str) -> bool:
        return self.g.has(name)

    def keys(self):
        return self.g.tensors.keys()

    def type_of(self, name: str):
        return GGMLType.F16 if name in self.touched and len(self.g.tensors[name].torch_shape) == 2 else self.g.tensors[name].dtype

    def __getitem__(self, name: str) -> QWeight:
        w = load_tensor(self.g, name)
        return merge(w, self.adapters) if name in self.touched else w

    def close(self) -> None:
        for ad in self.adapters:
            ad.close()
