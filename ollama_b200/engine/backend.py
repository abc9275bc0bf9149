"""Execution backends behind the runner.

``ModelBackend`` is the narrow interface the batching loop drives: allocate a slot-partitioned KV
cache, prefill a chunk for one slot, run one decode step for a batch of slots.  ``TorchBackend`` is the
portable implementation (reference graph, any torch device); the sm_100a engine in
``ollama_b200.engine.b200`` implements the same interface with hand-written kernels.
"""
from __future__ import annotations

from typing import Protocol, Sequence

import torch

from ..gguf.compat import normalise
from ..gguf.reader import GGUFFile, open_gguf
from ..models.config import ModelConfig, config_from_gguf
from ..models.reference import ReferenceModel
from ..models.weights import load_all


class ModelBackend(Protocol):
    cfg: ModelConfig
    n_slots: int
    n_ctx: int

    def alloc(self, n_slots: int, n_ctx: int) -> None: ...
    def prefill(self, slot: int, tokens: Sequence[int], pos0: int, need_logits: bool = True) -> torch.Tensor | None: ...
    def decode(self, slots: Sequence[int], tokens: Sequence[int], positions: Sequence[int]) -> torch.Tensor: ...
    def hidden(self, slot: int, tokens: Sequence[int]) -> torch.Tensor: ...
    def weight_bytes(self) -> int: ...
    def kv_bytes(self) -> int: ...
    def close(self) -> None: ...


class TorchBackend:
    """Reference execution: fp32 torch ops over weights dequantised from the GGUF."""

    name = "torch"
    supports_verify = True

    def __init__(self, g: GGUFFile, device: str = "cpu", adapters: Sequence[str] = ()):
        self.cfg = config_from_gguf(g)
        self.device = device
        self.weights = load_all(g, "cpu")
        if adapters:                 # LoRA adapters are merged into the matrices they name (models/lora.py)
            from ..models.lora import LoraTensors
            src = LoraTensors(g, adapters)
            try:
                for name in src.touched:
                    self.weights[name] = src[name]
            finally:
                src.close()
        self.model = ReferenceModel(self.cfg, self.weights, device)
        self.cache = None
        self.n_slots = self.n_ctx = 0

    def alloc(self, n_slots: int, n_ctx: int) -> None:
        self.n_slots, self.n_ctx = n_slots, n_ctx
        self.cache = self.model.new_cache(n_slots, n_ctx)

    supports_embeds = True

    @torch.no_grad()
    def prefill(self, slot, tokens, pos0, need_logits=True, embeds=None, spans=()):
        """``embeds`` = (rows of the chunk, [n, d_model] values) replaces the input embedding of those rows (image positions);
        ``spans``: position ranges that attend to themselves in both directions (each must lie inside one chunk)."""
        t = torch.tensor(list(tokens), dtype=torch.long)
        pos = torch.arange(pos0, pos0 + len(tokens))
        out = self.model.forward(t, pos, self.cache, slot, embeds=embeds, spans=spans)
        return out[0] if need_logits else None

    def copy_rows(self, src: int, dst: int, n: int) -> None:
        """Cache rows [0, n) of slot ``src`` become rows [0, n) of slot ``dst`` (a prompt prefix evaluated for another request)."""
        for k, v in zip(self.cache.k, self.cache.v):
            k[dst, :n] = k[src, :n]
            v[dst, :n] = v[src, :n]

    def shift(self, slot: int, keep: int, discard: int, n: int) -> None:
        """Context shift without re-evaluating the prompt: cache rows [keep, keep + discard) of ``slot`` are dropped, the
        ``n - keep - discard`` rows behind them move down and their keys are re-rotated to the new positions."""
        self.model.shift_cache(self.cache, slot, keep, discard, n)

    def prefill_many(self, segs, need_logits):
        """Chunks of several sequences in one call; the reference graph runs them one after another."""
        return [self.prefill(slot, toks, pos0, need) for (slot, toks, pos0), need in zip(segs, need_logits)]

    @torch.no_grad()
    def decode(self, slots, tokens, positions):
        rows = []
        for s, t, p in zip(slots, tokens, positions):
            rows.append(self.model.forward(torch.tensor([t]), torch.tensor([p]), self.cache, s)[0])
        return torch.stack(rows)

    @torch.no_grad()
    def verify(self, slot, tokens, pos0):
        """Logits of every token of the chunk, [T, vocab]: the target-model pass of speculative decoding."""
        t = torch.tensor(list(tokens), dtype=torch.long)
        pos = torch.arange(pos0, pos0 + len(tokens))
        return self.model.forward(t, pos, self.cache, slot, logit_rows=torch.arange(len(tokens)))

    @torch.no_grad()
    def hidden(self, slot, tokens):
        t = torch.tensor(list(tokens), dtype=torch.long)
        return self.model.forward(t, torch.arange(len(tokens)), self.cache, slot, return_hidden=True)

    def weight_bytes(self) -> int:
        return sum(w.nbytes for w in self.weights.values())

    def kv_bytes(self) -> int:
        return self.cache.nbytes() if self.cache is not None else 0

    def close(self) -> None:
        self.cache = None


def open_model(path: str) -> GGUFFile:
    return normalise(open_gguf(path))


def make_backend(g: GGUFFile, device: str = "auto", adapters: Sequence[str] = (), **kw):
    """Pick the engine: the sm_100a kernels when a CUDA device is present, the torch graph otherwise.
    ``adapters``: LoRA adapter files merged into the weights at load time."""
    if device == "auto":
        device = "cuda" if torch.cuda.is_available() else "cpu"
    if device.startswith("cuda"):
        from .b200 import B200Backend, supports
        if supports(config_from_gguf(g)):
            if adapters:
                from ..models.lora import LoraTensors
                src = LoraTensors(g, adapters)
                try:
                    return B200Backend(g, device=device, tensors=src, **kw)
                finally:
                    src.close()
            return B200Backend(g, device=device, **kw)
        return TorchBackend(g, device, adapters)
    return TorchBackend(g, device, adapters)
