"""Layer pipeline over several GPUs: consecutive blocks of the model live on consecutive devices.

This is the multi-GPU mode of the reference (llama.cpp's layer split, which the reference requests by leaving the
split mode at its default: llm/llama_server.go:641-647; memory is assigned layer by layer in server/sched.go).  Here
it is the fallback for models that the tensor-parallel engine does not take (sandwich-norm families, d_model above
8192, head counts that do not divide): every stage is a :class:`B200Backend` restricted to its layer range, one
process drives all devices, and the residual stream crosses from one device to the next as a peer-to-peer DMA
copy ordered by events on the two streams, so no host synchronisation happens between stages.

Decode runs one CUDA graph per stage and step.  Prefill chunks are enqueued stage after stage without waiting for
their results, so stage ``s`` works on chunk ``i`` while stage ``s - 1`` already works on chunk ``i + 1``.
"""
from __future__ import annotations

from typing import Sequence

import torch

from ..gguf.reader import GGUFFile
from ..ops import reference as R
from ..models.config import ModelConfig, config_from_gguf
from .b200 import MAX_DECODE_BATCH, B200Backend, supports


def split_layers(n_layers: int, n_stages: int, weights: Sequence[float] | None = None) -> list[tuple[int, int]]:
    """Contiguous layer ranges, one per stage.  ``weights`` (free memory per device, any unit) skews the split the way
    the reference assigns more layers to devices with more free memory; the last stage also holds the output matrix,
    so with equal weights the remainder goes to the earlier stages."""
    if n_stages < 1 or n_layers < n_stages:
        raise ValueError(f"cannot split {n_layers} layers over {n_stages} devices")
    w = [1.0] * n_stages if weights is None else [max(float(x), 0.0) for x in weights]
    if len(w) != n_stages or sum(w) <= 0:
        raise ValueError("one positive weight per stage is needed")
    total = sum(w)
    counts = [max(1, int(n_layers * x / total)) for x in w]
    i = 0
    while sum(counts) < n_layers:           # hand out the remainder front to back
        counts[i % n_stages] += 1
        i += 1
    while sum(counts) > n_layers:           # the minimum of one layer per stage may overshoot: take from the largest
        counts[max(range(n_stages), key=lambda t: counts[t])] -= 1
    out, lo = [], 0
    for n in counts:
        out.append((lo, lo + n))
        lo += n
    return out


class PipelineBackend:
    name = "b200-pp"
    supports_verify = True

    def __init__(self, g: GGUFFile | None, devices: Sequence[int | str], opts=None, cfg: ModelConfig | None = None, tensors=None,
                 stage_weights: Sequence[float] | None = None, **kw):
        self.cfg = cfg if cfg is not None else config_from_gguf(g)
        if not supports(self.cfg):
            raise NotImplementedError(f"{self.cfg.arch} is not supported by the sm_100a engine")
        self.devices = [torch.device(d if isinstance(d, str) else f"cuda:{d}") for d in devices]
        self.ranges = split_layers(self.cfg.n_layers, len(self.devices), stage_weights)
        self.stages: list[B200Backend] = []
        for dev, rng in zip(self.devices, self.ranges):
            with torch.cuda.device(dev):
                src = tensors(dev) if callable(tensors) else tensors        # a factory gives every stage a source on its own device
                self.stages.append(B200Backend(g, device=str(dev), opts=opts, cfg=self.cfg, tensors=src, layers=rng, **kw))
        self.device = self.devices[-1]          # logits and sampled ids live on the last stage
        self.n_slots = self.n_ctx = 0
        self.kv_type = self.stages[0].kv_type

    # -- bookkeeping ------------------------------------------------------------------------------------
    @property
    def kernel_launches(self) -> int:
        return sum(s.kernel_launches for s in self.stages)

    @property
    def h2d_bytes(self) -> int:
        return sum(s.h2d_bytes for s in self.stages)

    @property
    def d2h_bytes(self) -> int:
        return sum(s.d2h_bytes for s in self.stages)

    def weight_bytes(self) -> int:
        return sum(s.weight_bytes() for s in self.stages)

    def kv_bytes(self) -> int:
        return sum(s.kv_bytes() for s in self.stages)

    def alloc(self, n_slots: int, n_ctx: int) -> None:
        self.n_slots, self.n_ctx = n_slots, n_ctx
        for s in self.stages:
            with torch.cuda.device(s.device):
                s.alloc(n_slots, n_ctx)

    def close(self) -> None:
        for s in self.stages:
            s.close()

    # -- decode -----------------------------------------------------------------------------------------
    def _step(self, slots, tokens, positions, mode, staged: bool = False) -> int:
        """One decode step through every stage; the hand-over of the residual stream is a device-to-device copy that
        torch orders after the producer's stream and before the consumer's.  ``staged``: the step's inputs are
        already in every stage's buffers."""
        prev = None
        nb = len(slots)
        for s in self.stages:
            with torch.cuda.device(s.device):
                if not staged:
                    s._stage(slots, tokens, positions)
                if prev is not None:
                    s.buf.x[:nb].copy_(prev.buf.x[:nb], non_blocking=True)
                s._run_step(nb, mode if s.last else False)
            prev = s
        return nb

    @torch.no_grad()
    def decode_loop(self, slots: Sequence[int], tokens: Sequence[int], positions: Sequence[int], n_steps: int,
                    first_tokens: torch.Tensor | None = None) -> torch.Tensor:
        """Greedy-decode ``n_steps`` tokens per sequence without a host round trip: the sampled ids travel from the last
        stage back to the first one as a device-to-device copy.  Returns int32 [n_steps, nb] on the last stage's device."""
        if len(slots) > MAX_DECODE_BATCH:
            parts = []
            for i in range(0, len(slots), MAX_DECODE_BATCH):
                j = i + MAX_DECODE_BATCH
                parts.append(self.decode_loop(slots[i:j], tokens[i:j], positions[i:j], n_steps,
                                              None if first_tokens is None else first_tokens[i:j]))
            return torch.cat(parts, 1)
        nb = len(slots)
        first, last = self.stages[0], self.stages[-1]
        for s in self.stages:
            with torch.cuda.device(s.device):
                s._stage(slots, tokens, positions)
        if first_tokens is not None:
            with torch.cuda.device(first.device):
                first.buf.tokens[:nb].copy_(first_tokens.to(torch.int32), non_blocking=True)
        out = torch.empty(n_steps, nb, device=last.device, dtype=torch.int32)
        for i in range(n_steps):
            self._step(slots, tokens, positions, True, staged=True)
            with torch.cuda.device(last.device):
                out[i].copy_(last.buf.sampled[:nb])
            with torch.cuda.device(first.device):
                first.buf.tokens[:nb].copy_(last.buf.sampled[:nb], non_blocking=True)
            for s in self.stages:
                with torch.cuda.device(s.device):
                    s.buf.positions[:nb] += 1
        return out

    @torch.no_grad()
    def decode(self, slots: Sequence[int], tokens: Sequence[int], positions: Sequence[int]) -> torch.Tensor:
        if len(slots) > MAX_DECODE_BATCH:
            return torch.cat([self.decode(slots[i:i + MAX_DECODE_BATCH], tokens[i:i + MAX_DECODE_BATCH], positions[i:i + MAX_DECODE_BATCH])
                              for i in range(0, len(slots), MAX_DECODE_BATCH)])
        nb = self._step(slots, tokens, positions, False)
        last = self.stages[-1]
        with torch.cuda.device(last.device):
            return R.softcap(last.buf.logits[:nb].clone(), self.cfg.final_softcap)

    @torch.no_grad()
    def decode_argmax(self, slots: Sequence[int], tokens: Sequence[int], positions: Sequence[int]) -> list[int]:
        if len(slots) > MAX_DECODE_BATCH:
            out: list[int] = []
            for i in range(0, len(slots), MAX_DECODE_BATCH):
                j = i + MAX_DECODE_BATCH
                out += self.decode_argmax(slots[i:j], tokens[i:j], positions[i:j])
            return out
        nb = self._step(slots, tokens, positions, True)
        last = self.stages[-1]
        with torch.cuda.device(last.device):
            last.buf.host_out.copy_(last.buf.sampled, non_blocking=True)
            last.d2h_bytes += last.buf.host_out.numel() * 4
            torch.cuda.current_stream().synchronize()
        return last.buf.host_out_np[:nb].tolist()

    # -- prefill ----------------------------------------------------------------------------------------
    def _chunk(self, slot: int, tokens: Sequence[int], pos0: int) -> torch.Tensor:
        x = None
        for s in self.stages:
            with torch.cuda.device(s.device):
                if x is not None:
                    x = x.to(s.device, non_blocking=True)
                x = s._forward_chunk(slot, tokens, pos0, x=x)
        return x

    @torch.no_grad()
    def prefill(self, slot: int, tokens: Sequence[int], pos0: int, need_logits: bool = True):
        x = self._chunk(slot, tokens, pos0)
        if not need_logits:
            return None
        last = self.stages[-1]
        with torch.cuda.device(last.device):
            h = R.rmsnorm(x[-1:], last.out_norm, self.cfg.norm_eps).to(torch.bfloat16)
            return R.softcap(last._mm(h, last.head)[0], self.cfg.final_softcap)

    @torch.no_grad()
    def verify(self, slot: int, tokens: Sequence[int], pos0: int) -> torch.Tensor:
        x = self._chunk(slot, tokens, pos0)
        last = self.stages[-1]
        with torch.cuda.device(last.device):
            h = R.rmsnorm(x, last.out_norm, self.cfg.norm_eps).to(torch.bfloat16)
            return R.softcap(last._mm(h, last.head), self.cfg.final_softcap)

    @torch.no_grad()
    def hidden(self, slot: int, tokens: Sequence[int]) -> torch.Tensor:
        x = self._chunk(slot, tokens, 0)
        last = self.stages[-1]
        with torch.cuda.device(last.device):
            return R.rmsnorm(x, last.out_norm, self.cfg.norm_eps)
