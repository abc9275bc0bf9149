"""Token sampling.

Chain order: repetition / presence / frequency penalties over the last ``repeat_last_n`` tokens, then
greedy when ``temperature <= 0``; otherwise top-k -> typical-p -> top-p -> min-p -> temperature ->
seeded categorical draw.  This is the subset of samplers the public options expose
(api/types.go:568-585; defaults :1096-1123); the reference's in-tree sampler for its other engine
documents the same steps (x/mlxrunner/sample/sample.go:822-871, penalties ring :884-911, logprobs
:422-441).

All tensor work uses torch ops, so the same code samples from logits that live on the GPU; the CUDA
engine replaces the greedy path by a fused arg-max kernel.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass
class SamplingParams:
    temperature: float = 0.8
    top_k: int = 40
    top_p: float = 0.9
    min_p: float = 0.0
    typical_p: float = 1.0
    repeat_last_n: int = 64
    repeat_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    seed: int = -1
    logprobs: bool = False
    top_logprobs: int = 0

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0

    @property
    def has_penalties(self) -> bool:
        return self.repeat_last_n != 0 and (self.repeat_penalty != 1.0 or self.presence_penalty != 0.0 or self.frequency_penalty != 0.0)


@dataclass
class TokenLogprob:
    token: int
    logprob: float
    top: list[tuple[int, float]] = field(default_factory=list)


class Sampler:
    """Per-request sampler state (history ring and random stream)."""

    def __init__(self, params: SamplingParams, n_vocab: int, n_ctx: int = 0, history: list[int] | None = None, device="cpu"):
        self.p = params
        self.n_vocab = n_vocab
        n = params.repeat_last_n
        if n < 0:
            n = n_ctx or 1 << 30          # -1 means "the whole context"
        self.window = n
        self.history: list[int] = list(history[-n:]) if (history and n > 0) else []
        self.gen = torch.Generator(device="cpu")
        if params.seed is not None and params.seed >= 0:
            self.gen.manual_seed(int(params.seed))
        else:
            self.gen.seed()

    def accept(self, tok: int) -> None:
        if self.window > 0:
            self.history.append(tok)
            if len(self.history) > self.window:
                del self.history[: len(self.history) - self.window]

    def _penalise(self, logits: torch.Tensor) -> torch.Tensor:
        p = self.p
        if not p.has_penalties or not self.history:
            return logits
        ids = torch.tensor(self.history, device=logits.device, dtype=torch.long)
        uniq, counts = torch.unique(ids, return_counts=True)
        uniq = uniq[uniq < logits.shape[-1]]
        counts = counts[: uniq.numel()].to(logits.dtype)
        vals = logits[uniq]
        if p.repeat_penalty != 1.0:
            vals = torch.where(vals <= 0, vals * p.repeat_penalty, vals / p.repeat_penalty)
        vals = vals - counts * p.frequency_penalty - p.presence_penalty
        out = logits.clone()
        out[uniq] = vals
        return out

    def distribution(self, logits: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """Candidate ids and their final probabilities after the whole filter chain."""
        p = self.p
        lg = self._penalise(logits.float())
        k = p.top_k if 0 < p.top_k < lg.numel() else lg.numel()
        vals, idx = torch.topk(lg, k) if k < lg.numel() else torch.sort(lg, descending=True)
        if 0.0 < p.typical_p < 1.0:
            pr = torch.softmax(vals, -1)
            ent = -(pr * torch.log(pr.clamp_min(1e-30))).sum()
            dev = (-torch.log(pr.clamp_min(1e-30)) - ent).abs()
            order = torch.argsort(dev)
            cum = torch.cumsum(pr[order], 0)
            last = int(torch.searchsorted(cum, torch.tensor(p.typical_p, device=cum.device)).item()) + 1
            keep = torch.sort(order[: max(last, 1)]).values
            vals, idx = vals[keep], idx[keep]
        if 0.0 < p.top_p < 1.0:
            pr = torch.softmax(vals, -1)
            cum = torch.cumsum(pr, 0)
            # keep a candidate while the mass of the candidates before it is still below p
            keep = (cum - pr) < p.top_p
            keep[0] = True
            vals, idx = vals[keep], idx[keep]
        if p.min_p > 0.0:
            pr = torch.softmax(vals, -1)
            keep = pr >= p.min_p * pr[0]
            keep[0] = True
            vals, idx = vals[keep], idx[keep]
        probs = torch.softmax(vals / max(p.temperature, 1e-6), -1)
        return idx, probs

    def _on_device(self, logits: torch.Tensor, allowed) -> bool:
        """The sampling kernel covers top-k candidate sets up to 256 without typical-p, grammar or log-probabilities."""
        p = self.p
        return (logits.is_cuda and allowed is None and not p.logprobs and 0 < p.top_k <= 256 and not (0.0 < p.typical_p < 1.0)
                and logits.shape[-1] >= p.top_k)

    def sample(self, logits: torch.Tensor, allowed=None) -> tuple[int, TokenLogprob | None]:
        """Draw one token from ``logits`` ([vocab]).  ``allowed(token) -> bool`` is the grammar filter."""
        p = self.p
        lg = logits
        if p.greedy:
            lg = self._penalise(logits.float())
            tok = int(torch.argmax(lg).item())
            if allowed is not None and not allowed(tok):
                tok = self._constrained(lg, allowed, greedy=True)
        elif self._on_device(logits, allowed):
            # the whole chain in one kernel on the logits where they are; only the sampled id comes back
            from collections import Counter

            from ..ops import cuda as K
            u = float(torch.rand(1, generator=self.gen).item())
            hist = dict(Counter(t for t in self.history if 0 <= t < logits.shape[-1])) if (p.has_penalties and self.history) else {}
            row = logits.reshape(1, -1)
            if row.dtype != torch.float32 or not row.is_contiguous():
                row = row.float().contiguous()
            with torch.cuda.device(row.device):      # a pipelined model keeps its logits on the last stage's GPU
                tok = int(K.sample(row, [u], p.top_k, p.top_p, p.min_p, p.temperature, [hist], p.repeat_penalty, p.frequency_penalty,
                                   p.presence_penalty)[0].item())
        else:
            idx, probs = self.distribution(logits)
            j = int(torch.multinomial(probs.cpu(), 1, generator=self.gen).item())
            tok = int(idx[j].item())
            if allowed is not None and not allowed(tok):
                tok = self._constrained(logits.float(), allowed, greedy=False)
        lp = None
        if p.logprobs:
            ls = torch.log_softmax(logits.float(), -1)
            top = []
            if p.top_logprobs > 0:
                tv, ti = torch.topk(ls, min(p.top_logprobs, ls.numel()))
                top = [(int(i), float(v)) for i, v in zip(ti.tolist(), tv.tolist())]
            lp = TokenLogprob(tok, float(ls[tok].item()), top)
        self.accept(tok)
        return tok, lp

    def _constrained(self, logits: torch.Tensor, allowed, greedy: bool) -> int:
        """Slow path taken only when the unconstrained draw violates the grammar: mask, then redo."""
        order = torch.argsort(logits, descending=True).tolist()
        ok = [t for t in order[:4096] if allowed(t)]
        if not ok:
            ok = [t for t in order[4096:] if allowed(t)]
        if not ok:
            raise RuntimeError("grammar rejects every token")
        if greedy:
            return ok[0]
        masked = torch.full_like(logits, float("-inf"))
        ids = torch.tensor(ok, device=logits.device)
        masked[ids] = logits[ids]
        idx, probs = self.distribution(masked)
        good = torch.isfinite(masked[idx])
        idx, probs = idx[good], probs[good] / probs[good].sum()
        j = int(torch.multinomial(probs.cpu(), 1, generator=self.gen).item())
        return int(idx[j].item())
