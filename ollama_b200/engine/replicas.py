"""Data-parallel replicas of one model: several runners with the same weights on different GPUs behind one runner interface.

The reference serves a model from one runner and scales a node by splitting layers; throughput-bound deployments of a model
that fits one GPU are better served by whole copies, each with its own slots, K/V cache and decode loop, and no traffic
between them.  ``B200_REPLICAS=N`` makes the scheduler's runner a :class:`ReplicaSet` of N runners, one per GPU of the
placement (or per group of GPUs when the model is also split).  A request goes to the replica with the fewest requests in
flight; among equals to the one that served the longest shared token prefix last time (its slot cache can reuse it), then
round-robin.  Everything that does not depend on the device (tokenizer, context length) is answered by the first replica.
"""
from __future__ import annotations

import threading
from typing import Any, Callable, Iterator, Sequence


class ReplicaSet:
    def __init__(self, make: Callable[[int], Any], n: int):
        """``make(i)`` builds replica i; a failure closes the replicas already built and is raised."""
        self.replicas: list[Any] = []
        try:
            for i in range(n):
                self.replicas.append(make(i))
        except BaseException:
            self.close()
            raise
        self.lock = threading.Lock()
        self.inflight = [0] * n
        self.last_prompt: list[Sequence[int]] = [()] * n
        self.turn = 0
        self.served = [0] * n

    # -- device-independent state: the first replica answers ------------------------------------------
    def __getattr__(self, name: str) -> Any:
        if name in ("replicas", "lock"):
            raise AttributeError(name)
        return getattr(self.replicas[0], name)

    def tokenize(self, *a, **kw):
        return self.replicas[0].tokenize(*a, **kw)

    def detokenize(self, *a, **kw):
        return self.replicas[0].detokenize(*a, **kw)

    # -- dispatch ---------------------------------------------------------------------------------------
    @staticmethod
    def _shared(a: Sequence[int], b: Sequence[int]) -> int:
        n = 0
        for x, y in zip(a, b):
            if x != y:
                break
            n += 1
        return n

    def _pick(self, prompt: Sequence[int]) -> int:
        with self.lock:
            least = min(self.inflight)
            cands = [i for i, c in enumerate(self.inflight) if c == least]
            best = max(cands, key=lambda i: (self._shared(prompt, self.last_prompt[i]), -((i - self.turn) % len(self.replicas))))
            if self._shared(prompt, self.last_prompt[best]) == 0:
                best = min(cands, key=lambda i: (i - self.turn) % len(self.replicas))
                self.turn = (best + 1) % len(self.replicas)
            self.inflight[best] += 1
            self.served[best] += 1
            self.last_prompt[best] = tuple(prompt[:4096])
            return best

    def _done(self, i: int) -> None:
        with self.lock:
            self.inflight[i] -= 1

    def completion(self, req: Any) -> Iterator[Any]:
        prompt = getattr(req, "prompt", None)
        i = self._pick(prompt if isinstance(prompt, (list, tuple)) else ())
        try:
            yield from self.replicas[i].completion(req)
        finally:
            self._done(i)

    def embedding(self, text):
        i = self._pick(())
        try:
            return self.replicas[i].embedding(text)
        finally:
            self._done(i)

    # -- aggregate state --------------------------------------------------------------------------------
    def ping(self) -> bool:
        return all(r.ping() for r in self.replicas)

    def memory(self) -> dict:
        out: dict[str, int] = {}
        for r in self.replicas:
            for k, v in r.memory().items():
                out[k] = out.get(k, 0) + v
        return out

    @property
    def stats(self) -> dict[str, float]:
        out: dict[str, float] = {}
        for r in self.replicas:
            for k, v in (getattr(r, "stats", None) or {}).items():
                out[k] = out.get(k, 0) + v
        out["replicas"] = len(self.replicas)
        return out

    def close(self) -> None:
        errs = []
        for r in self.replicas:
            try:
                r.close()
            except Exception as e:          # close the others all the same
                errs.append(e)
        if errs:
            raise errs[0]
