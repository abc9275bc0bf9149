"""Host-side messaging between the ranks of a tensor-parallel group.

Only three things ever travel on the host: the IPC handles of the peer-mapped regions (an all-gather at buffer
allocation), barriers around allocation and teardown, and the leader's call records.  Two carriers provide them:

* :class:`DistTransport` — a ``torch.distributed`` group (NCCL for the collectives, a gloo group for the CPU
  records); used when the ranks were started together by ``torch.distributed.run`` (benchmarks, self-test).
* :class:`PipeTransport` — ``multiprocessing`` pipes between a leader process and the followers it spawned; used by
  the server, which may hold several models (several groups) in one process and therefore cannot be a member of
  one global process group.
"""
from __future__ import annotations

from typing import Any


class DistTransport:
    def __init__(self, rank: int, world: int, group=None):
        self.rank, self.world, self.group = rank, world, group
        self._gloo = None

    def all_gather(self, obj: Any) -> list[Any]:
        import torch.distributed as dist
        out: list[Any] = [None] * self.world
        dist.all_gather_object(out, obj, group=self.group)
        return out

    def barrier(self) -> None:
        import torch.distributed as dist
        dist.barrier(group=self.group)

    def _cpu_group(self):
        import torch.distributed as dist
        if self._gloo is None:
            self._gloo = dist.new_group(backend="gloo")      # collective: every rank creates it at its first record
        return self._gloo

    def bcast_ints(self, ints: list[int] | None, n: int) -> list[int]:
        """Leader: send ``ints`` (length n); followers: receive n ints."""
        import torch
        import torch.distributed as dist
        buf = torch.zeros(n, dtype=torch.int32) if ints is None else torch.as_tensor(ints, dtype=torch.int32)
        dist.broadcast(buf, 0, group=self._cpu_group())
        return buf.tolist()


class TransportError(RuntimeError):
    pass


class PipeTransport:
    """Leader: ``conns`` = one connection per follower (index rank - 1).  Follower: ``conns`` = [connection to the leader].

    Every message is a (tag, payload) pair: "gather" (one rank's share of an all-gather, and the combined list on the way
    back), "ints" (a call record), "ready" / "error" (a follower's load result).  The leader never blocks without a limit:
    a follower that hangs while loading, or dies, ends the wait with a :class:`TransportError` instead of holding the
    scheduler's load lock for ever; a follower's "error" arriving in the middle of an all-gather is raised at once rather
    than being taken for that rank's share.  A follower that finds the pipe closed knows that the leader is gone.
    """

    def __init__(self, rank: int, world: int, conns: list, timeout: float | None = None):
        import os
        self.rank, self.world, self.conns = rank, world, conns
        self.timeout = float(os.environ.get("B200_TP_LOAD_TIMEOUT", "600")) if timeout is None else timeout
        self.ready: set[int] = set()          # leader: followers whose "ready" has been seen (index into conns)

    def _recv(self, i: int, want: str) -> Any:
        c = self.conns[i]
        while True:
            if self.rank == 0 and not c.poll(self.timeout):
                raise TransportError(f"tensor-parallel rank {i + 1} did not answer within {self.timeout:.0f} s")
            try:
                msg = c.recv()
            except (EOFError, OSError) as e:
                raise TransportError("tensor-parallel peer closed the control pipe" if self.rank == 0 else "leader gone") from e
            if not isinstance(msg, tuple) or len(msg) != 2:
                raise TransportError("tensor-parallel control channel out of step")
            tag, payload = msg
            if tag == want:
                return payload
            if tag == "error":
                raise TransportError(f"tensor-parallel follower failed: {payload}")
            if tag == "ready" and self.rank == 0:
                self.ready.add(i)
                continue
            raise TransportError(f"tensor-parallel control channel out of step: got {tag!r}, expected {want!r}")

    def wait_ready(self) -> None:
        """Leader: block (bounded) until every follower has reported that it finished loading."""
        for i in range(len(self.conns)):
            if i not in self.ready:
                self._await_ready(i)

    def _await_ready(self, i: int) -> None:
        c = self.conns[i]
        while i not in self.ready:
            if not c.poll(self.timeout):
                raise TransportError("a tensor-parallel follower did not finish loading in time")
            try:
                tag, payload = c.recv()
            except (EOFError, OSError) as e:
                raise TransportError("a tensor-parallel follower exited while loading") from e
            if tag == "ready":
                self.ready.add(i)
            elif tag == "error":
                raise TransportError(f"tensor-parallel follower failed to load: {payload}")
            else:
                raise TransportError(f"tensor-parallel control channel out of step: got {tag!r} while waiting for a load result")

    def all_gather(self, obj: Any) -> list[Any]:
        if self.rank == 0:
            out = [obj] + [self._recv(i, "gather") for i in range(len(self.conns))]
            for c in self.conns:
                c.send(("gather", out))
            return out
        self.conns[0].send(("gather", obj))
        return self._recv(0, "gather")

    def barrier(self) -> None:
        self.all_gather(None)

    def bcast_ints(self, ints: list[int] | None, n: int) -> list[int]:
        if self.rank == 0:
            for c in self.conns:
                c.send(("ints", ints))
            return list(ints)
        got = self._recv(0, "ints")
        if not isinstance(got, list) or len(got) != n:
            raise TransportError("tensor-parallel control channel out of step")
        return got


class LocalTransport:
    """A group of one: nothing to exchange (single-GPU use of the peer-region plumbing, tests of the bounded waits)."""

    rank, world = 0, 1

    def all_gather(self, obj: Any) -> list[Any]:
        return [obj]

    def barrier(self) -> None:
        pass

    def bcast_ints(self, ints: list[int] | None, n: int) -> list[int]:
        return list(ints or [])
