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


class PipeTransport:
    """Leader: ``conns`` = one connection per follower (index rank - 1).  Follower: ``conns`` = [connection to the leader]."""

    def __init__(self, rank: int, world: int, conns: list):
        self.rank, self.world, self.conns = rank, world, conns

    def all_gather(self, obj: Any) -> list[Any]:
        if self.rank == 0:
            out = [obj] + [c.recv() for c in self.conns]
            for c in self.conns:
                c.send(out)
            return out
        self.conns[0].send(obj)
        return self.conns[0].recv()

    def barrier(self) -> None:
        self.all_gather(None)

    def bcast_ints(self, ints: list[int] | None, n: int) -> list[int]:
        if self.rank == 0:
            for c in self.conns:
                c.send(ints)
            return list(ints)
        got = self.conns[0].recv()
        if not isinstance(got, list) or len(got) != n:
            raise RuntimeError("tensor-parallel control channel out of step")
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
