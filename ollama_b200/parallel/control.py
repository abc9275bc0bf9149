"""Leader / follower control of a tensor-parallel group.

The serving stack (scheduler, runner, HTTP) lives in rank 0 only.  Every call rank 0 makes on its
tensor-parallel backend is first announced to the other ranks over a host-side channel (a gloo broadcast of a
small int32 record), and each follower repeats the call on its own shard; the device-side exchanges then
meet inside the kernels.  Followers never see requests, samplers or tokenizers: what they need is the call
and its integer arguments.

A decode step fits in one fixed-size record (one broadcast); a prefill sends the record and then the token
ids.  The record also carries a sequence number so that a follower that lost a message fails loudly instead
of running a different step than its peers.

In the reference every GPU of a model is driven by one process (the runner owns all devices of its model:
llm/server.go), so there is no counterpart of this channel there.
"""
from __future__ import annotations

from typing import Sequence

import torch
import torch.distributed as dist

OP_ALLOC, OP_PREFILL, OP_DECODE, OP_DECODE_ARGMAX, OP_DECODE_LOOP, OP_HIDDEN, OP_CLOSE, OP_SET = range(8)
REC = 40          # int32 words per record: [op, seq, a, b, c, d, n, payload[32] ...]
_HDR = 8


class TPControl:
    def __init__(self, rank: int, world: int, group=None):
        """``group`` must be a gloo group spanning the tensor-parallel ranks (created on every rank in the same order)."""
        self.rank, self.world = rank, world
        self.group = group if group is not None else dist.new_group(backend="gloo")
        self.seq = 0
        self.src = dist.get_global_rank(self.group, 0) if hasattr(dist, "get_global_rank") else 0

    # -- leader -------------------------------------------------------------------------------------
    def send(self, op: int, a: int = 0, b: int = 0, c: int = 0, d: int = 0, payload: Sequence[int] = ()) -> None:
        self.seq += 1
        rec = torch.zeros(REC, dtype=torch.int32)
        n = len(payload)
        rec[0], rec[1], rec[2], rec[3], rec[4], rec[5], rec[6] = op, self.seq & 0x7FFFFFFF, a, b, c, d, n
        inline = n <= REC - _HDR
        if inline and n:
            rec[_HDR:_HDR + n] = torch.as_tensor(list(payload), dtype=torch.int32)
        dist.broadcast(rec, self.src, group=self.group)
        if not inline:
            dist.broadcast(torch.as_tensor(list(payload), dtype=torch.int32), self.src, group=self.group)

    # -- follower -----------------------------------------------------------------------------------
    def recv(self) -> tuple[int, int, int, int, int, list[int]]:
        rec = torch.zeros(REC, dtype=torch.int32)
        dist.broadcast(rec, self.src, group=self.group)
        op, seq, a, b, c, d, n = rec[:7].tolist()
        self.seq += 1
        if seq != self.seq & 0x7FFFFFFF:
            raise RuntimeError(f"tensor-parallel control channel out of step: got record {seq}, expected {self.seq}")
        if n <= REC - _HDR:
            payload = rec[_HDR:_HDR + n].tolist()
        else:
            buf = torch.zeros(n, dtype=torch.int32)
            dist.broadcast(buf, self.src, group=self.group)
            payload = buf.tolist()
        return op, a, b, c, d, payload


class TPLeader:
    """Rank 0's view of the group: the backend interface of the runner, with every call announced first."""

    def __init__(self, backend, ctl: TPControl):
        self.be, self.ctl = backend, ctl
        self.name = backend.name

    def __getattr__(self, item):           # cfg, counters, n_slots ... come from the local shard
        return getattr(self.be, item)

    def set_flags(self, use_graphs: bool, pdl: bool) -> None:
        self.ctl.send(OP_SET, int(use_graphs), int(pdl))
        self.be.use_graphs, self.be.pdl = use_graphs, pdl

    def alloc(self, n_slots: int, n_ctx: int) -> None:
        self.ctl.send(OP_ALLOC, n_slots, n_ctx)
        self.be.alloc(n_slots, n_ctx)

    def prefill(self, slot, tokens, pos0, need_logits=True):
        self.ctl.send(OP_PREFILL, slot, pos0, int(need_logits), payload=tokens)
        return self.be.prefill(slot, tokens, pos0, need_logits)

    def hidden(self, slot, tokens):
        self.ctl.send(OP_HIDDEN, slot, payload=tokens)
        return self.be.hidden(slot, tokens)

    def decode(self, slots, tokens, positions):
        self.ctl.send(OP_DECODE, len(slots), payload=list(slots) + list(tokens) + list(positions))
        return self.be.decode(slots, tokens, positions)

    def decode_argmax(self, slots, tokens, positions):
        self.ctl.send(OP_DECODE_ARGMAX, len(slots), payload=list(slots) + list(tokens) + list(positions))
        return self.be.decode_argmax(slots, tokens, positions)

    def decode_loop(self, slots, tokens, positions, n_steps, first_tokens=None):
        if first_tokens is not None:       # followers have the same logits, hence the same first tokens, on their own device
            tokens = [int(t) for t in first_tokens.tolist()]
        self.ctl.send(OP_DECODE_LOOP, len(slots), n_steps, payload=list(slots) + list(tokens) + list(positions))
        return self.be.decode_loop(slots, tokens, positions, n_steps)

    def close(self) -> None:
        self.ctl.send(OP_CLOSE)
        self.be.close()


def follow(backend, ctl: TPControl) -> None:
    """Follower loop of ranks 1..N-1: repeat the leader's calls until it closes the group."""
    while True:
        op, a, b, c, d, p = ctl.recv()
        if op == OP_CLOSE:
            backend.close()
            return
        if op == OP_SET:
            backend.use_graphs, backend.pdl = bool(a), bool(b)
        elif op == OP_ALLOC:
            backend.alloc(a, b)
        elif op == OP_PREFILL:
            backend.prefill(a, p, b, bool(c))
        elif op == OP_HIDDEN:
            backend.hidden(a, p)
        elif op in (OP_DECODE, OP_DECODE_ARGMAX, OP_DECODE_LOOP):
            n = a
            slots, tokens, positions = p[:n], p[n:2 * n], p[2 * n:3 * n]
            if op == OP_DECODE:
                backend.decode(slots, tokens, positions)
            elif op == OP_DECODE_ARGMAX:
                backend.decode_argmax(slots, tokens, positions)
            else:
                backend.decode_loop(slots, tokens, positions, b)
        else:
            raise RuntimeError(f"unknown tensor-parallel control record {op}")
