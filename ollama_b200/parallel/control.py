"""Leader / follower control of a tensor-parallel group.

The serving stack (scheduler, runner, HTTP) lives in rank 0 only.  Every call rank 0 makes on its
tensor-parallel backend is first announced to the other ranks over the group's host transport (a gloo broadcast
or a pipe per follower carrying a small int32 record), and each follower repeats the call on its own shard; the device-side exchanges then
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

OP_ALLOC, OP_PREFILL, OP_DECODE, OP_DECODE_ARGMAX, OP_DECODE_LOOP, OP_HIDDEN, OP_CLOSE, OP_SET = range(8)
REC = 40          # int32 words per record: [op, seq, a, b, c, d, n, payload[32] ...]
_HDR = 8


class TPControl:
    def __init__(self, rank: int, world: int, group=None):
        """``group``: a transport (parallel/transport.py), or a torch.distributed group / None for the default group."""
        from .transport import DistTransport
        self.rank, self.world = rank, world
        self.tr = group if hasattr(group, "bcast_ints") else DistTransport(rank, world, group)
        self.seq = 0

    # -- leader -------------------------------------------------------------------------------------
    def send(self, op: int, a: int = 0, b: int = 0, c: int = 0, d: int = 0, payload: Sequence[int] = ()) -> None:
        self.seq += 1
        payload = [int(v) for v in payload]
        n = len(payload)
        rec = [op, self.seq & 0x7FFFFFFF, a, b, c, d, n, 0] + [0] * (REC - _HDR)
        inline = n <= REC - _HDR
        if inline:
            rec[_HDR:_HDR + n] = payload
        self.tr.bcast_ints(rec, REC)
        if not inline:
            self.tr.bcast_ints(payload, n)

    # -- follower -----------------------------------------------------------------------------------
    def recv(self) -> tuple[int, int, int, int, int, list[int]]:
        rec = self.tr.bcast_ints(None, REC)
        op, seq, a, b, c, d, n = rec[:7]
        self.seq += 1
        if seq != self.seq & 0x7FFFFFFF:
            raise RuntimeError(f"tensor-parallel control channel out of step: got record {seq}, expected {self.seq}")
        payload = rec[_HDR:_HDR + n] if n <= REC - _HDR else self.tr.bcast_ints(None, n)
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
