"""Starting a tensor-parallel group from inside the serving process.

The server (one process, possibly several models) becomes rank 0 of a group of ``world`` ranks: it spawns
``world - 1`` follower processes, one per further GPU, connected by pipes (parallel/transport.py), builds its
own shard of the model and returns a :class:`TPLeader` that the runner drives like any single-GPU backend.
Followers open the same GGUF file (memory-mapped), build their shard and repeat the leader's calls until the
leader closes the group; a follower that dies is noticed by the leader at the next message (broken pipe) and
fails the request instead of hanging the server, while the device-side waits are bounded on their own.

The reference hands all GPUs of a model to one runner process (llm/server.go GPU layer assignment); one process
per GPU is this runtime's execution model.
"""
from __future__ import annotations

import multiprocessing as mp
import os
from typing import Sequence

from ..gguf.reader import GGUFFile
from ..models.config import config_from_gguf
from ..models.weights import QWeight, load_tensor


class GGUFTensors:
    """name -> QWeight mapping over an opened GGUF that reads a tensor when it is asked for."""

    def __init__(self, g: GGUFFile):
        self.g = g

    def __contains__(self, name: str) -> bool:
        return self.g.has(name)

    def keys(self):
        return self.g.tensors.keys()

    def type_of(self, name: str):
        return self.g.tensors[name].dtype

    def __getitem__(self, name: str) -> QWeight:
        return load_tensor(self.g, name)


def _source(g: GGUFFile, adapters):
    """Tensor source of a rank: the GGUF itself, or the GGUF with LoRA adapters merged in."""
    if adapters:
        from ..models.lora import LoraTensors
        return LoraTensors(g, adapters)
    return GGUFTensors(g)


def _follower(model_path: str, rank: int, world: int, device: str, conn, max_chunk: int, kv_type: str = "f16", adapters=()) -> None:
    import torch

    from ..engine.backend import open_model
    from .control import TPControl, follow
    from .tp_engine import TPBackend
    from .transport import PipeTransport
    torch.cuda.set_device(torch.device(device))
    tr = PipeTransport(rank, world, [conn])
    try:
        g = open_model(model_path)
        be = TPBackend(config_from_gguf(g), _source(g, adapters), device=device, rank=rank, world=world, group=tr, max_chunk=max_chunk,
                       kv_type=kv_type)
        conn.send(("ready", rank))
    except Exception as e:      # the leader turns this into a load error
        conn.send(("error", f"rank {rank}: {e}"))
        return
    from .transport import TransportError
    try:
        follow(be, TPControl(rank, world, tr))
    except TransportError:      # the leader closed the pipe or died: nothing left to follow
        be.close()


class TPGroup:
    """Owns the follower processes of one model; ``backend`` is the leader-side backend for the runner."""

    def __init__(self, model_path: str, devices: Sequence[int], max_chunk: int = 2048, kv_type: str = "f16", adapters: Sequence[str] = ()):
        import torch

        from ..engine.backend import open_model
        from .control import TPControl, TPLeader
        from .tp_engine import TPBackend
        from .transport import PipeTransport
        world = len(devices)
        if world < 2:
            raise ValueError("a tensor-parallel group needs at least two devices")
        ctx = mp.get_context("spawn")
        self.procs, conns = [], []
        for r in range(1, world):
            parent, child = ctx.Pipe()
            p = ctx.Process(target=_follower, args=(model_path, r, world, f"cuda:{devices[r]}", child, max_chunk, kv_type, tuple(adapters)), daemon=True)
            p.start()
            child.close()
            self.procs.append(p)
            conns.append(parent)
        self.conns = conns
        dev0 = f"cuda:{devices[0]}"
        try:
            torch.cuda.set_device(torch.device(dev0))
            g = open_model(model_path)
            tr = PipeTransport(0, world, conns)
            be = TPBackend(config_from_gguf(g), _source(g, adapters), device=dev0, rank=0, world=world, group=tr, max_chunk=max_chunk,
                           kv_type=kv_type)
            tr.wait_ready()
        except Exception:
            self.kill()
            raise
        self.backend = TPLeader(be, TPControl(0, world, tr))

    def alive(self) -> bool:
        """Every follower process is still running (the runner's ``ping`` and with it the scheduler's reload check use this,
        the way the reference asks a runner process for its health: server/sched.go needsReload)."""
        return all(p.is_alive() for p in self.procs)

    def close(self) -> None:
        try:
            self.backend.close()
        finally:
            for p in self.procs:
                p.join(timeout=30)
            self.kill()

    def kill(self) -> None:
        for p in self.procs:        # exact processes this object started
            if p.is_alive():
                p.terminate()
        for c in self.conns:
            c.close()
