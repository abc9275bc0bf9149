"""Peer-mapped memory and flag channels for the tensor-parallel engine.

Each rank (one process per GPU) allocates one region with ``cudaMalloc``, exports it as a CUDA IPC handle,
and opens every other rank's region; handles travel over the group's host transport (``parallel/transport.py``:
a ``torch.distributed`` group or pipes to spawned followers), which carries this rendezvous, barriers and the
leader's call records and nothing else.  All data of a forward pass moves through
stores to peer addresses issued by the compute kernels themselves (``kernels/comm.cuh``).

The reference stack spreads a model over GPUs by layer / row splits inside ggml's scheduler and exchanges
activations with device-to-device copies (llm/server.go GPU layer assignment; ml/backend/ggml/ggml.go tensor
splits); this module is the sm_100a + NVLink counterpart.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from ..ops import cuda as K

CHAN_BYTES = 128
N_CHANNELS = 8
# CommChan field offsets (kernels/comm.cuh)
_OFF_EPOCH, _OFF_STATUS, _OFF_WAIT_MS, _OFF_FLAGS = 4, 8, 12, 32


class _DevArray:
    """Minimal ``__cuda_array_interface__`` carrier so torch can wrap raw device memory without copying."""

    def __init__(self, ptr: int, shape: tuple[int, ...], typestr: str):
        self.__cuda_array_interface__ = {"shape": shape, "typestr": typestr, "data": (ptr, False), "version": 3, "strides": None}


_TYPESTR = {torch.float32: "<f4", torch.int32: "<i4", torch.uint8: "|u1", torch.int8: "|i1", torch.float16: "<f2", torch.int16: "<i2"}


def tensor_at(ptr: int, shape: tuple[int, ...], dtype: torch.dtype, device) -> torch.Tensor:
    """A tensor view of device memory at ``ptr`` (bf16 is viewed through int16)."""
    if dtype == torch.bfloat16:
        return torch.as_tensor(_DevArray(ptr, shape, "<i2"), device=device).view(torch.bfloat16)
    return torch.as_tensor(_DevArray(ptr, shape, _TYPESTR[dtype]), device=device)


@dataclass
class Block:
    offset: int
    nbytes: int


class Layout:
    """Byte offsets of named blocks inside the region (identical on every rank)."""

    def __init__(self):
        self.size = N_CHANNELS * CHAN_BYTES
        self.blocks: dict[str, Block] = {}

    def add(self, name: str, nbytes: int) -> Block:
        off = (self.size + 255) // 256 * 256
        self.blocks[name] = Block(off, nbytes)
        self.size = off + nbytes
        return self.blocks[name]


class PeerRegion:
    """One peer-mapped allocation per rank; ``base[r]`` is rank r's region as seen from this process."""

    def __init__(self, nbytes: int, rank: int, world: int, device, group=None):
        """``group``: a transport (parallel/transport.py), or a torch.distributed group / None for the default group."""
        from .transport import DistTransport
        tr = group if hasattr(group, "all_gather") else DistTransport(rank, world, group)
        self.rank, self.world, self.device, self.nbytes = rank, world, torch.device(device), nbytes
        if world > K.COMM_MAX_RANKS:
            raise ValueError(f"at most {K.COMM_MAX_RANKS} ranks per tensor-parallel group")
        lib = K.lib()
        lib.b2_ipc_alloc.argtypes = [C.c_size_t, C.POINTER(C.c_void_p), C.c_char_p]
        lib.b2_ipc_open.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
        lib.b2_ipc_close.argtypes = [C.c_void_p]
        lib.b2_ipc_free.argtypes = [C.c_void_p]
        p = C.c_void_p()
        handle = C.create_string_buffer(64)
        with torch.cuda.device(self.device):
            K._check(lib.b2_ipc_alloc(nbytes, C.byref(p), handle), "ipc_alloc")
            handles: list = tr.all_gather(handle.raw)
            self.base: list[int] = []
            for r in range(world):
                if r == rank:
                    self.base.append(p.value)
                    continue
                q = C.c_void_p()
                K._check(lib.b2_ipc_open(handles[r], C.byref(q)), f"ipc_open(rank {r})")
                self.base.append(q.value)
        tr.barrier()
        self.transport = tr
        self._open = True

    def chan(self, idx: int, r: int | None = None) -> int:
        return self.base[self.rank if r is None else r] + idx * CHAN_BYTES

    def addr(self, block: Block, r: int | None = None, byte_off: int = 0) -> int:
        return self.base[self.rank if r is None else r] + block.offset + byte_off

    def tensor(self, block: Block, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        return tensor_at(self.addr(block), shape, dtype, self.device)

    def send(self, chan_idx: int, dst: list[int], parity_stride: int = 0) -> "K.CommSend":
        """Producer-side descriptor: ``dst[r]`` is the destination address on rank r (already offset for this rank)."""
        cm = K.CommSend()
        cm.n_dst, cm.rank = self.world, self.rank
        cm.local = self.chan(chan_idx)
        for r in range(self.world):
            cm.peer_flag[r] = self.chan(chan_idx, r) + _OFF_FLAGS + 4 * self.rank
            cm.dst[r] = dst[r] if dst else 0
        cm.parity_stride = parity_stride
        return cm

    def set_wait_ms(self, chan_idx: int, ms: int) -> None:
        tensor_at(self.chan(chan_idx) + _OFF_WAIT_MS, (1,), torch.int32, self.device).fill_(ms)

    def status(self, chan_idx: int) -> int:
        """0 = ok, 1 = a wait on this channel ran out on this rank (synchronises the current stream)."""
        return int(tensor_at(self.chan(chan_idx) + _OFF_STATUS, (1,), torch.int32, self.device).item())

    def failed_channels(self) -> list[int]:
        """Channels whose waits ran out on this rank since the last clear (one device read of the channel block)."""
        words = tensor_at(self.chan(0), (N_CHANNELS, CHAN_BYTES // 4), torch.int32, self.device)[:, _OFF_STATUS // 4].tolist()
        return [i for i, w in enumerate(words) if w != 0]

    def clear_status(self, chan_idx: int) -> None:
        tensor_at(self.chan(chan_idx) + _OFF_STATUS, (1,), torch.int32, self.device).zero_()

    def barrier(self, chan_idx: int) -> None:
        """Device-side barrier on the current stream (all earlier work of every rank has finished when it returns)."""
        cm = self.send(chan_idx, [])
        K.lib().b2_comm_barrier.argtypes = [C.c_void_p, C.c_void_p]
        K._check(K.lib().b2_comm_barrier(C.addressof(cm), K.stream()), "comm_barrier")

    def wait(self, chan_idx: int, pdl: bool = False) -> None:
        f = K.lib().b2_comm_wait
        f.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        K._check(f(self.chan(chan_idx), self.world, int(pdl), K.stream()), "comm_wait")

    def close(self) -> None:
        if not self._open:
            return
        self._open = False
        torch.cuda.synchronize(self.device)
        try:
            self.transport.barrier()      # nobody may still be writing into a region that is about to go away
        except Exception:
            pass
        lib = K.lib()
        for r, b in enumerate(self.base):
            if r != self.rank:
                lib.b2_ipc_close(b)
        lib.b2_ipc_free(self.base[self.rank])
