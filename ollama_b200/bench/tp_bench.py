"""Latency of the tensor-parallel exchanges (run under torch.distributed.run, one rank per GPU).

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 --master-port 29561 \
        -m ollama_b200.bench.tp_bench [--pairs 200] [--nb 1]

Times, with CUDA events around a CUDA graph, a chain of (row-parallel GEMV that stores its partial rows into every
rank's buffer and raises the flags) -> (add + RMSNorm + quantise that waits for all flags) pairs on a small model, and
the same chain on one GPU without the exchange.  The difference is the cost of one all-reduce as the engine performs it.
Rank 0 prints one JSON line; times are the maximum over ranks.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--pairs", type=int, default=200)
    ap.add_argument("--nb", type=int, default=1)
    ap.add_argument("--model", default="tiny-tp")
    args = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    dist.init_process_group("nccl", device_id=torch.device(dev))
    from ..models.config import config_from_gguf
    from ..models.synth import SyntheticTensors, synthetic_header
    from ..parallel.tp_engine import TPBackend

    cfg = config_from_gguf(synthetic_header(args.model, "Q8_0"))
    tp = TPBackend(cfg, SyntheticTensors(args.model, "Q8_0", seed=0, device=dev), device=dev, rank=rank, world=world)
    tp.alloc(1, 512)
    b, c, L, nb = tp.buf, tp.cfg, tp.layers[0], args.nb

    def chain(comm: bool):
        tp._n = 0
        for _ in range(args.pairs):
            if comm:
                tp._gemv_send(L.wo, nb, b.aq, b.ads, b.ao, tp.cm_dec, c.d_model)
                tp._norm_quant_reduce(L.ffn_norm, nb)
            else:
                tp._gemv([L.wo], nb, b.aq, b.ads, b.ao, b.tmp, b.tmp.stride(0))
                tp._norm_quant(b.tmp, L.ffn_norm, nb, c.d_model)

    out = {}
    for name, comm in (("local_us", False), ("exchange_us", True)):
        chain(comm)
        torch.cuda.synchronize()
        dist.barrier()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            chain(comm)
        ts = []
        for _ in range(5):
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3 / args.pairs)
        t = torch.tensor([sorted(ts)[2]], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out[name] = round(t.item(), 2)
        b.x.zero_()
    out.update(world=world, pairs=args.pairs, nb=nb, d_model=c.d_model, comm_status=tp.comm_status())
    if rank == 0:
        print(json.dumps(out), flush=True)
    tp.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
