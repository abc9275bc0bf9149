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


def prefill_exchanges(tp, L, T: int, dev: str, reps: int = 10) -> dict:
    """Times of the prefill kernels that carry a collective, on the model's own shapes, with their rooflines.

    gemm_rs: attention-output GEMM whose epilogue stores every partial row into its owner (GEMM + reduce-scatter);
    target = max(FLOPs / measured bf16 peak, remote bytes / 770 GB/s).  gemm_local: the same product into local memory.
    norm_ag: sum of the partial rows + residual + RMSNorm + bf16 rows to every rank (reduction + all-gather);
    target = bytes sent per rank / 770 GB/s.
    """
    from ..ops import cuda as K
    from .gemm_bench import peak_tflops
    c, N = tp.cfg, tp.world
    rpr = (T + N - 1) // N
    row0 = min(tp.rank * rpr, T)
    rows = min(rpr, T - row0)
    x = (torch.randn(T, L.wo.k, device=dev) * 0.1).to(torch.bfloat16)
    wb = getattr(L.wo, "bf16", None)
    if wb is None:
        wb = K.dequant_to_bf16(L.wo)
    local = torch.empty(T, c.d_model, device=dev, dtype=torch.float32)

    def timed(fn) -> float:
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) * 1e3 / reps], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    def rs():          # one exchange = scatter GEMM, then the consumer that waits for every rank's rows
        K.gemm_bf16_scatter(x, wb, c.d_model, tp.cm_rs, rpr, None)
        tp._norm_gather(L.ffn_norm, rows, row0, reduce=True)

    tp.region.barrier(4)
    t_pair = timed(rs)
    t_ag = timed(lambda: tp._norm_gather(L.ffn_norm, rows, row0, reduce=False))
    t_local = timed(lambda: K.gemm_bf16(x, wb, None, out=local))
    peak, _ = peak_tflops()
    flops = 2.0 * T * c.d_model * L.wo.k
    remote = (T - rows) * c.d_model * 2          # partial rows travel as bf16
    target_rs = max(flops / (peak * 1e6), remote / 770e3)                     # us
    target_ag = rows * c.d_model * 2 * (N - 1) / 770e3
    t_rs = t_pair - t_ag
    return {"tokens": T, "gemm_local_us": round(t_local, 1), "gemm_rs_plus_reduce_us": round(t_pair, 1), "norm_ag_us": round(t_ag, 1),
            "gemm_rs_us_est": round(t_rs, 1), "gemm_rs_target_us": round(target_rs, 1), "gemm_rs_frac_of_roofline": round(target_rs / max(t_rs, 1e-3), 2),
            "norm_ag_target_us": round(target_ag, 1), "norm_ag_frac_of_roofline": round(target_ag / max(t_ag, 1e-3), 2)}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--pairs", type=int, default=200)
    ap.add_argument("--nb", type=int, default=1)
    ap.add_argument("--model", default="tiny-tp")
    ap.add_argument("--quant", default="Q8_0")
    ap.add_argument("--layers", type=int, default=0, help="truncate the model to this many layers (shapes are what matters here)")
    ap.add_argument("--tokens", type=int, default=0, help="also time the prefill exchanges on a chunk of this many tokens")
    args = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    dist.init_process_group("nccl", device_id=torch.device(dev))
    from ..models.config import config_from_gguf
    from ..models.synth import SyntheticTensors, synthetic_header
    from ..parallel.tp_engine import TPBackend

    if args.layers:
        import dataclasses

        from ..models import synth
        synth.SPECS[args.model] = dataclasses.replace(synth.SPECS[args.model], n_layers=args.layers)
    cfg = config_from_gguf(synthetic_header(args.model, args.quant))
    tp = TPBackend(cfg, SyntheticTensors(args.model, args.quant, seed=0, device=dev), device=dev, rank=rank, world=world,
                   max_chunk=max(args.tokens, 512))
    tp.alloc(1, max(512, args.tokens))
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
    if args.tokens:
        out.update(prefill_exchanges(tp, L, args.tokens, dev))
    out.update(world=world, pairs=args.pairs, nb=nb, d_model=c.d_model, comm_status=tp.comm_status())
    if rank == 0:
        print(json.dumps(out), flush=True)
    tp.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
