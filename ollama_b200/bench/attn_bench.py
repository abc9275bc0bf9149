"""Timing of the two prefill-attention kernels on Llama-3.1-8B / 70B head shapes.

    python -m ollama_b200.bench.attn_bench [--chunk 2048] [--ctx 2048,6144] [--heads 32:8] [--hd 128] [--reps 5]

A chunk of ``--chunk`` query tokens that ends at position ``ctx`` attends causally to the f16 cache rows [0, ctx).  Each
timed launch uses another slot of the cache (the slots together are larger than the 126 MB L2 for the longer contexts).
Launches are recorded in a CUDA graph and timed with CUDA events after warm-up; reported are microseconds and the FLOP rate counted on the causal
part only (4 * head size FLOP per visible query-key pair), as a fraction of the measured cuBLAS bf16 peak in
MEASURED_PEAKS.json (fallback 1590 TFLOP/s).  ``tc`` = tcgen05 kernel (``tc-ptmem``: its variant that keeps the probabilities in TMEM, ``tc-pipe``: the pipelined kernel), ``mma`` = mma.sync kernel.
"""
from __future__ import annotations

import argparse
import json
import math

import torch

from ..ops import cuda as K
from .gemm_bench import peak_tflops


def visible_pairs(chunk: int, ctx: int) -> int:
    pos0 = ctx - chunk
    return sum(min(pos0 + i + 1, ctx) for i in range(chunk))


def time_mode(mode: str, q, kc, vc, pos0: int, ctx: int, scale: float, reps: int) -> float:
    """Median microseconds per launch: ``reps`` launches (one cache slot after the other) recorded in a CUDA graph, so that no
    host work sits between the two events."""
    slots = kc.shape[0]
    for i in range(3):
        K.attn_prefill(q, kc, vc, i % slots, pos0, ctx, scale, True, mode=mode)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(reps):
            K.attn_prefill(q, kc, vc, i % slots, pos0, ctx, scale, True, mode=mode)
    g.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(5):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b) * 1e3 / reps)
    return sorted(ts)[len(ts) // 2]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--chunk", type=int, default=2048)
    ap.add_argument("--ctx", default="2048,6144")
    ap.add_argument("--heads", default="32:8")
    ap.add_argument("--hd", type=int, default=128)
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--slots", type=int, default=4)
    args = ap.parse_args()
    H, Hkv = (int(x) for x in args.heads.split(":"))
    peak, src = peak_tflops()
    g = torch.Generator(device="cuda").manual_seed(0)
    rows = []
    for ctx in (int(x) for x in args.ctx.split(",")):
        chunk = min(args.chunk, ctx)
        kc = (torch.randn(args.slots, Hkv, ctx, args.hd, device="cuda", generator=g) * 0.5).to(torch.float16)
        vc = (torch.randn(args.slots, Hkv, ctx, args.hd, device="cuda", generator=g) * 0.5).to(torch.float16)
        q = torch.randn(chunk, H, args.hd, device="cuda", generator=g)
        flop = 4.0 * args.hd * H * visible_pairs(chunk, ctx)
        outs = {}
        for name in ("mma", "tc", "tc-ptmem", "tc-pipe"):
            mode = name.split("-")[0]
            K.attn_prefill_tc_variant({"tc-ptmem": 1, "tc-pipe": 2}.get(name, 0))
            us = time_mode(mode, q, kc, vc, ctx - chunk, ctx, 1 / math.sqrt(args.hd), args.reps)
            outs[name] = K.attn_prefill(q, kc, vc, 0, ctx - chunk, ctx, 1 / math.sqrt(args.hd), True, mode=mode).float()
            K.attn_prefill_tc_variant(2)
            rows.append({"kernel": name, "chunk": chunk, "ctx": ctx, "heads": args.heads, "hd": args.hd, "us": round(us, 1),
                         "tflops": round(flop / us / 1e6, 1), f"of_{src}_bf16_peak": round(flop / us / 1e6 / peak, 3)})
            if name != "mma":
                rows[-1]["max_abs_diff_vs_mma"] = float((outs[name] - outs["mma"]).abs().max())
                rows[-1]["wait_status"] = K.attn_prefill_tc_status()
    for r in rows:
        print(json.dumps(r))


if __name__ == "__main__":
    main()
