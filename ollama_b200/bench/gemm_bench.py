"""Timing of the prefill tensor-core GEMM on Llama-8B/70B-shaped operands.

    python -m ollama_b200.bench.gemm_bench [--m 512,2048] [--reps 10] [--only qkv]

out[m, n] = x[m, k] @ w[n, k]^T with bf16 operands.  Each timed launch uses a different copy of the
weights (copies add up to more than the 126 MB L2).  Launches are recorded in a CUDA graph and timed
with CUDA events; reported are microseconds, TFLOP/s and the fraction of the measured cuBLAS bf16 peak
in MEASURED_PEAKS.json (fallback 1590 TFLOP/s), plus the same shape through torch.matmul for reference.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from ..gguf.types import GGMLType
from ..ops import cuda as K
from .kernel_bench import random_weight

SHAPES = [("qkv-8b", 6144, 4096), ("o-8b", 4096, 4096), ("gate_up-8b", 28672, 4096), ("down-8b", 4096, 14336),
          ("gate_up-70b", 57344, 8192), ("down-70b", 8192, 28672)]


def peak_tflops() -> tuple[float, str]:
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["bf16_tflops"]), "measured"
    except (OSError, KeyError, ValueError):
        return 1590.0, "fallback"


def time_graph(fn, reps: int) -> float:
    for i in range(2):
        fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(reps):
            fn(i)
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
    ap.add_argument("--m", default="512,2048")
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--only", default="")
    args = ap.parse_args()
    peak, how = peak_tflops()
    for name, n, k in SHAPES:
        if args.only and args.only not in name:
            continue
        copies = max(2, int(300e6 // (n * k * 2)) + 1)
        ws = [(torch.randn(n, k, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(copies)]
        q0 = random_weight(n, k, GGMLType.Q4_K, 1)
        qcopies = max(2, int(300e6 // q0.nbytes) + 1)
        qs = [q0] + [K.DevWeight(q0.wtype, q0.n, q0.k, [p.clone() for p in q0.planes]) for _ in range(qcopies - 1)]
        for m in [int(x) for x in args.m.split(",")]:
            x = (torch.randn(m, k, device="cuda")).to(torch.bfloat16)
            out = torch.empty(m, n, device="cuda", dtype=torch.float32)
            out2 = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
            t_ours = time_graph(lambda i: K.gemm_bf16(x, ws[i % copies], None, out=out), args.reps)
            t_lib = time_graph(lambda i: torch.matmul(x, ws[i % copies].t(), out=out2), args.reps)
            t_q = time_graph(lambda i: K.gemm_q(x, qs[i % qcopies], out=out), args.reps)
            fl = 2.0 * m * n * k
            print(f"{name:12s} m={m:5d}  ours {t_ours:8.1f} us {fl / t_ours / 1e6:7.1f} TFLOP/s ({fl / t_ours / 1e6 / peak:4.2f} of {how} {peak:.0f})"
                  f"   q4_k fused {t_q:8.1f} us {fl / t_q / 1e6:7.1f} TFLOP/s ({fl / t_q / 1e6 / peak:4.2f})"
                  f"   torch.matmul {t_lib:8.1f} us {fl / t_lib / 1e6:7.1f} TFLOP/s", flush=True)
        del ws, qs
        torch.cuda.empty_cache()
    assert K.gemm_status() == 0


if __name__ == "__main__":
    main()
