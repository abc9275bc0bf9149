"""Per-kernel timing of the decode hot ops on Llama-8B/70B-shaped operands.

    python -m ollama_b200.bench.kernel_bench [--nb 1,4,8] [--only glu] [--reps 20]

Every case is timed with CUDA events on the launching stream after warm-up.  Each timed launch
reads a different copy of the weights (the copies add up to more than the 126 MB L2), so the bytes
really come from HBM.  Reported: microseconds, achieved GB/s over the algorithmic weight bytes and
the fraction of the measured copy bandwidth in MEASURED_PEAKS.json (fallback 6650 GB/s).
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from ..gguf.types import GGMLType
from ..models.weights import QWeight
from ..ops import cuda as K
from ..ops import sk

CASES = [
    # name, kind, [(rows, type)], k
    ("qkv-8b", "gemv", [(4096, GGMLType.Q4_K), (1024, GGMLType.Q4_K), (1024, GGMLType.Q6_K)], 4096),
    ("o-8b", "gemv", [(4096, GGMLType.Q4_K)], 4096),
    ("glu-8b", "glu", [(14336, GGMLType.Q4_K)], 4096),
    ("down-8b-q4k", "gemv", [(4096, GGMLType.Q4_K)], 14336),
    ("down-8b-q6k", "gemv", [(4096, GGMLType.Q6_K)], 14336),
    ("head-8b", "gemv", [(128256, GGMLType.Q6_K)], 4096),
    ("glu-70b", "glu", [(28672, GGMLType.Q4_K)], 8192),
    # per-rank shards of Llama-70B split 2 and 8 ways
    ("qkv-70b-tp2", "gemv", [(4096, GGMLType.Q4_K), (512, GGMLType.Q4_K), (512, GGMLType.Q6_K)], 8192),
    ("o-70b-tp2", "gemv", [(8192, GGMLType.Q4_K)], 4096),
    ("glu-70b-tp2", "glu", [(14336, GGMLType.Q4_K)], 8192),
    ("down-70b-tp2", "gemv", [(8192, GGMLType.Q6_K)], 14336),
    ("qkv-70b-tp8", "gemv", [(1024, GGMLType.Q4_K), (128, GGMLType.Q4_K), (128, GGMLType.Q6_K)], 8192),
    ("o-70b-tp8", "gemv", [(8192, GGMLType.Q4_K)], 1024),
    ("glu-70b-tp8", "glu", [(3584, GGMLType.Q4_K)], 8192),
    ("down-70b-tp8", "gemv", [(8192, GGMLType.Q6_K)], 3584),
    ("o-8b-q8", "gemv", [(4096, GGMLType.Q8_0)], 4096),
    ("o-8b-bf16", "gemv", [(4096, GGMLType.BF16)], 4096),
]


def peak_gbs() -> tuple[float, str]:
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        return 6650.0, "fallback"


def random_weight(n: int, k: int, t: GGMLType, seed: int) -> K.DevWeight:
    """Random valid blocks: quantise a slab of N(0, 0.02) values and tile it (content does not affect timing)."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    rows = min(n, 512)
    w = torch.randn(rows, k, device="cuda", generator=g) * 0.02
    q = QWeight.from_float("w", w, t)
    reps = (n + rows - 1) // rows
    raw = q.raw.view(rows, -1).repeat(reps, 1)[:n].reshape(-1)
    return K.repack(QWeight("w", t, (n, k), raw), "cuda")


def random_qweight(n: int, k: int, t: GGMLType, seed: int) -> QWeight:
    g = torch.Generator(device="cuda").manual_seed(seed)
    rows = min(n, 512)
    w = torch.randn(rows, k, device="cuda", generator=g) * 0.02
    q = QWeight.from_float("w", w, t)
    reps = (n + rows - 1) // rows
    return QWeight("w", t, (n, k), q.raw.view(rows, -1).repeat(reps, 1)[:n].reshape(-1))


def time_graph(run, copies: int, reps: int) -> float:
    """Median microseconds per launch of ``run(i)``, ``reps`` launches recorded into one CUDA graph."""
    for i in range(3):
        run(i % copies)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(reps):
            run(i % copies)
    graph.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(5):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b) * 1e3 / reps)
    ts.sort()
    return ts[len(ts) // 2]


def bench_sk(args, peak: float, how: str) -> None:
    """The streaming tensor-core GEMV (kernels/gemv_sk.cu) on the same shapes; the input is the fp32 row (quantised inside the
    kernel) where it fits into shared memory, otherwise the output of quant256."""
    for name, kind, segs, k in CASES:
        if args.only and args.only not in name:
            continue
        if not all(sk.supported(t, n, k) for n, t in segs):
            continue
        qs = [random_qweight(n, k, t, i) for i, (n, t) in enumerate(segs)]
        if kind == "glu":
            qs = [sk.interleave(qs[0], random_qweight(segs[0][0], k, segs[0][1], 7))]
        one = [sk.repack(q, "cuda") for q in qs]
        del qs
        nbytes = sum(w.nbytes for w in one)
        copies = args.copies or max(2, int(300e6 // nbytes) + 1)
        sets = [one] + [[sk.SkWeight(w.wtype, w.n, w.k, w.units.clone()) for w in one] for _ in range(1, copies)]
        for nb in [int(x) for x in args.nb.split(",")]:
            x = torch.randn(nb, k, device="cuda")
            xin = x if sk.fits_fused_input(nb, k) else sk.quant256(x)
            n_out = sum(w.n for w in one)
            out = torch.zeros(nb, n_out // 2 if kind == "glu" else n_out, device="cuda")
            mode = sk.MODE_GLU if kind == "glu" else sk.MODE_STORE

            def run(i):
                sk.gemv(sets[i], xin, out=out, mode=mode, max_ctas=args.ctas, split=args.split, ring=args.ring, pdl=bool(args.pdl))

            med = time_graph(run, copies, args.reps)
            sk.workspace("cuda").check()
            gbs = nbytes / med / 1e3
            print(f"sk {name:14s} nb={nb:2d}  {med:8.1f} us  {gbs:7.0f} GB/s  {gbs / peak:5.2f} of {how} {peak:.0f} GB/s  "
                  f"({nbytes / 1e6:.1f} MB, {copies} copies, {'fused' if xin is x else 'pre-quantised'} input, ctas={args.ctas} split={args.split} ring={args.ring} pdl={args.pdl})",
                  flush=True)
        del sets
        torch.cuda.empty_cache()


LAYERS = {
    # name: (d_model, q_dim, kv_dim, d_ff, down type)
    "layer-8b": (4096, 4096, 1024, 14336, GGMLType.Q4_K),
    "layer-8b-q6down": (4096, 4096, 1024, 14336, GGMLType.Q6_K),
    "layer-70b": (8192, 8192, 1024, 28672, GGMLType.Q4_K),
}


def bench_layer(args, peak: float, how: str) -> None:
    """The four products of a decoder layer between two attention calls (attention output, gate/up + activation, down, next
    layer's Q/K/V) as one multi-phase launch against the same four as separate launches."""
    for name, (d, qd, kvd, ff, down_t) in LAYERS.items():
        if args.only and args.only not in name:
            continue
        copies = 3
        sets = []
        for c in range(copies):
            wo = sk.repack(random_qweight(d, qd, GGMLType.Q4_K, 1), "cuda")
            wgu = sk.repack(sk.interleave(random_qweight(ff, d, GGMLType.Q4_K, 2), random_qweight(ff, d, GGMLType.Q4_K, 3)), "cuda")
            wd = sk.repack(random_qweight(d, ff, down_t, 4), "cuda")
            wqkv = [sk.repack(random_qweight(n, d, t, 5 + i), "cuda") for i, (n, t) in enumerate(((qd, GGMLType.Q4_K), (kvd, GGMLType.Q4_K), (kvd, GGMLType.Q6_K)))]
            sets.append((wo, wgu, wd, wqkv))
        nbytes = sum(w.nbytes for w in (sets[0][0], sets[0][1], sets[0][2], *sets[0][3]))
        nw = torch.ones(d, device="cuda")
        for nb in [int(v) for v in args.nb.split(",")]:
            if not (sk.fits_fused_input(nb, ff) and sk.fits_fused_input(nb, d)):
                continue
            ao, x, h, qkv = (torch.randn(nb, qd, device="cuda"), torch.randn(nb, d, device="cuda"), torch.zeros(nb, ff, device="cuda"),
                             torch.zeros(nb, qd + 2 * kvd, device="cuda"))

            def phases(i):
                wo, wgu, wd, wqkv = sets[i]
                return [sk.phase([wo], ao, x, mode=sk.MODE_ACCUM), sk.phase([wgu], x, h, norm_w=nw, eps=1e-5, mode=sk.MODE_GLU),
                        sk.phase([wd], h, x, mode=sk.MODE_ACCUM), sk.phase(wqkv, x, qkv, norm_w=nw, eps=1e-5)]

            def run_chain(i):
                sk.gemv_chain(phases(i), "cuda", max_ctas=args.ctas, split=args.split, ring=args.ring, pdl=bool(args.pdl))

            def run_separate(i):
                for ph in phases(i):
                    sk.gemv_chain([ph], "cuda", max_ctas=args.ctas, split=args.split, ring=args.ring, pdl=bool(args.pdl))

            for label, fn in (("one launch", run_chain), ("four launches", run_separate)):
                med = time_graph(fn, copies, max(2, args.reps // 4))
                sk.workspace("cuda").check()
                gbs = nbytes / med / 1e3
                print(f"sk {name:16s} nb={nb:2d} {label:13s} {med:8.1f} us  {gbs:7.0f} GB/s  {gbs / peak:5.2f} of {how} {peak:.0f} GB/s  ({nbytes / 1e6:.1f} MB)",
                      flush=True)
        del sets
        torch.cuda.empty_cache()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="both", choices=["dp4a", "sk", "both"], help="dp4a = kernels/gemv.cu, sk = kernels/gemv_sk.cu")
    ap.add_argument("--ctas", type=int, default=0, help="sk: CTAs per launch (0 = two per SM up to eight tokens)")
    ap.add_argument("--split", type=int, default=0, help="sk: 0 = chosen by the launcher, 1..4 = 1, 2, 4, 8 warps per range of units")
    ap.add_argument("--ring", type=int, default=0, help="sk: units per warp ring (0 = chosen by the launcher)")
    ap.add_argument("--pdl", type=int, default=1, help="sk: programmatic dependent launch between consecutive launches")
    ap.add_argument("--nb", default="1,4,8")
    ap.add_argument("--only", default="")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--copies", type=int, default=0, help="weight copies to rotate through (0 = enough to exceed L2)")
    args = ap.parse_args()
    peak, how = peak_gbs()
    rows_out = []
    if args.impl in ("sk", "both"):
        bench_sk(args, peak, how)
        bench_layer(args, peak, how)
    if args.impl == "sk":
        return
    for name, kind, segs, k in CASES:
        if args.only and args.only not in name:
            continue
        nbytes = 0
        one = [random_weight(n, k, t, i) for i, (n, t) in enumerate(segs)]
        if kind == "glu":
            one = [K.interleave_rows(one[0], random_weight(segs[0][0], k, segs[0][1], 7))]
        nbytes = sum(w.nbytes for w in one)
        copies = args.copies or max(2, int(300e6 // nbytes) + 1)
        sets = [one]
        for c in range(1, copies):
            sets.append([K.DevWeight(w.wtype, w.n, w.k, [p.clone() for p in w.planes]) for w in one])
        for nb in [int(x) for x in args.nb.split(",")]:
            x = torch.randn(nb, k, device="cuda")
            act = K.rmsnorm_quant(x, None, 0.0, do_norm=False)
            n_out = sum(w.n for w in one)
            out = torch.zeros(nb, n_out, device="cuda")

            def run(ws):
                if kind == "gemv":
                    K.gemv(ws, act, out=out, pdl=False)
                else:
                    K.gemv_glu_quant(ws[0], act, "silu", pdl=False)

            for i in range(3):
                run(sets[i % copies])
            torch.cuda.synchronize()
            # The launches are recorded into a CUDA graph so that the host-side cost of a launch
            # (tens of microseconds through Python) does not gate kernels that take a few microseconds.
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for i in range(args.reps):
                    run(sets[i % copies])
            graph.replay()
            torch.cuda.synchronize()
            ts = []
            for _ in range(5):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                graph.replay()
                b.record()
                torch.cuda.synchronize()
                ts.append(a.elapsed_time(b) * 1e3 / args.reps)
            ts.sort()
            med = ts[len(ts) // 2]
            gbs = nbytes / med / 1e3
            rows_out.append((name, nb, med, gbs, gbs / peak))
            print(f"{name:14s} nb={nb}  {med:8.1f} us  {gbs:7.0f} GB/s  {gbs / peak:5.2f} of {how} {peak:.0f} GB/s  "
                  f"({nbytes / 1e6:.1f} MB, {copies} copies)", flush=True)
        del sets
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
