"""Timing of the grouped expert GEMM of MoE prefill on gpt-oss-120b shapes (128 experts, top-4, gate/up 5760 x 2880).

    python -m ollama_b200.bench.moe_bench [tokens,tokens,...] [reps]

Two ways to the same product: the kernel that streams the MXFP4 blocks and expands them itself (kernels/gemm_q_grouped.cu), and
the grouped bf16 tensor-core GEMM over a 16-bit copy of the experts (kernels/gemm_tc.cu).  The expert blocks are random bytes
with scale bytes near 2^-7 (1.1 GB as MXFP4, 4.2 GB as bf16: both larger than L2); CUDA-event timed after warm-up; reported are
microseconds per launch and the wait-status word.
"""
import sys

import torch

from ..gguf.types import GGMLType
from ..models.weights import QWeight
from ..ops import cuda as K

torch.manual_seed(0)
E, n, k, topk = 128, 5760, 2880, 4
reps = int(sys.argv[2]) if len(sys.argv) > 2 else 5
# MXFP4 blocks straight from random bytes (17 bytes per 32 weights): scale bytes near 120
nblk = E * n * k // 32
raw = torch.randint(0, 256, (nblk, 17), dtype=torch.uint8, device='cuda')
raw[:, 0] = torch.randint(116, 124, (nblk,), dtype=torch.uint8, device='cuda')
qw = QWeight('w', GGMLType.MXFP4, (E, n, k), raw.view(-1))
dw = K.repack(qw, 'cuda')
for T in [int(x) for x in (sys.argv[1] if len(sys.argv) > 1 else '1024,2048').split(',')]:
    lids = torch.randint(0, E, (T * topk,), dtype=torch.int32, device='cuda')
    h = (torch.randn(T, k, device='cuda') * 0.5).to(torch.bfloat16)
    row, te, rows = K.moe_plan(lids, E)
    xs = K.moe_gather(h, row, topk, rows)
    def run_q():
        return K.gemm_q_grouped(xs, dw, te, glu='swiglu_oai')
    w16 = K.dequant_to_bf16(dw)
    def run_b():
        return K.gemm_bf16_grouped(xs, w16, E, te, None, glu='swiglu_oai')
    for name, fn in (('stream-mxfp4', run_q), ('bf16-copy', run_b)):
        for _ in range(2): fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record(); torch.cuda.synchronize(); ts.append(a.elapsed_time(b) * 1e3)
        ts.sort()
        print(f"T={T} rows={xs.shape[0]} {name}: {ts[len(ts)//2]:.1f} us  status={K.gemm_status()}")
    d = (run_q().float() - run_b().float()).abs().max().item()
    print('max diff', d)
