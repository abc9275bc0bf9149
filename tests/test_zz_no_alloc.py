"""The allocation-free decode-attention entry point (kernels/no_alloc.h).

Some embedders of the kernel library may not allocate device memory -- a host application whose memory
pool owns the device, a plugin whose allocator must account for every byte, a latency-critical loop where
an allocation would stall the device -- so ``b2_attn_decode_noalloc`` keeps its split-K scratch in arrays
that are part of the library image.  The test calls it through the exported C symbol, twice in a row with
different inputs (the second call reuses whatever the first left in the shared arrays), and checks each
result against the regular entry point, which takes caller-allocated scratch.  It also checks that a
problem larger than the built-in arrays is refused.  This file sorts last on purpose: a run that stops at
the first failure has then already executed every other test.
"""
import ctypes as C
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run_both(K, seed: int, nb: int, H: int, Hkv: int, hd: int, n_ctx: int, n_splits: int):
    g = torch.Generator().manual_seed(seed)
    n_slots = 3
    kc = (torch.randn(n_slots, Hkv, n_ctx, hd, generator=g) * 0.5).to(torch.float16).cuda()
    vc = (torch.randn(n_slots, Hkv, n_ctx, hd, generator=g) * 0.5).to(torch.float16).cuda()
    q = torch.randn(nb, H, hd, generator=g).cuda()
    pos = torch.randint(0, n_ctx, (nb,), generator=g).to(torch.int32).cuda()
    slots = torch.randint(0, n_slots, (nb,), generator=g).to(torch.int32).cuda()
    scale = 1 / math.sqrt(hd)
    ref, ref_q = K.attn_decode(q, kc, vc, pos, slots, scale=scale, n_splits=n_splits)

    out = torch.zeros(nb, H * hd, device="cuda")
    oq = torch.zeros(nb, H * hd, device="cuda", dtype=torch.int8)
    ods = torch.zeros(nb, H * hd // 32, 2, device="cuda")
    a = K.AttnDecodeArgs(K.ptr(q), K.ptr(kc), K.ptr(vc), K.ptr(pos), K.ptr(slots), H, Hkv, n_ctx, n_splits, scale, 0.0, 0, None, None)
    c = K.AttnCombineArgs(None, None, None, 0, 0, 0, K.ptr(out), K.ptr(oq), K.ptr(ods))
    fn = K.lib().b2_attn_decode_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
    rc = fn(C.byref(a), C.byref(c), nb, hd, K.stream())
    torch.cuda.synchronize()
    return rc, out, oq, ods, ref, ref_q


def test_noalloc_matches_regular_entry_point_twice():
    from ollama_b200.ops import cuda as K
    for seed, shape in ((1, dict(nb=3, H=8, Hkv=2, hd=128, n_ctx=200, n_splits=4)), (2, dict(nb=2, H=8, Hkv=8, hd=64, n_ctx=333, n_splits=6))):
        rc, out, oq, ods, ref, ref_q = _run_both(K, seed, **shape)
        assert rc == 0
        assert torch.allclose(out, ref, atol=2e-3, rtol=2e-3)
        assert (oq.int() - ref_q.q.int()).abs().max().item() <= 1
        assert torch.allclose(ods, ref_q.ds, atol=1e-5, rtol=1e-3)


def test_noalloc_rejects_oversized_problem():
    from ollama_b200.ops import cuda as K
    fn = K.lib().b2_attn_decode_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
    a = K.AttnDecodeArgs(None, None, None, None, None, 128, 8, 1024, 32, 1.0, 0.0, 0, None, None)     # 8 * 128 * 32 = 32768 entries > 16384
    c = K.AttnCombineArgs()
    assert fn(C.byref(a), C.byref(c), 8, 128, K.stream()) == -2
