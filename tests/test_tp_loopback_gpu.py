"""The tensor-parallel exchange kernels on ONE GPU: two peer regions on the same device stand in for two ranks.

Every producer kernel of both "ranks" is enqueued before any consumer, on one stream, so no kernel ever waits for a kernel
that has not run yet (two waiting kernels on one GPU are never in flight together): the waits find their flags or epochs
already there, and what is checked is the addressing, the protocols' bookkeeping (epochs, parity halves, tickets) and the
arithmetic, against fp32 statements of the same exchanges.  The same kernels run between real GPUs in test_tp_gpu.py.
"""
import ctypes as C

import pytest
import torch

from ollama_b200.gguf.types import GGMLType
from ollama_b200.models.weights import QWeight

pytestmark = pytest.mark.gpu

W = 2                      # emulated ranks
CH_DEC, CH_LOGITS, CH_RS, CH_AG = 0, 1, 2, 3


def _K():
    from ollama_b200.ops import cuda as K
    return K


class _Group:
    """``W`` peer regions of one layout on one device; ``regs[r]`` sees all of them the way rank r of a real group would."""

    def __init__(self, layout):
        from ollama_b200.parallel.comm import PeerRegion
        from ollama_b200.parallel.transport import LocalTransport
        self.regs = [PeerRegion(layout.size, 0, 1, "cuda", LocalTransport()) for _ in range(W)]
        self.own = [r.base[0] for r in self.regs]
        for i, r in enumerate(self.regs):
            r.rank, r.world, r.base = i, W, list(self.own)
            for ch in range(4):
                r.set_wait_ms(ch, 300)

    def failed(self):
        return [r.failed_channels() for r in self.regs]

    def close(self):
        for i, r in enumerate(self.regs):      # back to a group of one, so that close() frees only what this region allocated
            r.rank, r.world, r.base = 0, 1, [self.own[i]]
            r.close()


def test_row_parallel_gemm_scatter_then_reduce_norm_and_all_gather():
    """Prefill exchange: each rank's partial product rows land, as bf16, in the slab of their owner (GEMM epilogue stores);
    the owner adds the slabs to its shard of the residual stream, normalises and stores the bf16 row into every rank's
    activation buffer."""
    from ollama_b200.parallel.comm import Layout
    from ollama_b200.parallel.tp_engine import TpNormGatherArgs
    K = _K()
    T, d, kin, rpr = 256, 512, 384, 128
    lay = Layout()
    b_parts = lay.add("parts", W * rpr * d * 2)
    b_h = lay.add("h", T * d * 2)
    grp = _Group(lay)
    try:
        g = torch.Generator().manual_seed(0)
        xs = [(torch.randn(T, kin, generator=g) * 0.5).to(torch.bfloat16).cuda() for _ in range(W)]
        ws = [(torch.randn(d, kin, generator=g) * 0.05).to(torch.bfloat16).cuda() for _ in range(W)]
        resid = [torch.randn(rpr, d, generator=g).cuda() for _ in range(W)]
        norm_w = (1 + 0.1 * torch.randn(d, generator=g)).cuda()
        partial = [xs[r].float() @ ws[r].float().t() for r in range(W)]                      # [T, d] of rank r
        for r, reg in enumerate(grp.regs):                                                      # producers of both ranks first
            cm = reg.send(CH_RS, [reg.addr(b_parts, o, r * rpr * d * 2) for o in range(W)])
            K.gemm_bf16_scatter(xs[r], ws[r], d, cm, rpr, None)
        torch.cuda.synchronize()
        for o, reg in enumerate(grp.regs):
            got = reg.tensor(b_parts, (W, rpr, d), torch.bfloat16).float()
            for r in range(W):
                want = partial[r][o * rpr:(o + 1) * rpr]
                assert torch.allclose(got[r], want, atol=2e-2, rtol=2e-2), (o, r)
        shard = [t.clone() for t in resid]
        for o, reg in enumerate(grp.regs):                                                      # then the consumers / all-gather producers
            a = TpNormGatherArgs()
            a.x, a.w, a.eps, a.k, a.row0 = K.ptr(shard[o]), K.ptr(norm_w), 1e-5, d, o * rpr
            a.parts, a.n_part, a.part_stride = reg.addr(b_parts), W, rpr * d
            a.rs_chan = reg.chan(CH_RS)
            a.ag = reg.send(CH_AG, [reg.addr(b_h, q) for q in range(W)])
            f = K.lib().b2_tp_norm_gather
            f.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
            K._check(f(C.addressof(a), rpr, K.stream()), "tp_norm_gather")
        for reg in grp.regs:
            reg.wait(CH_AG)
        torch.cuda.synchronize()
        assert grp.failed() == [[], []]
        from ollama_b200.ops import reference as R
        for o in range(W):
            summed = resid[o] + sum(partial[r][o * rpr:(o + 1) * rpr].to(torch.bfloat16).float() for r in range(W))
            assert torch.allclose(shard[o], summed, atol=2e-2, rtol=1e-2)
        full = torch.cat([R.rmsnorm(s, norm_w, 1e-5) for s in shard])
        for reg in grp.regs:
            h = reg.tensor(b_h, (T, d), torch.bfloat16).float()
            assert torch.allclose(h, full.to(torch.bfloat16).float(), atol=2e-2, rtol=2e-2)
    finally:
        grp.close()


def test_expert_parallel_rows_go_to_their_owners():
    """Expert parallelism in prefill: a rank's weighted expert outputs for all tokens are scattered, as bf16 rows, to the slab
    of the rank that owns each row."""
    from ollama_b200.parallel.comm import Layout
    K = _K()
    T, d, rpr = 200, 256, 100
    lay = Layout()
    b_parts = lay.add("parts", W * rpr * d * 2)
    grp = _Group(lay)
    try:
        g = torch.Generator().manual_seed(1)
        part = [torch.randn(T, d, generator=g).cuda() for _ in range(W)]
        f = K.lib().b2_tp_scatter_rows
        f.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        for r, reg in enumerate(grp.regs):
            cm = reg.send(CH_RS, [reg.addr(b_parts, o, r * rpr * d * 2) for o in range(W)])
            K._check(f(K.ptr(part[r]), T, d, rpr, C.addressof(cm), K.stream()), "tp_scatter_rows")
        for reg in grp.regs:
            reg.wait(CH_RS)
        torch.cuda.synchronize()
        assert grp.failed() == [[], []]
        for o, reg in enumerate(grp.regs):
            got = reg.tensor(b_parts, (W, rpr, d), torch.bfloat16).float()
            for r in range(W):
                assert torch.equal(got[r], part[r][o * rpr:(o + 1) * rpr].to(torch.bfloat16).float()), (o, r)
    finally:
        grp.close()


def test_decode_exchange_value_epoch_words_and_logits_gather():
    """Decode exchange: a row-parallel GEMV stores (value, epoch) words into its slab on every rank; the next kernel adds the
    slabs of the epoch it expects to the residual, normalises and quantises.  Two rounds, so both parity halves and the epoch
    bookkeeping are used.  Then the column-parallel head: each rank's vocabulary rows land in every rank's logits buffer."""
    from ollama_b200.parallel.comm import Layout
    K = _K()
    nb, MB, d, kin, V = 3, 8, 512, 1024, 640
    lay = Layout()
    b_dec = lay.add("dec", 2 * W * MB * d * 8)
    b_logits = lay.add("logits", MB * V * 4)
    grp = _Group(lay)
    try:
        g = torch.Generator().manual_seed(2)
        wq = [QWeight.from_float("w", torch.randn(d, kin, generator=g) * 0.05, GGMLType.Q8_0) for _ in range(W)]
        dw = [K.repack(q, "cuda") for q in wq]
        x = [torch.randn(nb, d, generator=g).cuda() for _ in range(W)]          # every rank's copy of the residual stream
        x[1].copy_(x[0])
        norm_w = (1 + 0.1 * torch.randn(d, generator=g)).cuda()
        want_x = x[0].clone().cpu()
        from ollama_b200.ops import reference as R
        for rnd in range(2):
            acts_in = [torch.randn(nb, kin, generator=g).cuda() for _ in range(W)]
            partial = []
            for r, reg in enumerate(grp.regs):
                act = K.rmsnorm_quant(acts_in[r], None, 0.0, do_norm=False)
                cm = reg.send(CH_DEC, [reg.addr(b_dec, o, r * MB * d * 8) for o in range(W)], parity_stride=W * MB * d)
                cm.ll = 1
                a = K.GemvArgs()
                a.seg[0] = dw[r].desc()
                a.nseg, a.nb = 1, nb
                a.xq, a.xds, a.xf, a.out, a.ldo, a.accumulate = K.ptr(act.q), K.ptr(act.ds), K.ptr(act.f), None, d, 0
                a.cm = cm
                K._check(K.lib().b2_gemv(C.byref(a), 0, K.stream()), "gemv(send)")
                partial.append(K.gemv([dw[r]], act).cpu())          # the same product into a local buffer (its numerics are checked elsewhere)
            outs = []
            for o, reg in enumerate(grp.regs):
                xq = torch.empty(nb, d, dtype=torch.int8, device="cuda")
                xds = torch.empty(nb, d // 32, 2, device="cuda")
                xf = torch.empty(nb, d, device="cuda")
                a = K.NormQuantArgs(K.ptr(x[o]), K.ptr(norm_w), 1e-5, d, 1, K.ptr(xq), K.ptr(xds), K.ptr(xf), None)
                a.parts, a.n_part, a.part_stride, a.parity_stride, a.chan = reg.addr(b_dec), W, MB * d, W * MB * d, reg.chan(CH_DEC)
                K._check(K.lib().b2_rmsnorm_quant(C.byref(a), nb, 0, K.stream()), "rmsnorm_quant(reduce)")
                outs.append(xf)
            torch.cuda.synchronize()
            assert grp.failed() == [[], []], rnd
            want_x = want_x + sum(partial)
            for o in range(W):
                assert torch.allclose(x[o].cpu(), want_x, atol=2e-3, rtol=1e-3), (rnd, o)
                assert torch.allclose(outs[o].cpu(), R.rmsnorm(want_x, norm_w.cpu(), 1e-5), atol=3e-3, rtol=2e-3), (rnd, o)
        # column-parallel head: rank r owns vocabulary rows [r * V / W, (r + 1) * V / W)
        vh = V // W
        hq = [QWeight.from_float("h", torch.randn(vh, d, generator=g) * 0.05, GGMLType.Q8_0) for _ in range(W)]
        hd = [K.repack(q, "cuda") for q in hq]
        act = K.rmsnorm_quant(x[0], None, 0.0, do_norm=False)
        for r, reg in enumerate(grp.regs):
            cm = reg.send(CH_LOGITS, [reg.addr(b_logits, o, r * vh * 4) for o in range(W)])
            a = K.GemvArgs()
            a.seg[0] = hd[r].desc()
            a.nseg, a.nb = 1, nb
            a.xq, a.xds, a.xf, a.out, a.ldo, a.accumulate = K.ptr(act.q), K.ptr(act.ds), K.ptr(act.f), None, V, 0
            a.cm = cm
            K._check(K.lib().b2_gemv(C.byref(a), 0, K.stream()), "gemv(logits)")
        for reg in grp.regs:
            reg.wait(CH_LOGITS)
        torch.cuda.synchronize()
        assert grp.failed() == [[], []]
        want = torch.cat([K.gemv([hd[r]], act).cpu() for r in range(W)], dim=1)
        for reg in grp.regs:
            got = reg.tensor(b_logits, (MB, V), torch.float32)[:nb].cpu()
            assert torch.allclose(got, want, atol=1e-5, rtol=1e-5)
    finally:
        grp.close()
