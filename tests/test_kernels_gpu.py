"""sm_100a kernels against plain PyTorch fp32 statements of the same ops."""
import math

import pytest
import torch

from ollama_b200.gguf import quants
from ollama_b200.gguf.types import GGMLType
from ollama_b200.models.weights import QWeight
from ollama_b200.ops import reference as R

pytestmark = pytest.mark.gpu

TYPES = [GGMLType.Q4_K, GGMLType.Q6_K, GGMLType.Q5_K, GGMLType.Q8_0, GGMLType.Q4_0, GGMLType.MXFP4, GGMLType.F16, GGMLType.BF16,
         GGMLType.F32, GGMLType.Q4_1]


def _K():
    from ollama_b200.ops import cuda as K
    return K


def _weight(t, n, k, seed=0, bias=False):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(n, k, generator=g) * 0.05
    qw = QWeight.from_float("w", w, t) if quants.can_quantize(t) else None
    if qw is None:   # types we can decode but not encode: fill random valid blocks via a supported encoder of equal layout size
        pytest.skip(f"no encoder for {t}")
    b = torch.randn(n, generator=g) * 0.1 if bias else None
    return qw, b


def _quant_act_ref(x):
    """int8 blocks of 32 exactly as the kernels quantise activations."""
    xb = x.view(x.shape[0], -1, 32)
    d = xb.abs().amax(-1) / 127.0
    q = torch.where(d[..., None] > 0, torch.round(xb / d[..., None].clamp_min(1e-30)), torch.zeros_like(xb))
    return (q * d[..., None]).view_as(x)


@pytest.mark.parametrize("t", TYPES)
def test_repack_dequant_matches_codec(t):
    K = _K()
    if t == GGMLType.Q4_1:
        w = torch.randn(40, 512) * 0.05
        qw = QWeight.from_float("w", w, t)
    else:
        qw, _ = _weight(t, 40, 512)
    ref = qw.dequant()
    dw = K.repack(qw, "cuda")
    got = K.dequant_to_bf16(dw).float().cpu()
    assert torch.allclose(got, ref.to(torch.bfloat16).float(), atol=1e-6, rtol=1e-2)


@pytest.mark.parametrize("t", TYPES[:9])
@pytest.mark.parametrize("nb", [1, 3, 8])
def test_gemv_matches_reference(t, nb):
    K = _K()
    n, k = 200, 1024
    qw, bias = _weight(t, n, k, bias=True)
    dw = K.repack(qw, "cuda", bias=bias)
    x = torch.randn(nb, k, generator=torch.Generator().manual_seed(1)).cuda()
    act = K.rmsnorm_quant(x, None, 0.0, do_norm=False)
    y = K.gemv([dw], act).cpu()
    wf = qw.dequant()
    xr = _quant_act_ref(x.cpu()) if dw.quant_input else x.cpu()
    ref = xr @ wf.t() + bias
    assert torch.allclose(y, ref, atol=2e-3 * ref.abs().max().item(), rtol=1e-3), (y - ref).abs().max()
    # and against un-quantised activations within the int8 activation error
    full = x.cpu() @ wf.t() + bias
    assert ((y - full).norm() / full.norm()).item() < 2e-2
    # accumulate form
    out = torch.ones(nb, n, device="cuda")
    K.gemv([dw], act, out=out, accumulate=True)
    assert torch.allclose(out.cpu(), ref + 1.0, atol=2e-3 * ref.abs().max().item(), rtol=1e-3)


def test_gemv_multi_segment_and_large_rows():
    K = _K()
    k = 512
    qa, _ = _weight(GGMLType.Q4_K, 96, k, seed=1)
    qb, _ = _weight(GGMLType.Q6_K, 40, k, seed=2)
    qc, _ = _weight(GGMLType.Q8_0, 9000, k, seed=3)      # > 8192 rows takes the 4-rows-per-warp variant
    ws = [K.repack(q, "cuda") for q in (qa, qb, qc)]
    x = torch.randn(2, k).cuda()
    act = K.rmsnorm_quant(x, None, 0.0, do_norm=False)
    y = K.gemv(ws, act).cpu()
    xr = _quant_act_ref(x.cpu())
    ref = torch.cat([xr @ q.dequant().t() for q in (qa, qb, qc)], 1)
    assert y.shape == (2, 96 + 40 + 9000)
    assert torch.allclose(y, ref, atol=2e-3 * ref.abs().max().item(), rtol=1e-3)


@pytest.mark.parametrize("act", ["silu", "gelu_tanh", "swiglu_oai"])
def test_glu_quant(act):
    K = _K()
    n, k, nb = 256, 512, 3
    qg, bg = _weight(GGMLType.Q4_K, n, k, seed=1, bias=True)
    qu, bu = _weight(GGMLType.Q4_K, n, k, seed=2, bias=True)
    gu = K.interleave_rows(K.repack(qg, "cuda", bias=bg), K.repack(qu, "cuda", bias=bu))
    x = torch.randn(nb, k).cuda() * 3
    xa = K.rmsnorm_quant(x, None, 0.0, do_norm=False)
    h = K.gemv_glu_quant(gu, xa, act, want_f=True)
    xr = _quant_act_ref(x.cpu())
    ref = R.glu(xr @ qg.dequant().t() + bg, xr @ qu.dequant().t() + bu, act)
    assert torch.allclose(h.f.cpu(), ref, atol=2e-3 * ref.abs().max().item(), rtol=2e-3)
    deq = (h.q.cpu().float().view(nb, -1, 32) * h.ds.cpu()[..., 0:1]).view(nb, n)
    assert torch.allclose(deq, _quant_act_ref(h.f.cpu()), atol=1e-5 + 1e-2 * ref.abs().max().item() / 127)
    sums = (h.q.cpu().float().view(nb, -1, 32).sum(-1) * h.ds.cpu()[..., 0])
    assert torch.allclose(sums, h.ds.cpu()[..., 1], atol=1e-4, rtol=1e-4)


def test_rmsnorm_quant_and_residual():
    K = _K()
    x = torch.randn(5, 768).cuda() * 2
    w = torch.rand(768).cuda() + 0.5
    a = K.rmsnorm_quant(x, w, 1e-5)
    ref = R.rmsnorm(x.cpu(), w.cpu(), 1e-5)
    assert torch.allclose(a.f.cpu(), ref, atol=1e-5, rtol=1e-5)
    deq = (a.q.cpu().float().view(5, -1, 32) * a.ds.cpu()[..., 0:1]).view(5, 768)
    assert (deq - ref).abs().max() <= ref.abs().max() / 127 * 0.51 + 1e-6
    res = torch.ones(5, 768).cuda()
    K.rmsnorm_quant(x, w, 1e-5, residual=res)
    assert torch.allclose(res.cpu(), ref + 1, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("neox,qk_norm,hd,n_rot", [(False, False, 128, 128), (True, True, 64, 64), (True, False, 64, 32)])
def test_rope_kv(neox, qk_norm, hd, n_rot):
    K = _K()
    H, Hkv, nt, n_ctx, n_slots = 4, 2, 5, 64, 3
    qkv = torch.randn(nt, (H + 2 * Hkv) * hd).cuda()
    pos = torch.tensor([0, 7, 8, 31, 63], dtype=torch.int32).cuda()
    slots = torch.tensor([0, 1, 1, 2, 0], dtype=torch.int32).cuda()
    inv, ms = R.rope_inv_freq(n_rot, 10000.0, device="cuda")
    qn = (torch.rand(hd) + 0.5).cuda() if qk_norm else None
    kn = (torch.rand(hd) + 0.5).cuda() if qk_norm else None
    kc = torch.zeros(n_slots, Hkv, n_ctx, hd, device="cuda", dtype=torch.float16)
    vc = torch.zeros_like(kc)
    q = K.rope_kv(qkv, pos, slots, inv, n_heads=H, n_kv_heads=Hkv, hd=hd, n_rot=n_rot, neox=neox, mscale=1.3, k_cache=kc, v_cache=vc,
                  q_norm=qn, k_norm=kn, eps=1e-6)
    qr = qkv[:, :H * hd].view(nt, H, hd).cpu()
    kr = qkv[:, H * hd:(H + Hkv) * hd].view(nt, Hkv, hd).cpu()
    vr = qkv[:, (H + Hkv) * hd:].view(nt, Hkv, hd).cpu()
    if qk_norm:
        qr, kr = R.rmsnorm(qr, qn.cpu(), 1e-6), R.rmsnorm(kr, kn.cpu(), 1e-6)
    style = "neox" if neox else "norm"
    qr = R.rope(qr, pos.cpu(), inv.cpu(), style, 1.3)
    kr = R.rope(kr, pos.cpu(), inv.cpu(), style, 1.3)
    assert torch.allclose(q.cpu(), qr, atol=2e-4, rtol=1e-4)
    for t in range(nt):
        assert torch.allclose(kc[slots[t], :, pos[t]].float().cpu(), kr[t], atol=5e-3, rtol=2e-3)
        assert torch.allclose(vc[slots[t], :, pos[t]].float().cpu(), vr[t], atol=5e-3, rtol=2e-3)


@pytest.mark.parametrize("neox,qk_norm,hd,n_rot,H,Hkv,q8", [(False, False, 128, 128, 12, 2, False), (True, True, 64, 64, 9, 3, False),
                                                          (True, False, 64, 32, 4, 2, True), (True, True, 256, 256, 3, 1, False)])
def test_rope_kv_of_a_prefill_chunk(neox, qk_norm, hd, n_rot, H, Hkv, q8):
    """Chunks of 64 tokens and more take the per-token form of the kernel (a warp per head, the sines and cosines once per token):
    rotated queries, and keys / values in the f16 or int8 cache, against the fp32 statement; positions far into a long context."""
    K = _K()
    nt, n_ctx, n_slots, slot = 150, 200, 2, 1
    g = torch.Generator().manual_seed(hd + H)
    qkv = torch.randn(nt, (H + 2 * Hkv) * hd, generator=g).cuda()
    pos0 = 40
    pos = torch.arange(pos0, pos0 + nt, dtype=torch.int32).cuda()
    slots = torch.full((nt,), slot, dtype=torch.int32).cuda()
    inv, ms = R.rope_inv_freq(n_rot, 10000.0, device="cuda")
    qn = (torch.rand(hd, generator=g) + 0.5).cuda() if qk_norm else None
    kn = (torch.rand(hd, generator=g) + 0.5).cuda() if qk_norm else None
    kc = torch.zeros(n_slots, Hkv, n_ctx, hd, device="cuda", dtype=torch.int8 if q8 else torch.float16)
    vc = torch.zeros_like(kc)
    ks = torch.zeros(n_slots, Hkv, n_ctx, hd // 32, device="cuda", dtype=torch.float16) if q8 else None
    vs = torch.zeros_like(ks) if q8 else None
    q = K.rope_kv(qkv, pos, slots, inv, n_heads=H, n_kv_heads=Hkv, hd=hd, n_rot=n_rot, neox=neox, mscale=1.3, k_cache=kc, v_cache=vc,
                  q_norm=qn, k_norm=kn, eps=1e-6, k_scale=ks, v_scale=vs)
    qr = qkv[:, :H * hd].view(nt, H, hd).cpu()
    kr = qkv[:, H * hd:(H + Hkv) * hd].view(nt, Hkv, hd).cpu()
    vr = qkv[:, (H + Hkv) * hd:].view(nt, Hkv, hd).cpu()
    if qk_norm:
        qr, kr = R.rmsnorm(qr, qn.cpu(), 1e-6), R.rmsnorm(kr, kn.cpu(), 1e-6)
    style = "neox" if neox else "norm"
    qr = R.rope(qr, pos.cpu(), inv.cpu(), style, 1.3)
    kr = R.rope(kr, pos.cpu(), inv.cpu(), style, 1.3)
    assert torch.allclose(q.cpu(), qr, atol=3e-4, rtol=1e-4)
    kg, vg = kc[slot, :, pos0:pos0 + nt].float(), vc[slot, :, pos0:pos0 + nt].float()
    if q8:
        kg = (kg.view(Hkv, nt, -1, 32) * ks[slot, :, pos0:pos0 + nt].float()[..., None]).view(Hkv, nt, hd)
        vg = (vg.view(Hkv, nt, -1, 32) * vs[slot, :, pos0:pos0 + nt].float()[..., None]).view(Hkv, nt, hd)
    tol = 0.04 if q8 else 5e-3
    assert torch.allclose(kg.cpu().transpose(0, 1), kr, atol=tol, rtol=tol)
    assert torch.allclose(vg.cpu().transpose(0, 1), vr, atol=tol, rtol=tol)
    assert float(kc[slot, :, :pos0].float().abs().max()) == 0.0 and float(kc[0].float().abs().max()) == 0.0      # nothing outside the chunk's rows


@pytest.mark.parametrize("hd,H,Hkv", [(128, 8, 2), (64, 8, 8), (64, 6, 3), (256, 4, 1), (32, 8, 2)])
@pytest.mark.parametrize("window,softcap,use_sinks", [(0, 0.0, False), (24, 0.0, True), (0, 30.0, False)])
@pytest.mark.parametrize("mma", [0, 1])
def test_attn_decode(hd, H, Hkv, window, softcap, use_sinks, mma, attn_mode):
    """mma = 1: the tensor-core split-K kernel (head sizes 64 / 128; other sizes fall back to the scalar kernel)."""
    K = _K()
    attn_mode(mma)
    n_slots, n_ctx, nb = 3, 160, 3
    kc = (torch.randn(n_slots, Hkv, n_ctx, hd) * 0.5).to(torch.float16).cuda()
    vc = (torch.randn(n_slots, Hkv, n_ctx, hd) * 0.5).to(torch.float16).cuda()
    q = torch.randn(nb, H, hd).cuda()
    pos = torch.tensor([0, 77, 159], dtype=torch.int32).cuda()
    slots = torch.tensor([2, 0, 1], dtype=torch.int32).cuda()
    sinks = torch.randn(H).cuda() if use_sinks else None
    scale = 1 / math.sqrt(hd)
    for n_splits in (1, 4):
        out, qa = K.attn_decode(q, kc, vc, pos, slots, scale=scale, n_splits=n_splits, window=window, softcap=softcap, sinks=sinks)
        for b in range(nb):
            p, s = int(pos[b]), int(slots[b])
            tc = mma and hd in (64, 128)          # the tensor-core kernel multiplies f16 queries and f16 probabilities
            qr = q[b:b + 1].to(torch.float16).float().cpu() if tc else q[b:b + 1].cpu()
            ref = R.attention(qr, kc[s, :, :p + 1].transpose(0, 1).float().cpu(), vc[s, :, :p + 1].transpose(0, 1).float().cpu(),
                              torch.tensor([p]), torch.arange(p + 1), scale=scale, window=window, softcap=softcap,
                              sinks=sinks.cpu() if use_sinks else None)
            tol = dict(atol=1e-2, rtol=2e-2) if tc else dict(atol=2e-3, rtol=2e-3)
            assert torch.allclose(out[b].cpu(), ref.reshape(-1), **tol), (n_splits, b, (out[b].cpu() - ref.reshape(-1)).abs().max())
        deq = (qa.q.cpu().float().view(nb, -1, 32) * qa.ds.cpu()[..., 0:1]).view(nb, -1)
        assert (deq - out.cpu()).abs().max() <= out.abs().max().item() / 127 + 1e-6


@pytest.mark.parametrize("hd,H,Hkv,n_rot", [(128, 32, 8, 128), (64, 8, 4, 64), (128, 8, 2, 64), (64, 6, 3, 32)])
@pytest.mark.parametrize("neox", [False, True])
@pytest.mark.parametrize("window,n_splits", [(0, 1), (0, 4), (48, 4)])
def test_attn_decode_with_rotary_embedding_and_cache_append_inside(hd, H, Hkv, n_rot, neox, window, n_splits, attn_mode):
    """One launch that rotates Q and the new K, appends K / V and attends, against the two-kernel path (rope_kv, then the
    tensor-core attention): same cache rows bit for bit, same output; sequences at position 0, inside a tile, on a tile edge."""
    K = _K()
    attn_mode(1)
    n_slots, n_ctx, nb = 4, 320, 4
    kc = (torch.randn(n_slots, Hkv, n_ctx, hd) * 0.5).to(torch.float16).cuda()
    vc = (torch.randn(n_slots, Hkv, n_ctx, hd) * 0.5).to(torch.float16).cuda()
    qkv = torch.randn(nb, (H + 2 * Hkv) * hd).cuda()
    pos = torch.tensor([0, 63, 64, 300], dtype=torch.int32).cuda()
    slots = torch.tensor([2, 0, 3, 1], dtype=torch.int32).cuda()
    inv = (1.0 / (10000.0 ** (torch.arange(0, n_rot, 2).float() / n_rot))).cuda()
    scale = 1 / math.sqrt(hd)
    kc2, vc2 = kc.clone(), vc.clone()
    q = K.rope_kv(qkv, pos, slots, inv, n_heads=H, n_kv_heads=Hkv, hd=hd, n_rot=n_rot, neox=neox, mscale=1.3, k_cache=kc, v_cache=vc)
    want, _ = K.attn_decode(q, kc, vc, pos, slots, scale=scale, n_splits=n_splits, window=window, quant_out=False)
    for b in range(nb):                                 # the fused launch must not depend on what the cache row held before
        kc2[int(slots[b]), :, int(pos[b])] = float("nan")
        vc2[int(slots[b]), :, int(pos[b])] = float("nan")
    got = K.attn_decode_rope(qkv, kc2, vc2, pos, slots, inv, n_heads=H, n_rot=n_rot, neox=neox, mscale=1.3, scale=scale, n_splits=n_splits, window=window)
    assert got is not None
    torch.cuda.synchronize()
    assert torch.equal(kc2, kc) and torch.equal(vc2, vc)
    assert torch.allclose(got, want, atol=2e-3, rtol=2e-3), (got - want).abs().max()
    # quantised caches and head sizes without a tensor-core instantiation are refused before anything is launched
    assert K.attn_decode_rope(torch.randn(1, 3 * 256).cuda(), torch.zeros(1, 1, 32, 256, dtype=torch.float16).cuda(), torch.zeros(1, 1, 32, 256, dtype=torch.float16).cuda(),
                              pos[:1], slots[:1] * 0, inv, n_heads=1, n_rot=64, neox=neox, mscale=1.0, scale=1.0, n_splits=1) is None


@pytest.mark.parametrize("hd,H,Hkv", [(128, 32, 8), (64, 16, 2), (128, 16, 1)])
@pytest.mark.parametrize("q8", [False, True])
def test_attn_decode_tensor_core_long_context(hd, H, Hkv, q8, attn_mode):
    """Many tiles per split, several splits, 4 / 8 / 16 heads per KV head: the tensor-core kernel against the scalar one
    and against itself (two runs give the same bits: no dependence on timing)."""
    K = _K()
    n_slots, n_ctx, nb = 2, 4096, 2
    g = torch.Generator().manual_seed(hd + H)
    kf = torch.randn(n_slots, Hkv, n_ctx, hd, generator=g) * 0.5
    vf = torch.randn(n_slots, Hkv, n_ctx, hd, generator=g) * 0.5
    ks = vs = None
    if q8:
        def quant(x):
            b = x.view(n_slots, Hkv, n_ctx, hd // 32, 32)
            d = (b.abs().amax(-1, keepdim=True) / 127).to(torch.float16)
            qv = torch.where(d > 0, torch.round(b / d.float().clamp_min(1e-30)), torch.zeros_like(b)).clamp(-127, 127).to(torch.int8)
            return qv.view(n_slots, Hkv, n_ctx, hd).cuda(), d.squeeze(-1).cuda()
        (kc, ks), (vc, vs) = quant(kf), quant(vf)
    else:
        kc, vc = kf.to(torch.float16).cuda(), vf.to(torch.float16).cuda()
    q = torch.randn(nb, H, hd, generator=g).cuda()
    pos = torch.tensor([4001, 130], dtype=torch.int32).cuda()
    slots = torch.tensor([1, 0], dtype=torch.int32).cuda()
    scale = 1 / math.sqrt(hd)
    for n_splits in (1, 8):
        attn_mode(0)
        ref, _ = K.attn_decode(q, kc, vc, pos, slots, scale=scale, n_splits=n_splits, k_scale=ks, v_scale=vs)
        attn_mode(1)
        outs = []
        for stages in (2, 3, 4):               # the pipeline depths of the kernel compute the same sums in the same order
            K.attn_decode_stages(stages)
            try:
                a, _ = K.attn_decode(q, kc, vc, pos, slots, scale=scale, n_splits=n_splits, k_scale=ks, v_scale=vs)
                b, _ = K.attn_decode(q, kc, vc, pos, slots, scale=scale, n_splits=n_splits, k_scale=ks, v_scale=vs)
            finally:
                K.attn_decode_stages(0)
            assert torch.equal(a, b)
            assert torch.allclose(a, ref, atol=3e-3, rtol=2e-2), (a - ref).abs().max()
            outs.append(a)
        assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


def test_embed_and_argmax():
    K = _K()
    qw, _ = _weight(GGMLType.Q6_K, 300, 512)
    tab = K.repack(qw, "cuda")
    ids = torch.tensor([0, 299, 17], dtype=torch.int32).cuda()
    x = K.embed(tab, ids, 2.0).cpu()
    assert torch.allclose(x, qw.dequant()[[0, 299, 17]] * 2.0, atol=1e-6)
    lg = torch.randn(4, 50021).cuda()
    lg[2, 40000] = 100.0
    assert K.argmax(lg).cpu().tolist() == lg.argmax(-1).cpu().tolist()


@pytest.mark.parametrize("hd,H,Hkv", [(128, 8, 2), (64, 4, 4), (64, 6, 1), (256, 4, 2), (32, 8, 2)])
@pytest.mark.parametrize("T,pos0,window,softcap,use_sinks,causal", [(150, 0, 0, 0.0, False, True), (70, 131, 48, 0.0, True, True),
                                                                    (64, 64, 0, 30.0, False, True), (33, 0, 0, 0.0, False, False)])
def test_attn_prefill(hd, H, Hkv, T, pos0, window, softcap, use_sinks, causal):
    """Flash-attention prefill kernel against the fp32 statement of attention over the same f16 cache."""
    K = _K()
    n_slots, n_ctx, slot = 2, 300, 1
    g = torch.Generator().manual_seed(hd + T)
    kc = (torch.randn(n_slots, Hkv, n_ctx, hd, generator=g) * 0.7).to(torch.float16).cuda()
    vc = (torch.randn(n_slots, Hkv, n_ctx, hd, generator=g) * 0.7).to(torch.float16).cuda()
    q = torch.randn(T, H, hd, generator=g).cuda()
    sinks = torch.randn(H, generator=g).cuda() if use_sinks else None
    scale = 1 / math.sqrt(hd)
    p_end = pos0 + T
    out = K.attn_prefill(q, kc, vc, slot, pos0, p_end, scale, causal, window, softcap, sinks).float().cpu().view(T, H, hd)
    qh = q.to(torch.float16).float().cpu()            # the kernel multiplies f16 operands
    ref = R.attention(qh, kc[slot, :, :p_end].transpose(0, 1).float().cpu(), vc[slot, :, :p_end].transpose(0, 1).float().cpu(),
                      torch.arange(pos0, p_end), torch.arange(p_end), scale=scale, causal=causal, window=window, softcap=softcap,
                      sinks=sinks.cpu() if use_sinks else None)
    assert torch.allclose(out, ref, atol=1e-2, rtol=2e-2), (out - ref).abs().max()


@pytest.mark.parametrize("hd,H,Hkv", [(128, 8, 2), (64, 4, 4), (128, 2, 1)])
@pytest.mark.parametrize("T,pos0,window,softcap,use_sinks,causal", [(300, 517, 0, 0.0, False, True), (129, 0, 0, 0.0, True, True),
                                                                    (260, 400, 200, 0.0, True, True), (128, 256, 0, 30.0, False, True),
                                                                    (200, 0, 0, 0.0, False, False), (5, 0, 0, 0.0, False, True)])
@pytest.mark.parametrize("variant", [0, 1, 2])
def test_attn_prefill_on_tcgen05(hd, H, Hkv, T, pos0, window, softcap, use_sinks, causal, variant):
    """The tcgen05 / TMEM / TMA flash-attention kernel (several query tiles, several key tiles, a chunk that continues a cached
    prefix) against the fp32 statement of attention over the same f16 cache; no bounded wait inside it may run out."""
    K = _K()
    n_slots, n_ctx, slot = 3, 1024, 2
    g = torch.Generator().manual_seed(hd + T)
    kc = (torch.randn(n_slots, Hkv, n_ctx, hd, generator=g) * 0.7).to(torch.float16).cuda()
    vc = (torch.randn(n_slots, Hkv, n_ctx, hd, generator=g) * 0.7).to(torch.float16).cuda()
    q = torch.randn(T, H, hd, generator=g).cuda()
    sinks = torch.randn(H, generator=g).cuda() if use_sinks else None
    scale = 1 / math.sqrt(hd)
    p_end = pos0 + T
    before = K.attn_prefill_tc_variant(variant)          # 1: probabilities stay in TMEM, 2: the pipelined kernel
    try:
        out = K.attn_prefill(q, kc, vc, slot, pos0, p_end, scale, causal, window, softcap, sinks, mode="tc").float().cpu().view(T, H, hd)
        torch.cuda.synchronize()
    finally:
        K.attn_prefill_tc_variant(before)
    assert K.attn_prefill_tc_status(clear=True) == 0
    qh = q.to(torch.float16).float().cpu()
    ref = R.attention(qh, kc[slot, :, :p_end].transpose(0, 1).float().cpu(), vc[slot, :, :p_end].transpose(0, 1).float().cpu(),
                      torch.arange(pos0, p_end), torch.arange(p_end), scale=scale, causal=causal, window=window, softcap=softcap,
                      sinks=sinks.cpu() if use_sinks else None)
    assert torch.allclose(out, ref, atol=1e-2, rtol=2e-2), (out - ref).abs().max()


@pytest.fixture
def attn_mode():
    """Selects the decode-attention kernel for one test and restores the automatic choice afterwards."""
    K = _K()
    yield K.attn_decode_mode
    K.attn_decode_mode(-1)


@pytest.mark.parametrize("hd,H,Hkv", [(128, 8, 2), (64, 6, 3), (256, 4, 2), (32, 8, 2)])
@pytest.mark.parametrize("mma", [0, 1])
def test_kv_cache_q8(hd, H, Hkv, mma, attn_mode):
    """q8_0 K/V cache: the rope kernel writes int8 blocks of 32 dims with an f16 scale; both attention kernels expand them.

    The written blocks are compared with the fp32 values (error within half a quantisation step), the attention
    kernels with fp32 attention over the dequantised cache.
    """
    K = _K()
    attn_mode(mma)
    n_slots, n_ctx, slot, T = 2, 192, 1, 150
    g = torch.Generator().manual_seed(hd)
    qkv = torch.randn(T, (H + 2 * Hkv) * hd, generator=g).cuda()
    pos = torch.arange(T, dtype=torch.int32).cuda()
    slots = torch.full((T,), slot, dtype=torch.int32).cuda()
    inv, _ = R.rope_inv_freq(hd, 10000.0, device="cuda")
    kc = torch.zeros(n_slots, Hkv, n_ctx, hd, device="cuda", dtype=torch.int8)
    vc = torch.zeros_like(kc)
    ks = torch.zeros(n_slots, Hkv, n_ctx, hd // 32, device="cuda", dtype=torch.float16)
    vs = torch.zeros_like(ks)
    q = K.rope_kv(qkv, pos, slots, inv, n_heads=H, n_kv_heads=Hkv, hd=hd, n_rot=hd, neox=True, mscale=1.0, k_cache=kc, v_cache=vc,
                  k_scale=ks, v_scale=vs)
    kr = R.rope(qkv[:, H * hd:(H + Hkv) * hd].view(T, Hkv, hd).cpu(), pos.cpu(), inv.cpu(), "neox", 1.0)
    vr = qkv[:, (H + Hkv) * hd:].view(T, Hkv, hd).cpu()

    def deq(c, s):
        return (c.float().view(*c.shape[:-1], hd // 32, 32) * s.float().unsqueeze(-1)).view(c.shape)

    kd, vd = deq(kc, ks).cpu(), deq(vc, vs).cpu()
    for got, want in ((kd[slot, :, :T].transpose(0, 1), kr), (vd[slot, :, :T].transpose(0, 1), vr)):
        step = want.view(T, Hkv, hd // 32, 32).abs().amax(-1, keepdim=True) / 127
        err = (got - want).view(T, Hkv, hd // 32, 32).abs()
        assert (err <= 0.51 * step + 2e-3 * want.abs().max()).all()
    assert kc[0].abs().max().item() == 0 and kc[slot, :, T:].abs().max().item() == 0      # nothing outside the written rows
    scale = 1 / math.sqrt(hd)
    # decode over the quantised cache
    dpos = torch.tensor([0, 77, T - 1], dtype=torch.int32).cuda()
    dslots = torch.full((3,), slot, dtype=torch.int32).cuda()
    qd = torch.randn(3, H, hd, generator=g).cuda()
    for n_splits in (1, 4):
        out, _ = K.attn_decode(qd, kc, vc, dpos, dslots, scale=scale, n_splits=n_splits, k_scale=ks, v_scale=vs)
        for b in range(3):
            p = int(dpos[b])
            ref = R.attention(qd[b:b + 1].to(torch.float16).float().cpu() if mma else qd[b:b + 1].cpu(), kd[slot, :, :p + 1].transpose(0, 1),
                              vd[slot, :, :p + 1].transpose(0, 1), torch.tensor([p]), torch.arange(p + 1), scale=scale)
            tol = dict(atol=1e-2, rtol=2e-2) if mma else dict(atol=2e-3, rtol=2e-3)
            assert torch.allclose(out[b].cpu(), ref.reshape(-1), **tol), (n_splits, b)
    # prefill over the quantised cache
    out = K.attn_prefill(q, kc, vc, slot, 0, T, scale, True, 0, 0.0, None, k_scale=ks, v_scale=vs).float().cpu().view(T, H, hd)
    ref = R.attention(q.to(torch.float16).float().cpu(), kd[slot, :, :T].transpose(0, 1), vd[slot, :, :T].transpose(0, 1),
                      torch.arange(T), torch.arange(T), scale=scale, causal=True)
    assert torch.allclose(out, ref, atol=1e-2, rtol=2e-2), (out - ref).abs().max()


@pytest.mark.parametrize("spec,ft", [("tiny-qwen3", "Q4_K_M"), ("tiny-gemma3", "Q8_0"), ("tiny-gpt-oss", "MXFP4")])
def test_engine_kv_cache_q8(tmp_path, spec, ft):
    """Whole model with the q8_0 K/V cache: logits stay close to the fp32 graph, the cache takes about half the bytes."""
    from ollama_b200.engine.b200 import B200Backend
    from ollama_b200.engine.backend import TorchBackend, open_model
    from ollama_b200.models.synth import write_synthetic_gguf
    p = str(tmp_path / "m.gguf")
    write_synthetic_gguf(p, spec, ft)
    g = open_model(p)
    ref, eng, f16 = TorchBackend(g, "cpu"), B200Backend(g, "cuda", kv_type="q8_0"), B200Backend(g, "cuda")
    for b in (ref, eng, f16):
        b.alloc(2, 64)
    if eng.cfg.head_dim not in _K().ATTN_PREFILL_HEAD_DIMS:
        assert eng.kv_type == "f16"
        return
    assert eng.kv_type == "q8_0" and eng.kv_bytes() < 0.6 * f16.kv_bytes()
    prompt = torch.randint(259, 4096, (20,), generator=torch.Generator().manual_seed(3)).tolist()
    lr = ref.prefill(1, prompt, 0)
    le = eng.prefill(1, prompt, 0).cpu()
    tol = 0.06 * lr.abs().max().item()
    assert (le - lr).abs().max().item() < tol
    tok = int(lr.argmax())
    for step in range(6):
        pos = len(prompt) + step
        lr = ref.decode([1], [tok], [pos])[0]
        le = eng.decode([1], [tok], [pos])[0].cpu()
        assert (le - lr).abs().max().item() < tol, step
        tok = int(lr.argmax())
    a = eng.decode_argmax([1], [tok], [len(prompt) + 6])
    assert a[0] == int(eng.decode([1], [tok], [len(prompt) + 6])[0].argmax())


@pytest.mark.parametrize("top_k,top_p,min_p,temp,penalties", [(40, 0.9, 0.0, 0.8, False), (1, 1.0, 0.0, 1.0, False), (256, 0.5, 0.05, 1.3, True),
                                                              (64, 1.0, 0.2, 0.7, True)])
def test_sample_kernel_matches_filter_chain(top_k, top_p, min_p, temp, penalties):
    """Device sampler: candidate set and probabilities equal the torch filter chain; the draw follows the inverse CDF."""
    K = _K()
    from ollama_b200.engine.sampler import Sampler, SamplingParams
    V, rows = 50257, 3
    g = torch.Generator().manual_seed(top_k)
    logits = (torch.randn(rows, V, generator=g) * 3).cuda()
    logits[1, 100:110] = logits[1].max() + 1.0              # equal values at the top: ties are taken lowest id first
    hist = [{5: 2, 77: 1, 40000: 3}, {}, {104: 1}] if penalties else None
    params = SamplingParams(temperature=temp, top_k=top_k, top_p=top_p, min_p=min_p, repeat_penalty=1.3 if penalties else 1.0,
                            frequency_penalty=0.2 if penalties else 0.0, presence_penalty=0.1 if penalties else 0.0, repeat_last_n=64)
    us = [0.0, 0.37, 0.999]
    ref_in = logits.clone()
    tok, prob, ci, cp, cn = K.sample(logits.clone(), us, top_k, top_p, min_p, temp, hist, params.repeat_penalty, params.frequency_penalty,
                                     params.presence_penalty, want_candidates=True)
    for r in range(rows):
        s = Sampler(params, V)
        s.history = [t for t, c in (hist[r] if hist else {}).items() for _ in range(c)]
        idx, probs = s.distribution(ref_in[r])
        n = int(cn[r])
        assert n == idx.numel(), (r, n, idx.numel())
        got_i, got_p = ci[r, :n].cpu().long(), cp[r, :n].cpu()
        assert torch.allclose(got_p, probs.cpu(), atol=1e-5, rtol=1e-4)
        same = got_i == idx.cpu()
        # equal logits may be ordered differently by torch.topk; everywhere else the ids agree
        assert bool((same | (got_p == probs.cpu())).all()) and set(got_i.tolist()) == set(idx.cpu().tolist())
        cdf = torch.cumsum(got_p, 0)
        want = int(torch.searchsorted(cdf, torch.tensor(us[r] * float(cdf[-1])), right=True).clamp(max=n - 1))
        assert int(tok[r]) == int(got_i[want]) and abs(float(prob[r]) - float(got_p[want])) < 1e-6
    if top_k >= 10 and not penalties:
        assert ci[1, :min(10, int(cn[1]))].tolist() == list(range(100, 110))[:min(10, int(cn[1]))]


def test_moe_route_kernel():
    K = _K()
    import ctypes as C
    T, E, k = 37, 128, 8
    logits = torch.randn(T, E, generator=torch.Generator().manual_seed(2)).cuda()
    for mode, router, norm in ((0, "softmax_topk", True), (0, "softmax_topk", False), (1, "topk_softmax", True)):
        ids = torch.zeros(T * k, dtype=torch.int32, device="cuda")
        lids, wts = torch.zeros_like(ids), torch.zeros(T * k, device="cuda")
        a = K.MoeRouteArgs(K.ptr(logits), E, E, k, mode, int(norm), 32, 64, K.ptr(ids), K.ptr(lids), K.ptr(wts))
        K._check(K.lib().b2_moe_route(C.byref(a), T, 0, K.stream()), "moe_route")
        rid, rw = R.moe_route(logits.cpu(), k, router, norm)
        assert torch.equal(ids.view(T, k).cpu().long(), rid)
        assert torch.allclose(wts.view(T, k).cpu(), rw, atol=1e-6, rtol=1e-5)
        exp_l = torch.where((rid >= 32) & (rid < 96), rid - 32, torch.full_like(rid, -1))
        assert torch.equal(lids.view(T, k).cpu().long(), exp_l)


@pytest.mark.parametrize("spec,ft", [("tiny-qwen3", "Q4_K_M"), ("tiny-gemma3", "Q8_0"), ("tiny-qwen2", "F16"), ("tiny-gemma2", "Q4_K_M"),
                                     ("tiny-qwen3moe", "Q4_K_M"), ("tiny-gpt-oss", "MXFP4"), ("tiny-mixtral", "Q8_0")])
def test_engine_matches_reference_graph(tmp_path, spec, ft, attn_mode):
    """Whole-model check: prefill logits and 6 decode steps of the sm_100a engine vs the fp32 reference graph."""
    from ollama_b200.engine.b200 import B200Backend
    from ollama_b200.engine.backend import TorchBackend, open_model
    from ollama_b200.models.synth import write_synthetic_gguf
    p = str(tmp_path / "m.gguf")
    write_synthetic_gguf(p, spec, ft)
    g = open_model(p)
    ref, eng = TorchBackend(g, "cpu"), B200Backend(g, "cuda")
    ref.alloc(2, 64)
    eng.alloc(2, 64)
    prompt = torch.randint(259, 4096, (20,), generator=torch.Generator().manual_seed(3)).tolist()
    lr = ref.prefill(1, prompt, 0)
    le = eng.prefill(1, prompt, 0).cpu()
    tol = 0.05 * lr.abs().max().item()
    assert (le - lr).abs().max().item() < tol
    tok = int(lr.argmax())
    for step in range(6):
        pos = len(prompt) + step
        lr = ref.decode([1], [tok], [pos])[0]
        le = eng.decode([1], [tok], [pos])[0].cpu()
        assert (le - lr).abs().max().item() < tol, step
        tok = int(lr.argmax())
    # graph replay path returns the same tokens as the eager path
    a = eng.decode_argmax([1], [tok], [len(prompt) + 6])
    eng2 = eng.decode([1], [tok], [len(prompt) + 6])
    assert a[0] == int(eng2[0].argmax())
    # the single-launch attention (last CTA of a head group merges the splits) gives the same logits as the two-launch
    # form with the same (scalar) inner loop
    attn_mode(0)
    eng.use_graphs = False
    eng2 = eng.decode([1], [tok], [len(prompt) + 6])
    eng.fuse_attn_combine = True
    eng3 = eng.decode([1], [tok], [len(prompt) + 6])
    assert torch.allclose(eng3, eng2, atol=1e-4 * eng2.abs().max().item() + 1e-5)


@pytest.mark.parametrize("t", [GGMLType.Q4_K, GGMLType.Q6_K, GGMLType.Q8_0, GGMLType.BF16])
@pytest.mark.parametrize("nb", [1, 2, 4, 8])
def test_gemv_model_shapes(t, nb):
    """Shapes of an 8B model: exercises the row-length split across warps (small n) and long rows."""
    K = _K()
    for n, k in ((4096, 4096), (1024, 14336), (20000, 1024)):
        qw, bias = _weight(t, n, k, bias=True)
        dw = K.repack(qw, "cuda", bias=bias)
        x = torch.randn(nb, k, generator=torch.Generator().manual_seed(nb)).cuda()
        act = K.rmsnorm_quant(x, None, 0.0, do_norm=False)
        y = K.gemv([dw], act)
        wf = qw.dequant()
        xr = _quant_act_ref(x.cpu()) if dw.quant_input else x.cpu()
        ref = xr @ wf.t() + bias
        assert torch.allclose(y.cpu(), ref, atol=2e-3 * ref.abs().max().item(), rtol=1e-3)


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 128, 512), (512, 4096, 4096), (300, 200, 1000), (64, 64, 72), (1, 1024, 4096)])
def test_gemm_bf16_tensor_core(m, n, k):
    """tcgen05 GEMM against an fp32 matmul of the same bf16 operands."""
    K = _K()
    g = torch.Generator().manual_seed(m + n + k)
    a = (torch.randn(m, k, generator=g) * 0.5).to(torch.bfloat16).cuda()
    b = (torch.randn(n, k, generator=g) * 0.5).to(torch.bfloat16).cuda()
    bias = torch.randn(n, generator=g).cuda()
    ref = a.float() @ b.float().t() + bias
    out = K.gemm_bf16(a, b, bias)
    torch.cuda.synchronize()
    assert K.gemm_status() == 0
    assert torch.allclose(out, ref, atol=1e-2 + 1e-3 * ref.abs().max().item(), rtol=1e-3), (out - ref).abs().max()
    acc = torch.ones(m, n, device="cuda")
    K.gemm_bf16(a, b, None, out=acc, accumulate=True)
    assert torch.allclose(acc, ref - bias + 1, atol=1e-2 + 1e-3 * ref.abs().max().item(), rtol=1e-3)


@pytest.mark.parametrize("m,n,k", [(4, 5120, 2880), (8, 2880, 4096), (16, 20480, 512), (32, 192, 64)])
def test_gemm_bf16_of_a_decode_step(m, n, k):
    """A handful of rows against a wide 16-bit matrix (narrow tiles over many SMs), written into a strided slice of a wider buffer."""
    K = _K()
    g = torch.Generator().manual_seed(m + n + k)
    a = (torch.randn(m, k, generator=g) * 0.5).to(torch.bfloat16).cuda()
    b = (torch.randn(n, k, generator=g) * 0.5).to(torch.bfloat16).cuda()
    bias = torch.randn(n, generator=g).cuda()
    ref = a.float() @ b.float().t() + bias
    wide = torch.full((m + 3, n + 64), 7.0, device="cuda")
    K.gemm_bf16(a, b, bias, out=wide[:m, 32:32 + n])
    torch.cuda.synchronize()
    assert K.gemm_status() == 0
    assert torch.allclose(wide[:m, 32:32 + n], ref, atol=1e-2 + 1e-3 * ref.abs().max().item(), rtol=1e-3)
    assert (wide[m:] == 7).all() and (wide[:, :32] == 7).all() and (wide[:, 32 + n:] == 7).all()


@pytest.mark.parametrize("spec,ft,nb", [("tiny-gpt-oss", "MXFP4", 6), ("tiny-gpt-oss", "MXFP4", 12), ("tiny-qwen2", "BF16", 6), ("tiny-gemma3", "F16", 6)])
def test_engine_decode_steps_of_several_sequences_on_the_gemm(tmp_path, spec, ft, nb):
    """Several sequences per step: the 16-bit matrices of the step (attention projections, LM head) on the tcgen05 GEMM give the
    logits of the GEMV route and of the fp32 graph, eagerly and from the recorded graph.  A model of expert layers only, with
    16-bit dense matrices, takes more than eight sequences in one step (the GEMV route then runs eight rows per launch)."""
    from ollama_b200.engine.b200 import B200Backend
    from ollama_b200.engine.backend import TorchBackend, open_model
    from ollama_b200.models.synth import write_synthetic_gguf
    p = str(tmp_path / "m.gguf")
    write_synthetic_gguf(p, spec, ft)
    g = open_model(p)
    ref, eng = TorchBackend(g, "cpu"), B200Backend(g, "cuda")
    assert eng.tc_decode_min == 4
    assert eng.max_batch == (32 if spec == "tiny-gpt-oss" else 8)
    ref.alloc(nb, 64)
    eng.alloc(nb, 64)
    gen = torch.Generator().manual_seed(11)
    prompts = [torch.randint(259, 4096, (5 + 2 * i,), generator=gen).tolist() for i in range(nb)]
    toks = []
    for i, pr in enumerate(prompts):
        lr = ref.prefill(i, pr, 0)
        eng.prefill(i, pr, 0)
        toks.append(int(lr.argmax()))
    slots, pos = list(range(nb)), [len(pr) for pr in prompts]
    lr = ref.decode(slots, toks, pos)
    tol = 0.05 * lr.abs().max().item()
    n0 = eng.kernel_launches
    eng.use_graphs = False
    le = eng.decode(slots, toks, pos).cpu()                 # GEMM route, eager (same positions again: the cache rows are rewritten)
    assert (le - lr).abs().max().item() < tol and K_status_ok()
    eng.tc_decode_min = 0
    lv = eng.decode(slots, toks, pos).cpu()                 # GEMV route
    assert (lv - lr).abs().max().item() < tol
    assert (le - lv).abs().max().item() < 0.02 * lr.abs().max().item()
    eng.tc_decode_min, eng.use_graphs = 4, True
    for _ in range(3):                                      # warm-up, capture, replay
        lg = eng.decode(slots, toks, pos).cpu()
    assert torch.allclose(lg, le, atol=1e-3 * lr.abs().max().item())
    assert K_status_ok() and eng.kernel_launches > n0
    eng.close()


@pytest.mark.parametrize("mode,keep", [("fused", False), ("bf16", False), ("bf16", True)])
def test_engine_prefill_gemm_modes(tmp_path, mode, keep):
    """Prefill logits agree with the fp32 graph whichever way the weights reach the tensor cores."""
    from ollama_b200.engine.b200 import B200Backend
    from ollama_b200.engine.backend import TorchBackend, open_model
    from ollama_b200.models.synth import write_synthetic_gguf
    p = str(tmp_path / "m.gguf")
    write_synthetic_gguf(p, "tiny-qwen3", "Q4_K_M")
    g = open_model(p)
    ref, eng = TorchBackend(g, "cpu"), B200Backend(g, "cuda", keep_bf16=keep, prefill_gemm=mode)
    ref.alloc(1, 256)
    eng.alloc(1, 256)
    prompt = torch.randint(259, 4096, (150,), generator=torch.Generator().manual_seed(5)).tolist()
    lr = ref.prefill(0, prompt, 0)
    le = eng.prefill(0, prompt, 0).cpu()
    assert (le - lr).abs().max().item() < 0.05 * lr.abs().max().item()
    assert K_status_ok()


@pytest.mark.parametrize("stream_q", ["1", "0"])
def test_engine_moe_prefill_on_mxfp4_experts(tmp_path, monkeypatch, stream_q):
    """gpt-oss prefill without a resident 16-bit copy of the experts: the grouped kernel that streams the MXFP4 blocks (and, with
    the switch off, the expand-per-chunk path) agree with the fp32 graph."""
    from ollama_b200.engine.b200 import B200Backend
    from ollama_b200.engine.backend import TorchBackend, open_model
    from ollama_b200.models.synth import write_synthetic_gguf
    monkeypatch.setenv("B200_MOE_STREAM_Q", stream_q)
    p = str(tmp_path / "m.gguf")
    write_synthetic_gguf(p, "tiny-gpt-oss", "MXFP4")
    g = open_model(p)
    ref, eng = TorchBackend(g, "cpu"), B200Backend(g, "cuda", keep_bf16=False)
    assert eng.moe_stream_q == (stream_q == "1")
    ref.alloc(1, 256)
    eng.alloc(1, 256)
    prompt = torch.randint(259, 4096, (150,), generator=torch.Generator().manual_seed(5)).tolist()
    lr = ref.prefill(0, prompt, 0)
    n0 = eng.kernel_launches
    le = eng.prefill(0, prompt, 0).cpu()
    assert (le - lr).abs().max().item() < 0.05 * lr.abs().max().item()
    assert K_status_ok() and eng.kernel_launches > n0
    eng.close()


def K_status_ok() -> bool:
    return _K().gemm_status() == 0


@pytest.mark.parametrize("t", [GGMLType.Q4_K, GGMLType.Q6_K, GGMLType.Q8_0, GGMLType.BF16, GGMLType.F16])
@pytest.mark.parametrize("m,n,k", [(128, 128, 256), (512, 1024, 4096), (77, 200, 512), (1, 128, 1024)])
def test_gemm_q_dequant_fused(t, m, n, k):
    """Dequant-fused tcgen05 GEMM: the reference multiplies the same bf16 activations with the bf16-rounded decoded weights."""
    K = _K()
    qw, bias = _weight(t, n, k, seed=m + n, bias=True)
    dw = K.repack(qw, "cuda", bias=bias)
    x = (torch.randn(m, k, generator=torch.Generator().manual_seed(k)) * 0.5).to(torch.bfloat16).cuda()
    ref = x.float().cpu() @ qw.dequant().to(torch.bfloat16).float().t() + bias
    out = torch.zeros(m, n + 8, device="cuda")
    K.gemm_q(x, dw, out=out, out_off=4)
    torch.cuda.synchronize()
    assert K.gemm_status() == 0
    # block scales / minima of the K-quants are rounded to bf16 inside the kernel (the expansion runs in packed bf16 arithmetic)
    tol = 1e-3 + (6e-3 if t in (GGMLType.Q4_K, GGMLType.Q6_K) else 2e-3) * ref.abs().max().item()
    assert torch.allclose(out[:, 4:4 + n].cpu(), ref, atol=tol, rtol=2e-3), (out[:, 4:4 + n].cpu() - ref).abs().max()
    assert out[:, :4].abs().max() == 0 and out[:, 4 + n:].abs().max() == 0      # neighbours of the output window stay untouched
    K.gemm_q(x, dw, out=out, accumulate=True, out_off=4)
    assert torch.allclose(out[:, 4:4 + n].cpu(), 2 * ref, atol=2 * tol, rtol=2e-3)


def test_bounded_waits_report_a_missing_rank():
    """Failure detection on the device without a fault: a wait for a rank that never writes gives up after the channel's
    time limit, records a status that the host reads, and leaves the context usable."""
    import ctypes as C
    import time

    from ollama_b200.parallel.comm import CHAN_BYTES, Layout, PeerRegion
    from ollama_b200.parallel.transport import LocalTransport
    K = _K()
    lay = Layout()
    k = 512
    blk = lay.add("parts", 2 * 2 * 8 * k * 8)                 # two halves x two ranks x eight rows of (value, epoch) pairs
    reg = PeerRegion(lay.size, 0, 1, "cuda", LocalTransport())
    try:
        for ch in (0, 1):
            reg.set_wait_ms(ch, 200)
        # 1. flag wait: two ranks expected at epoch 5; rank 0 has announced it, nobody ever raises flag 1
        from ollama_b200.parallel.comm import tensor_at
        tensor_at(reg.chan(1) + 4, (1,), torch.int32, reg.device).fill_(5)          # this rank's epoch
        tensor_at(reg.chan(1) + 32, (1,), torch.int32, reg.device).fill_(5)         # flag[0]
        torch.cuda.synchronize()
        t0 = time.time()
        reg.world = 2
        reg.wait(1)
        torch.cuda.synchronize()
        reg.world = 1
        assert 0.15 < time.time() - t0 < 5.0
        assert reg.failed_channels() == [1] and reg.status(1) == 1
        reg.clear_status(1)
        assert reg.failed_channels() == []
        # 2. low-latency reduce: rank 0's partial row is there (epoch 1), rank 1's never arrives
        parts = reg.tensor(blk, (2, 2, 8, k, 2), torch.int32)
        parts.zero_()
        vals = torch.randn(k, device="cuda")
        half = 1                                               # epoch 1 uses the odd half
        parts[half, 0, 0, :, 0] = vals.view(torch.int32)
        parts[half, 0, 0, :, 1] = 1
        x = torch.ones(1, k, device="cuda")
        xq = torch.empty(1, k, dtype=torch.int8, device="cuda")
        xds = torch.empty(1, k // 32, 2, device="cuda")
        xf = torch.empty(1, k, device="cuda")
        a = K.NormQuantArgs(K.ptr(x), None, 1e-5, k, 0, K.ptr(xq), K.ptr(xds), K.ptr(xf), None)
        a.parts, a.n_part, a.part_stride, a.parity_stride, a.chan = reg.addr(blk), 2, 8 * k, 2 * 8 * k, reg.chan(0)
        t0 = time.time()
        K._check(K.lib().b2_rmsnorm_quant(C.byref(a), 1, 0, K.stream()), "rmsnorm_quant")
        torch.cuda.synchronize()
        assert 0.15 < time.time() - t0 < 5.0
        assert reg.failed_channels() == [0]
        assert torch.allclose(x[0], 1.0 + vals, atol=1e-6)     # the rank that did arrive was added; the missing one contributed zeros
        # the context is intact: an ordinary kernel still runs
        assert float(K.rmsnorm_quant(torch.ones(1, 64, device="cuda"), None, 1e-5).f.sum()) == pytest.approx(64.0, rel=1e-4)
    finally:
        reg.clear_status(0)
        reg.close()


@pytest.mark.parametrize("spec", ["tiny-qwen3", "tiny-gpt-oss"])
def test_prefill_of_several_sequences_in_one_pass(tmp_path, spec):
    """Chunks of three sequences (two of them continuing an earlier chunk) through one set of GEMMs: the logits after each
    chunk and the next decode step equal those of the same chunks run one sequence at a time."""
    from ollama_b200.engine.b200 import B200Backend
    from ollama_b200.engine.backend import open_model
    from ollama_b200.models.synth import write_synthetic_gguf
    p = str(tmp_path / "m.gguf")
    write_synthetic_gguf(p, spec, "Q8_0")
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(259, 4096, (n,), generator=g).tolist() for n in (70, 33, 150)]
    first = [30, 0, 100]                              # rows already in the cache before the shared pass
    one, many = B200Backend(open_model(p), "cuda"), B200Backend(open_model(p), "cuda")
    for e in (one, many):
        e.alloc(3, 256)
        for slot, (toks, n0) in enumerate(zip(prompts, first)):
            if n0:
                e.prefill(slot, toks[:n0], 0, need_logits=False)
    want = [one.prefill(slot, toks[n0:], n0) for slot, (toks, n0) in enumerate(zip(prompts, first))]
    got = many.prefill_many([(slot, toks[n0:], n0) for slot, (toks, n0) in enumerate(zip(prompts, first))], [True, False, True])
    assert got[1] is None
    for i in (0, 2):
        assert (got[i] - want[i]).abs().max().item() < 5e-3 * want[i].abs().max().item() + 1e-4, i
    step = lambda e: e.decode([0, 1, 2], [5, 6, 7], [len(t) for t in prompts])       # noqa: E731
    a, b = step(one), step(many)
    assert (a - b).abs().max().item() < 5e-3 * a.abs().max().item() + 1e-4
    one.close()
    many.close()


@pytest.mark.parametrize("spec,kv_type", [("tiny-gemma3", "f16"), ("tiny-qwen3", "q8_0")])
def test_prefill_with_image_rows_on_the_engine(tmp_path, spec, kv_type):
    """Rows of a prompt whose input is a given embedding (an image's projected features) and whose positions attend to each
    other in both directions: the engine's logits, and the decode step after them, follow the fp32 graph's; the same prompt
    without the two-way span gives different logits."""
    from ollama_b200.engine.b200 import B200Backend
    from ollama_b200.engine.backend import TorchBackend, open_model
    from ollama_b200.models.synth import write_synthetic_gguf
    p = str(tmp_path / "m.gguf")
    write_synthetic_gguf(p, spec, "F16")
    ref, eng = TorchBackend(open_model(p), "cpu"), B200Backend(open_model(p), "cuda", kv_type=kv_type)
    g = torch.Generator().manual_seed(4)
    toks = torch.randint(259, 4096, (60,), generator=g).tolist()
    rows = list(range(20, 36))
    for r in rows:
        toks[r] = -(1 + r)
    emb = torch.randn(len(rows), ref.cfg.d_model, generator=g) * 0.5
    spans = [(20, 36)]
    for e in (ref, eng):
        e.alloc(1, 128)
    a = ref.prefill(0, toks, 0, embeds=(rows, emb), spans=spans)
    b = eng.prefill(0, toks, 0, embeds=(rows, emb.cuda()), spans=spans).float().cpu()
    tol = 0.05 * a.abs().max().item()
    assert (a - b).abs().max().item() < tol
    a1, b1 = ref.decode([0], [7], [60])[0], eng.decode([0], [7], [60])[0].float().cpu()
    assert (a1 - b1).abs().max().item() < 0.05 * a1.abs().max().item()
    # in two chunks, the second one starting inside the prompt but after the image: the cached image rows are used as they are
    eng.prefill(0, toks[:40], 0, need_logits=False, embeds=(rows, emb.cuda()), spans=spans)
    c = eng.prefill(0, toks[40:], 40, spans=spans).float().cpu()
    assert (a - c).abs().max().item() < tol
    eng.close()


def test_phi3_checkpoint_with_fused_matrices_on_the_engine(tmp_path):
    """A converted Phi-3 checkpoint (Q | K | V and gate | up stored fused, long-context rotary factors and attention factor)
    runs on the sm_100a engine through row-range views of the fused tensors and agrees with the fp32 graph."""
    transformers = pytest.importorskip("transformers")
    from test_convert import _tiny_tokenizer
    from ollama_b200.convert.hf import convert_hf
    from ollama_b200.engine.b200 import B200Backend
    from ollama_b200.engine.backend import TorchBackend, open_model
    from ollama_b200.store.create import quantize_gguf
    torch.manual_seed(0)
    g = torch.Generator().manual_seed(3)
    cfg = transformers.Phi3Config(vocab_size=64, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                                  num_key_value_heads=2, rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False, pad_token_id=0,
                                  max_position_embeddings=512, original_max_position_embeddings=64,
                                  rope_scaling={"type": "longrope", "long_factor": (1 + 3 * torch.rand(32, generator=g)).tolist(),
                                                "short_factor": (1 + 0.2 * torch.rand(32, generator=g)).tolist()})
    src = tmp_path / "hf"
    transformers.Phi3ForCausalLM(cfg).float().save_pretrained(src, safe_serialization=True)
    _tiny_tokenizer(str(src))
    f16, q8 = str(tmp_path / "m.gguf"), str(tmp_path / "q.gguf")
    convert_hf(str(src), f16, outtype="f16")
    quantize_gguf(f16, q8, "q8_0")
    ids = torch.randint(0, 64, (90,), generator=torch.Generator().manual_seed(1)).tolist()
    for path in (f16, q8):
        ref, eng = TorchBackend(open_model(path), "cpu"), B200Backend(open_model(path), "cuda")
        assert eng.cfg.arch == "phi3" and eng.mscale > 1.0
        for e in (ref, eng):
            e.alloc(1, 128)
        a, b = ref.prefill(0, ids, 0), eng.prefill(0, ids, 0).float().cpu()
        assert (a - b).abs().max().item() < 0.05 * a.abs().max().item()
        a, b = ref.decode([0], [7], [90])[0], eng.decode([0], [7], [90])[0].float().cpu()
        assert (a - b).abs().max().item() < 0.05 * a.abs().max().item()
        eng.close()


@pytest.mark.parametrize("kv_type,spec", [("f16", "tiny-tp"), ("q8_0", "tiny-qwen3"), ("f16", "tiny-gemma3")])
def test_context_shift_on_the_engine_cache(tmp_path, kv_type, spec):
    """Rows [keep, keep + discard) leave a slot: afterwards the engine's cache holds what the fp32 graph's cache holds after
    the same shift (keys re-rotated, values moved), and the next decode step agrees with the fp32 graph's."""
    from ollama_b200.engine.b200 import B200Backend
    from ollama_b200.engine.backend import TorchBackend, open_model
    from ollama_b200.models.synth import write_synthetic_gguf
    p = str(tmp_path / "m.gguf")
    write_synthetic_gguf(p, spec, "F16")
    ref, eng = TorchBackend(open_model(p), "cpu"), B200Backend(open_model(p), "cuda", kv_type=kv_type)
    toks = torch.randint(259, 4096, (90,), generator=torch.Generator().manual_seed(3)).tolist()
    keep, discard, n = 5, 40, 90
    for e in (ref, eng):
        e.alloc(1, 128)
        e.prefill(0, toks, 0)
        e.shift(0, keep, discard, n)
    tol = 0.03          # prefill runs bf16 GEMMs: a key of the second layer is a percent off; a wrong rotation is off by its own size
    for i in range(ref.cfg.n_layers):
        k = eng.k_cache[i][0, :, :n - discard].float()
        v = eng.v_cache[i][0, :, :n - discard].float()
        if eng.k_scale[i] is not None:
            k = (k.view(*k.shape[:2], -1, 32) * eng.k_scale[i][0, :, :n - discard].float()[..., None]).view_as(k)
            v = (v.view(*v.shape[:2], -1, 32) * eng.v_scale[i][0, :, :n - discard].float()[..., None]).view_as(v)
        rk, rv = ref.cache.k[i][0, :n - discard].transpose(0, 1), ref.cache.v[i][0, :n - discard].transpose(0, 1)
        assert (k.cpu() - rk).abs().max().item() < tol * rk.abs().max().item(), i
        assert (v.cpu() - rv).abs().max().item() < tol * rv.abs().max().item(), i
    a = ref.decode([0], [toks[-1]], [n - discard])[0]
    b = eng.decode([0], [toks[-1]], [n - discard])[0].float().cpu()
    assert (a - b).abs().max().item() < 0.05 * a.abs().max().item()
    eng.close()


def test_verify_pass_and_speculative_decoding_on_the_engine(tmp_path):
    """The target pass of speculative decoding on the sm_100a engine: ``verify`` gives the logits of one-by-one decoding
    for every drafted position, and a runner with a draft model produces the tokens of the plain greedy run."""
    from ollama_b200.engine.b200 import B200Backend
    from ollama_b200.engine.backend import open_model
    from ollama_b200.engine.runner import CompletionRequest, Runner, RunnerOptions
    from ollama_b200.engine.sampler import SamplingParams
    from ollama_b200.models.synth import write_synthetic_gguf
    p, pd = str(tmp_path / "m.gguf"), str(tmp_path / "d.gguf")
    write_synthetic_gguf(p, "tiny-qwen3", "Q8_0")
    write_synthetic_gguf(pd, "tiny-qwen3", "Q4_K_M")             # the same weights, coarser: agrees most of the time
    eng = B200Backend(open_model(p), "cuda")
    eng.alloc(1, 128)
    prompt = torch.randint(259, 4096, (24,), generator=torch.Generator().manual_seed(7)).tolist()
    eng.prefill(0, prompt[:20], 0, need_logits=False)
    all_logits = eng.verify(0, prompt[20:], 20)
    assert all_logits.shape == (4, eng.cfg.vocab_size)
    eng.prefill(0, prompt[:20], 0, need_logits=False)
    for i, tok in enumerate(prompt[20:]):
        step = eng.decode([0], [tok], [20 + i])[0]
        assert (step - all_logits[i]).abs().max().item() < 0.03 * step.abs().max().item(), i
    eng.close()
    outs = []
    for draft in ("", pd):
        r = Runner(p, RunnerOptions(num_ctx=256, device="cuda", draft_path=draft, draft_num_predict=4))
        try:
            out = list(r.completion(CompletionRequest(prompt=prompt, sampling=SamplingParams(temperature=0), num_predict=40, ignore_eos=True)))
            outs.append([t for c in out for t in c.tokens])
            if draft:
                assert r.stats["draft_accepted_tokens"] > 0 and r.stats["decode_steps"] < 39
        finally:
            r.close()
    # the verification pass runs the prefill kernels (bf16 tensor-core GEMMs), the plain run the decode kernels: the
    # greedy paths agree until a near-tie between two logits
    same = next((i for i, (a, b) in enumerate(zip(*outs)) if a != b), 40)
    assert len(outs[0]) == len(outs[1]) == 40 and same >= 8


def test_engine_with_a_lora_adapter(tmp_path):
    """LoRA adapters merged at load: the sm_100a engine (merged matrices as F16 next to quantised ones, mixed gate / up
    encodings included) against the fp32 graph with the same adapter."""
    from ollama_b200.engine.backend import TorchBackend, make_backend, open_model
    from ollama_b200.gguf.types import GGMLType
    from ollama_b200.gguf.writer import WriteTensor, write_gguf
    from ollama_b200.models.synth import write_synthetic_gguf
    p, ad = str(tmp_path / "m.gguf"), str(tmp_path / "a.gguf")
    write_synthetic_gguf(p, "tiny-qwen3", "Q4_K_M")
    g = open_model(p)
    gen = torch.Generator().manual_seed(0)
    tensors = []
    for n in ("blk.0.attn_q.weight", "blk.0.ffn_gate.weight", "blk.1.attn_output.weight", "blk.1.ffn_down.weight"):
        out_dim, in_dim = g.tensors[n].torch_shape
        a, b = torch.randn(4, in_dim, generator=gen) * 0.05, torch.randn(out_dim, 4, generator=gen) * 0.05
        tensors += [WriteTensor(n + ".lora_a", (in_dim, 4), GGMLType.F32, a.numpy().tobytes()),
                    WriteTensor(n + ".lora_b", (4, out_dim), GGMLType.F32, b.numpy().tobytes())]
    write_gguf(ad, {"general.architecture": "qwen3", "general.type": "adapter", "adapter.type": "lora", "adapter.lora.alpha": 8.0}, tensors)
    ref, base, eng = TorchBackend(g, "cpu", adapters=[ad]), TorchBackend(g, "cpu"), make_backend(g, "cuda", adapters=[ad])
    assert eng.name == "b200"
    for b in (ref, base, eng):
        b.alloc(1, 64)
    prompt = torch.randint(259, 4096, (20,), generator=torch.Generator().manual_seed(3)).tolist()
    lr, lb, le = ref.prefill(0, prompt, 0), base.prefill(0, prompt, 0), eng.prefill(0, prompt, 0).cpu()
    tol = 0.05 * lr.abs().max().item()
    assert (le - lr).abs().max().item() < tol and (lb - lr).abs().max().item() > 0.01 * lr.abs().max().item()
    tok = int(lr.argmax())
    for step in range(4):
        lr = ref.decode([0], [tok], [20 + step])[0]
        le = eng.decode([0], [tok], [20 + step])[0].cpu()
        assert (le - lr).abs().max().item() < tol, step
        tok = int(lr.argmax())


@pytest.mark.parametrize("glu", [None, "silu", "swiglu_oai"])
def test_grouped_gemm_and_moe_plan(glu):
    """One grouped tensor-core launch over 128 experts (top-4 routing of 300 tokens) against a per-expert fp32 loop."""
    K = _K()
    g = torch.Generator().manual_seed(11)
    T, k, E, d, n = 300, 4, 128, 320, 256
    lids = torch.randint(-1, E, (T * k,), generator=g).to(torch.int32)
    lids[5] = -1
    h = (torch.randn(T, d, generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(E * n, d, generator=g) * 0.1).to(torch.bfloat16)
    bias = torch.randn(E * n, generator=g) * 0.1
    row, te, rows = K.moe_plan(lids.cuda(), E)
    row_c, te_c = row.cpu(), te.cpu()
    used = row_c[lids >= 0]
    assert (row_c[lids < 0] == -1).all() and used.min() >= 0 and used.unique().numel() == used.numel()
    assert (te_c[(used // 128).long()] == lids[lids >= 0]).all()          # every pair sits in a tile of its own expert
    xs = K.moe_gather(h.cuda(), row, k, rows)
    out = K.gemm_bf16_grouped(xs, w.cuda(), E, te, bias.cuda(), glu=glu).cpu().float()
    for p in torch.randperm(T * k, generator=g)[:200].tolist():
        e = int(lids[p])
        if e < 0:
            continue
        y = h[p // k].float() @ w[e * n:(e + 1) * n].float().t() + bias[e * n:(e + 1) * n]
        ref = R.glu(y[0::2], y[1::2], glu) if glu else y
        got = out[int(row_c[p])]
        assert torch.allclose(got, ref, atol=3e-2 * ref.abs().max().item() + 1e-3, rtol=2e-2), (p, (got - ref).abs().max())
    if glu is None:
        wts = torch.rand(T * k, generator=g)
        comb = K.moe_scatter_combine(out.cuda(), row, wts.cuda(), T, k).cpu()
        ref = torch.zeros(T, n)
        for p in range(T * k):
            if lids[p] >= 0:
                ref[p // k] += wts[p] * out[int(row_c[p])]
        assert torch.allclose(comb, ref, atol=1e-4, rtol=1e-4)
    assert K.gemm_status() == 0


@pytest.mark.parametrize("glu", [None, "swiglu_oai"])
@pytest.mark.parametrize("E,n,k,T", [(8, 256, 320, 300), (32, 192, 2880, 500), (4, 2880 // 4 * 2, 512, 1100)])
def test_grouped_gemm_over_mxfp4_experts(glu, E, n, k, T):
    """The grouped kernel that streams MXFP4 expert blocks and expands them itself, against the product with the dequantised
    experts: partial N tiles, experts with no row, experts with several tiles, bias, gated epilogue."""
    K = _K()
    g = torch.Generator().manual_seed(E + n)
    topk = 2
    lids = torch.randint(-1, E, (T * topk,), generator=g).to(torch.int32)
    lids[lids == 1] = 0                                           # expert 1 gets no row, expert 0 twice the share
    h = (torch.randn(T, k, generator=g) * 0.5).to(torch.bfloat16)
    qw = QWeight.from_float("w", torch.randn(E, n, k, generator=g) * 0.05, GGMLType.MXFP4)
    if E == 8:          # block scales from 2^-9 to 2^7: both ways of applying them, and codes of every magnitude next to each other
        blocks = qw.raw.view(-1, 17)
        blocks[:, 0] = torch.randint(118, 135, (blocks.shape[0],), generator=g).to(torch.uint8)
        h = h * 0.02
    bias = torch.randn(E * n, generator=g) * 0.1
    dw = K.repack(qw, "cuda", bias=bias)
    assert dw.experts == E and K.gemm_q_grouped_supported(dw)
    row, te, rows = K.moe_plan(lids.cuda(), E)
    xs = K.moe_gather(h.cuda(), row, topk, rows)
    out = K.gemm_q_grouped(xs, dw, te, glu=glu)
    assert out is not None
    torch.cuda.synchronize()
    assert K.gemm_status() == 0
    out, row_c = out.cpu().float(), row.cpu()
    wf = qw.dequant().view(E, n, k)
    for p in torch.randperm(T * topk, generator=g)[:150].tolist():
        e = int(lids[p])
        if e < 0:
            continue
        y = h[p // topk].float() @ wf[e].t() + bias[e * n:(e + 1) * n]
        ref = R.glu(y[0::2], y[1::2], glu) if glu else y
        got = out[int(row_c[p])]
        assert torch.allclose(got, ref, atol=2e-2 * ref.abs().max().item() + 1e-3, rtol=2e-2), (p, e, (got - ref).abs().max())


def test_dense_gemm_with_gated_epilogue():
    K = _K()
    g = torch.Generator().manual_seed(12)
    a = (torch.randn(200, 512, generator=g) * 0.5).to(torch.bfloat16)
    b = (torch.randn(1024, 512, generator=g) * 0.05).to(torch.bfloat16)
    bias = torch.randn(1024, generator=g) * 0.1
    y = a.float() @ b.float().t() + bias
    for act in ("silu", "gelu_tanh", "swiglu_oai"):
        got = K.gemm_bf16_glu(a.cuda(), b.cuda(), act, bias.cuda()).cpu().float()
        ref = R.glu(y[:, 0::2], y[:, 1::2], act)
        assert torch.allclose(got, ref, atol=2e-2 * ref.abs().max().item(), rtol=2e-2), act
