"""The streaming tensor-core decode GEMV (kernels/gemv_sk.cu) against plain PyTorch fp32 statements."""
import pytest
import torch

from ollama_b200.gguf.types import GGMLType
from ollama_b200.models.weights import QWeight
from ollama_b200.ops import reference as R

pytestmark = pytest.mark.gpu


def _mods():
    from ollama_b200.ops import cuda as K
    from ollama_b200.ops import sk
    return K, sk


def _qw(t, n, k, seed):
    g = torch.Generator().manual_seed(seed)
    return QWeight.from_float("w", torch.randn(n, k, generator=g) * 0.05, t)


def _quant256_ref(x):
    """int8 with one scale per 256 elements, as the kernels quantise activations; returns the de-quantised values."""
    xb = x.view(x.shape[0], -1, 256)
    amax = xb.abs().amax(-1, keepdim=True)
    inv = torch.where(amax > 0, 127.0 / amax.clamp_min(1e-30), torch.zeros_like(amax))
    return (torch.round(xb * inv) * (amax / 127.0)).view_as(x)


def _close(y, ref, tol=2e-3):
    return torch.allclose(y, ref, atol=tol * ref.abs().max().item(), rtol=1e-3)


def test_quant256_matches_reference():
    K, sk = _mods()
    x = torch.randn(5, 1024, generator=torch.Generator().manual_seed(3)) * 2
    w = torch.rand(1024) + 0.5
    xq, xd, xbs = sk.quant256(x.cuda(), w.cuda(), 1e-5)
    assert torch.equal(xbs.cpu().int(), xq.cpu().int().view(5, -1, 32).sum(-1))
    ref = _quant256_ref(R.rmsnorm(x, w, 1e-5))
    got = (xq.cpu().float().view(5, -1, 256) * xd.cpu()[..., None]).view(5, 1024)
    assert torch.allclose(got, ref, atol=2e-2 * ref.abs().max().item() / 127 + 1e-6)
    # a single row comes in the word order of the one-token kernel
    xq1, xd1, xbs1 = sk.quant256(x[:1].cuda(), w.cuda(), 1e-5)
    assert torch.equal(sk.natural_order(xq1).cpu(), xq[:1].cpu()) and torch.equal(xbs1.cpu(), xbs[:1].cpu())


@pytest.mark.parametrize("t", [GGMLType.Q4_K, GGMLType.Q6_K])
@pytest.mark.parametrize("nb", [1, 3, 8, 13, 32])
@pytest.mark.parametrize("ctas", [0, 1, 5])
def test_gemv_sk_matches_reference(t, nb, ctas):
    K, sk = _mods()
    n, k = 208, 1024
    qw = _qw(t, n, k, 11)
    bias = torch.randn(n, generator=torch.Generator().manual_seed(2)) * 0.1
    w = sk.repack(qw, "cuda", bias=bias)
    x = torch.randn(nb, k, generator=torch.Generator().manual_seed(1))
    ref = _quant256_ref(x) @ qw.dequant().t() + bias
    y = sk.gemv([w], x.cuda(), max_ctas=ctas).cpu()          # fp32 rows, quantised inside the kernel
    assert _close(y, ref), (y - ref).abs().max()
    y2 = sk.gemv([w], sk.quant256(x.cuda()), max_ctas=ctas).cpu()      # pre-quantised input
    assert _close(y2, ref), (y2 - ref).abs().max()
    full = x @ qw.dequant().t() + bias
    assert ((y - full).norm() / full.norm()).item() < 2e-2
    out = torch.ones(nb, n, device="cuda")
    sk.gemv([w], x.cuda(), out=out, mode=sk.MODE_ACCUM, max_ctas=ctas)
    assert _close(out.cpu(), ref + 1.0)
    sk.workspace("cuda").check()


@pytest.mark.parametrize("nb", [1, 4])
def test_gemv_sk_norm_prologue_and_segments(nb):
    K, sk = _mods()
    k = 512
    qs = [_qw(GGMLType.Q4_K, 96, k, 1), _qw(GGMLType.Q6_K, 48, k, 2), _qw(GGMLType.Q4_K, 4096, k, 3)]
    ws = [sk.repack(q, "cuda") for q in qs]
    x = torch.randn(nb, k, generator=torch.Generator().manual_seed(5)) * 3
    nw = torch.rand(k, generator=torch.Generator().manual_seed(6)) + 0.5
    xr = _quant256_ref(R.rmsnorm(x, nw, 1e-5))
    ref = torch.cat([xr @ q.dequant().t() for q in qs], 1)
    for ctas in (0, 7, 148):
        for _ in range(2):      # back-to-back launches reuse the hand-over flags
            y = sk.gemv(ws, x.cuda(), norm_w=nw.cuda(), eps=1e-5, max_ctas=ctas).cpu()
            assert y.shape == (nb, 96 + 48 + 4096)
            assert _close(y, ref), (ctas, (y - ref).abs().max())
    sk.workspace("cuda").check()


@pytest.mark.parametrize("act", ["silu", "gelu_tanh", "swiglu_oai"])
def test_gemv_sk_glu(act):
    K, sk = _mods()
    n, k, nb = 256, 512, 3
    qg, qu = _qw(GGMLType.Q4_K, n, k, 1), _qw(GGMLType.Q4_K, n, k, 2)
    g = torch.Generator().manual_seed(9)
    bg, bu = torch.randn(n, generator=g) * 0.1, torch.randn(n, generator=g) * 0.1
    gu = sk.repack(sk.interleave(qg, qu), "cuda", bias=torch.stack([bg, bu], 1).reshape(-1))
    x = torch.randn(nb, k, generator=g) * 3
    xr = _quant256_ref(x)
    ref = R.glu(xr @ qg.dequant().t() + bg, xr @ qu.dequant().t() + bu, act)
    h = sk.gemv([gu], x.cuda(), mode=sk.MODE_GLU, act=act).cpu()
    assert h.shape == (nb, n)
    assert _close(h, ref, 3e-3), (h - ref).abs().max()


def test_gemv_sk_model_shapes():
    """Llama-8B gate/up and down shapes: every SM streams a slice, tiles are split between CTAs."""
    K, sk = _mods()
    dev = "cuda"
    for (n, k, t) in ((2 * 14336, 4096, GGMLType.Q4_K), (4096, 14336, GGMLType.Q6_K)):
        w = torch.randn(512, k, device=dev, generator=torch.Generator(device=dev).manual_seed(n)) * 0.02
        q = QWeight.from_float("w", w, t)
        raw = q.raw.view(512, -1).repeat(n // 512, 1).reshape(-1)
        qw = QWeight("w", t, (n, k), raw)
        u = sk.repack(qw, dev)
        for nb in (1, 8):
            x = torch.randn(nb, k, device=dev)
            ref = _quant256_ref(x) @ q.dequant().t().to(dev)
            ref = ref.repeat(1, n // 512)
            y = sk.gemv([u], x if sk.fits_fused_input(nb, k) else sk.quant256(x))
            assert _close(y.cpu(), ref.cpu()), (n, k, nb, (y - ref).abs().max())
    sk.workspace(dev).check()


@pytest.mark.parametrize("nb", [1, 3])
def test_gemv_chain_runs_dependent_products_in_one_launch(nb):
    """attention-output projection -> gated FFN -> down projection -> next Q/K/V, each phase reading the previous one's output."""
    K, sk = _mods()
    d, f = 512, 1024
    g = torch.Generator().manual_seed(4)
    qo, qg, qu, qd, qq = (_qw(GGMLType.Q4_K, d, d, 1), _qw(GGMLType.Q4_K, f, d, 2), _qw(GGMLType.Q4_K, f, d, 3), _qw(GGMLType.Q6_K, d, f, 4),
                          _qw(GGMLType.Q4_K, 3 * d, d, 5))
    wo, wgu, wd, wq = sk.repack(qo, "cuda"), sk.repack(sk.interleave(qg, qu), "cuda"), sk.repack(qd, "cuda"), sk.repack(qq, "cuda")
    ao = torch.randn(nb, d, generator=g)
    x0 = torch.randn(nb, d, generator=g)
    n1, n2 = torch.rand(d, generator=g) + 0.5, torch.rand(d, generator=g) + 0.5
    # reference
    x1 = x0 + _quant256_ref(ao) @ qo.dequant().t()
    hn = _quant256_ref(R.rmsnorm(x1, n1, 1e-5))
    h = R.glu(hn @ qg.dequant().t(), hn @ qu.dequant().t(), "silu")
    x2 = x1 + _quant256_ref(h) @ qd.dequant().t()
    qkv = _quant256_ref(R.rmsnorm(x2, n2, 1e-5)) @ qq.dequant().t()
    ao_d, n1_d, n2_d = ao.cuda(), n1.cuda(), n2.cuda()      # phases hold raw pointers: the tensors must outlive the launch
    for _ in range(2):      # twice: the barrier counters must be back at zero
        x = x0.cuda().clone()
        hbuf = torch.zeros(nb, f, device="cuda")
        out = torch.zeros(nb, 3 * d, device="cuda")
        ph = [sk.phase([wo], ao_d, x, mode=sk.MODE_ACCUM),
              sk.phase([wgu], x, hbuf, norm_w=n1_d, eps=1e-5, mode=sk.MODE_GLU),
              sk.phase([wd], hbuf, x, mode=sk.MODE_ACCUM),
              sk.phase([wq], x, out, norm_w=n2_d, eps=1e-5)]
        sk.gemv_chain(ph, "cuda")
        sk.workspace("cuda").check()
        assert _close(x.cpu(), x2, 5e-3), (x.cpu() - x2).abs().max()
        assert _close(out.cpu(), qkv, 1e-2), (out.cpu() - qkv).abs().max()


def test_engine_decodes_up_to_32_sequences_in_one_step(tmp_path):
    """A model whose matrices all have a unit layout takes 32 sequences per step; a batched step gives every sequence the
    logits it gets when it is decoded alone, and both agree with the fp32 reference graph."""
    from ollama_b200.engine.b200 import B200Backend, MAX_STREAM_BATCH
    from ollama_b200.engine.backend import TorchBackend, open_model
    from ollama_b200.models.synth import write_synthetic_gguf
    p = str(tmp_path / "m.gguf")
    write_synthetic_gguf(p, "tiny-qwen3", "Q4_K_M")
    g = open_model(p)
    eng = B200Backend(g, "cuda")
    assert eng.max_batch == MAX_STREAM_BATCH and all(L.sk is not None for L in eng.layers) and eng.sk_head is not None
    ref = TorchBackend(g, "cpu")
    n = 32
    eng.alloc(n, 64)
    ref.alloc(n, 64)
    gen = torch.Generator().manual_seed(5)
    prompts = [torch.randint(259, 4096, (5 + s % 7,), generator=gen).tolist() for s in range(n)]
    toks = []
    for s, pr in enumerate(prompts):
        lr = ref.prefill(s, pr, 0)
        eng.prefill(s, pr, 0)
        toks.append(int(lr.argmax()))
    pos = [len(pr) for pr in prompts]
    want = ref.decode(list(range(n)), toks, pos)
    tol = 0.05 * want.abs().max().item()
    for nb in (32, 13, 3, 1):
        got = eng.decode(list(range(nb)), toks[:nb], pos[:nb]).cpu()
        assert (got - want[:nb]).abs().max().item() < tol, nb
        assert eng.decode_argmax(list(range(nb)), toks[:nb], pos[:nb]) == got.argmax(-1).tolist()
    from ollama_b200.ops import sk
    sk.workspace("cuda").check()
