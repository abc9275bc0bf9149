"""Plain PyTorch (fp32) statements of every operator the model graphs use.

These are the numerical oracle for the CUDA kernels and the execution path on machines
without a GPU.  The op list mirrors the tensor interface the reference keeps as a checklist
(ml/backend.go:130-246): RMSNorm, RoPE (interleaved and half-split, with frequency factors and
YaRN, cf. x/models/nn/rope.go:34-107), scaled-dot-product attention with causal / sliding-window
masks, sinks and soft-capping, SwiGLU / GELU-GLU / clamped SwiGLU (ml/backend.go:183-184) and the
two mixture-of-experts routers.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def rmsnorm(x: torch.Tensor, w: torch.Tensor | None, eps: float) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return y * w.float() if w is not None else y


def layernorm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None, eps: float) -> torch.Tensor:
    return F.layer_norm(x.float(), (x.shape[-1],), w.float(), None if b is None else b.float(), eps)


def yarn_corr_dims(n_dims: int, n_ctx_orig: int, base: float, beta_fast: float, beta_slow: float) -> tuple[float, float]:
    def corr(n_rot: float) -> float:
        return n_dims * math.log(n_ctx_orig / (n_rot * 2 * math.pi)) / (2 * math.log(base))
    lo = max(0.0, math.floor(corr(beta_fast)))
    hi = min(n_dims - 1.0, math.ceil(corr(beta_slow)))
    return lo, hi


def rope_inv_freq(n_dims: int, base: float, *, scaling: str = "none", factor: float = 1.0, orig_ctx: int = 0,
                  beta_fast: float = 32.0, beta_slow: float = 1.0, freq_factors: torch.Tensor | None = None,
                  device=None) -> tuple[torch.Tensor, float]:
    """Per-pair angular frequency (angle = position * inv_freq) and the magnitude scale for cos/sin."""
    half = n_dims // 2
    i = torch.arange(half, device=device, dtype=torch.float32)
    inv = base ** (-2.0 * i / n_dims)
    mscale = 1.0
    if freq_factors is not None:
        inv = inv / freq_factors.float().to(inv.device)[:half]
    if scaling == "linear" and factor > 0:
        inv = inv / factor
    elif scaling == "yarn" and factor > 1.0:
        lo, hi = yarn_corr_dims(n_dims, orig_ctx or 4096, base, beta_fast, beta_slow)
        ramp = 1.0 - ((i - lo) / max(0.001, hi - lo)).clamp(0, 1)   # 1 = keep extrapolated frequency
        inv = (inv / factor) * (1 - ramp) + inv * ramp
        mscale = 1.0 + 0.1 * math.log(factor)
    return inv, mscale


def rope(x: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor, style: str, mscale: float = 1.0) -> torch.Tensor:
    """x: [T, H, D]; pos: [T]; rotates the first ``2*len(inv_freq)`` dims of every head."""
    xf = x.float()
    n_rot = inv_freq.numel() * 2
    ang = pos.float()[:, None] * inv_freq[None, :]
    cos, sin = (ang.cos() * mscale)[:, None, :], (ang.sin() * mscale)[:, None, :]
    rot, rest = xf[..., :n_rot], xf[..., n_rot:]
    if style == "norm":
        a, b = rot[..., 0::2], rot[..., 1::2]
        out = torch.stack([a * cos - b * sin, a * sin + b * cos], -1).flatten(-2)
    else:
        a, b = rot[..., : n_rot // 2], rot[..., n_rot // 2:]
        out = torch.cat([a * cos - b * sin, a * sin + b * cos], -1)
    return torch.cat([out, rest], -1) if rest.shape[-1] else out


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_pos: torch.Tensor, k_pos: torch.Tensor, *,
              scale: float, causal: bool = True, window: int = 0, softcap: float = 0.0,
              sinks: torch.Tensor | None = None, spans=()) -> torch.Tensor:
    """q: [T,H,D]; k: [S,Hkv,D]; v: [S,Hkv,Dv]; returns [T,H,Dv].

    A key at position p_k is visible to a query at p_q when p_k <= p_q (causal) and, with a
    sliding window W, p_q - p_k < W.  ``sinks`` ([H]) adds one value-less logit per head to the
    softmax denominator.  ``spans``: position ranges [lo, hi) inside which every query sees every key,
    whatever the two rules above say (the positions of one image attend to each other in both directions).
    """
    T, H, D = q.shape
    S, Hkv, Dv = v.shape
    g = H // Hkv
    qf = q.float().view(T, Hkv, g, D)
    s = torch.einsum("thgd,shd->hgts", qf, k.float()) * scale
    if softcap > 0:
        s = softcap * torch.tanh(s / softcap)
    dp = q_pos[:, None] - k_pos[None, :]
    mask = torch.zeros(T, S, dtype=torch.bool, device=q.device)
    if causal:
        mask |= dp < 0
    if window > 0:
        mask |= dp >= window
    for lo, hi in spans:
        inside_q, inside_k = (q_pos >= lo) & (q_pos < hi), (k_pos >= lo) & (k_pos < hi)
        mask &= ~(inside_q[:, None] & inside_k[None, :])
    s = s.masked_fill(mask[None, None], float("-inf"))
    if sinks is not None:
        sk = sinks.float().view(Hkv, g, 1, 1).expand(Hkv, g, T, 1)
        s = torch.cat([s, sk], -1)
        p = torch.softmax(s, -1)[..., :S]
    else:
        p = torch.softmax(s, -1)
    p = torch.nan_to_num(p)
    o = torch.einsum("hgts,shd->thgd", p, v.float())
    return o.reshape(T, H, Dv)


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    return F.gelu(x.float(), approximate="tanh")


def glu(gate: torch.Tensor, up: torch.Tensor, act: str, alpha: float = 1.702, limit: float = 7.0) -> torch.Tensor:
    g, u = gate.float(), up.float()
    if act == "silu":
        return F.silu(g) * u
    if act == "gelu_tanh":
        return gelu_tanh(g) * u
    if act == "swiglu_oai":
        g = g.clamp(max=limit)
        u = u.clamp(-limit, limit)
        return g * torch.sigmoid(alpha * g) * (u + 1.0)
    raise ValueError(act)


def moe_route(logits: torch.Tensor, k: int, router: str, norm_topk: bool = True) -> tuple[torch.Tensor, torch.Tensor]:
    """Router logits [T,E] -> (expert ids [T,k] int64, weights [T,k] fp32)."""
    lf = logits.float()
    if router == "softmax_topk":
        p = torch.softmax(lf, -1)
        w, ids = torch.topk(p, k, -1)
        if norm_topk:
            w = w / w.sum(-1, keepdim=True)
    elif router == "topk_softmax":
        top, ids = torch.topk(lf, k, -1)
        w = torch.softmax(top, -1)
    else:
        raise ValueError(router)
    return ids, w


def softcap(x: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(x.float() / cap) if cap > 0 else x
