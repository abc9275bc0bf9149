"""GGML block-quantisation codecs written with torch tensor ops.

They run on CPU or on a CUDA device (the same code quantises an 8-billion-parameter random
checkpoint on the GPU in seconds) and are the reference the CUDA kernels are tested against.

Block layouts follow the GGUF specification (sizes listed in the reference at
fs/ggml/ggml.go:442-513; MXFP4 nibble order at convert/convert_gptoss.go:229-239):

  Q8_0   half d | int8 q[32]                                   x = d*q
  Q4_0   half d | u8 qs[16]                                    x[i] = d*((qs[i]&15)-8), x[i+16] = d*((qs[i]>>4)-8)
  Q4_1   half d, half m | qs[16]                               x = d*q + m
  Q5_0   half d | u8 qh[4] | qs[16]                            5th bit from qh
  Q5_1   half d, half m | qh[4] | qs[16]
  Q2_K   u8 scales[16] | u8 qs[64] | half d, half dmin
  Q3_K   u8 hmask[32] | u8 qs[64] | u8 scales[12] | half d
  Q4_K   half d, half dmin | u8 scales[12] | u8 qs[128]
  Q5_K   half d, half dmin | u8 scales[12] | u8 qh[32] | u8 qs[128]
  Q6_K   u8 ql[128] | u8 qh[64] | int8 scales[16] | half d
  Q8_K   float d | int8 q[256] | int16 bsums[16]
  MXFP4  u8 e8m0 | u8 qs[16]                                   x = e2m1(q) * 2^(e-127)
  IQ4_NL half d | u8 qs[16]                                    non-linear 4-bit codebook
"""
from __future__ import annotations

import torch

from .types import GGMLType, block_size, type_size

_MXFP4_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0)
_IQ4NL_VALUES = (-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113)


def _f16(b: torch.Tensor) -> torch.Tensor:
    """[..., 2] uint8 -> [...] float32 (little-endian IEEE half)."""
    return b.contiguous().view(torch.float16).squeeze(-1).float()


def _blocks(raw: torch.Tensor, t: GGMLType) -> torch.Tensor:
    raw = raw.reshape(-1)
    if raw.dtype != torch.uint8:
        raw = raw.view(torch.uint8)
    ts = type_size(t)
    if raw.numel() % ts:
        raise ValueError(f"{raw.numel()} bytes is not a whole number of {t.name} blocks")
    return raw.view(-1, ts)


def _scale_min_k4(sc: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Unpack the 12-byte 6-bit scale/min table of Q4_K / Q5_K: [N,12] u8 -> two [N,8] float."""
    s = sc.to(torch.int32)
    lo_sc = s[:, 0:4] & 63
    lo_m = s[:, 4:8] & 63
    hi_sc = (s[:, 8:12] & 0xF) | ((s[:, 0:4] >> 6) << 4)
    hi_m = (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 6) << 4)
    return torch.cat([lo_sc, hi_sc], 1).float(), torch.cat([lo_m, hi_m], 1).float()


def _native_dequantize(raw: torch.Tensor, t: GGMLType) -> torch.Tensor | None:
    """Host tensors go through the C++ codecs (native/codecs.cpp) when the library is there; None = use the tensor ops."""
    if raw.device.type != "cpu":
        return None
    from ..utils import hostlib
    if not hostlib.codec_supported(int(t), False):
        return None
    blocks = _blocks(raw, t).contiguous()
    out = torch.empty(blocks.shape[0] * block_size(t), dtype=torch.float32)
    if hostlib.lib().b2h_dequantize(int(t), blocks.data_ptr(), out.data_ptr(), blocks.shape[0]) != 0:
        return None
    return out


def _native_quantize(x: torch.Tensor, t: GGMLType) -> torch.Tensor | None:
    if x.device.type != "cpu":
        return None
    from ..utils import hostlib
    if not hostlib.codec_supported(int(t), True):
        return None
    xf = x.float().contiguous().reshape(-1)
    n = xf.numel() // block_size(t)
    out = torch.empty(n * type_size(t), dtype=torch.uint8)
    if hostlib.lib().b2h_quantize(int(t), xf.data_ptr(), out.data_ptr(), n) != 0:
        return None
    return out


def dequantize(raw: torch.Tensor, t: int, n_elements: int | None = None, native: bool = True) -> torch.Tensor:
    """Decode a flat byte tensor of type ``t`` into float32 (flat).  ``native=False`` forces the tensor-op codecs."""
    t = GGMLType(t)
    if native and t.value >= 2 and t not in (GGMLType.BF16, GGMLType.F64, GGMLType.I8, GGMLType.I16, GGMLType.I32, GGMLType.I64):
        y = _native_dequantize(raw, t)
        if y is not None:
            if n_elements is not None and y.numel() != n_elements:
                raise ValueError(f"decoded {y.numel()} elements, expected {n_elements}")
            return y
    if t == GGMLType.F32:
        return raw.reshape(-1).view(torch.uint8).view(torch.float32).clone()
    if t == GGMLType.F16:
        return raw.reshape(-1).view(torch.uint8).view(torch.float16).float()
    if t == GGMLType.BF16:
        return raw.reshape(-1).view(torch.uint8).view(torch.bfloat16).float()
    if t == GGMLType.F64:
        return raw.reshape(-1).view(torch.uint8).view(torch.float64).float()
    if t in (GGMLType.I8, GGMLType.I16, GGMLType.I32, GGMLType.I64):
        dt = {GGMLType.I8: torch.int8, GGMLType.I16: torch.int16, GGMLType.I32: torch.int32, GGMLType.I64: torch.int64}[t]
        return raw.reshape(-1).view(torch.uint8).view(dt).float()
    b = _blocks(raw, t)
    n = b.shape[0]
    i32 = torch.int32

    if t == GGMLType.Q8_0:
        d = _f16(b[:, 0:2])
        q = b[:, 2:34].view(torch.int8).float()
        out = q * d[:, None]
    elif t == GGMLType.Q4_0:
        d = _f16(b[:, 0:2])
        qs = b[:, 2:18].to(i32)
        q = torch.cat([qs & 15, qs >> 4], 1).float() - 8.0
        out = q * d[:, None]
    elif t == GGMLType.Q4_1:
        d, m = _f16(b[:, 0:2]), _f16(b[:, 2:4])
        qs = b[:, 4:20].to(i32)
        q = torch.cat([qs & 15, qs >> 4], 1).float()
        out = q * d[:, None] + m[:, None]
    elif t in (GGMLType.Q5_0, GGMLType.Q5_1):
        if t == GGMLType.Q5_0:
            d, m, o = _f16(b[:, 0:2]), None, 2
        else:
            d, m, o = _f16(b[:, 0:2]), _f16(b[:, 2:4]), 4
        qh = b[:, o:o + 4].contiguous().view(torch.int32)  # [N,1] little-endian u32 bits
        qs = b[:, o + 4:o + 20].to(i32)
        sh = torch.arange(32, device=b.device, dtype=i32)[None, :]
        hb = ((qh >> sh) & 1) << 4
        q = torch.cat([qs & 15, qs >> 4], 1) | hb
        out = (q.float() - 16.0) * d[:, None] if m is None else q.float() * d[:, None] + m[:, None]
    elif t == GGMLType.Q2_K:
        scales = b[:, 0:16].to(i32)
        qs = b[:, 16:80].to(i32).view(n, 2, 32)
        d, dmin = _f16(b[:, 80:82]), _f16(b[:, 82:84])
        shifts = torch.tensor([0, 2, 4, 6], device=b.device, dtype=i32).view(1, 1, 4, 1)
        q = (qs[:, :, None, :] >> shifts) & 3               # [N, half, shift j, 32]
        q = q.reshape(n, 16, 16).float()                     # 16 groups of 16 in output order
        dl = d[:, None] * (scales & 15).float()
        ml = dmin[:, None] * (scales >> 4).float()
        out = q * dl[:, :, None] - ml[:, :, None]
    elif t == GGMLType.Q3_K:
        hm = b[:, 0:32].to(i32)
        qs = b[:, 32:96].to(i32).view(n, 2, 32)
        sc = b[:, 96:108].to(i32)
        d = _f16(b[:, 108:110])
        # 16 six-bit scales: low 4 bits from bytes 0..7 (nibbles), high 2 bits from bytes 8..11
        lo = torch.cat([sc[:, 0:8] & 15, sc[:, 0:8] >> 4], 1)                      # [N,16]
        hi_src = sc[:, 8:12]
        hi = torch.cat([(hi_src >> (2 * k)) & 3 for k in range(4)], 1)             # [N,16]
        scales = ((lo | (hi << 4)) - 32).float()
        shifts = torch.tensor([0, 2, 4, 6], device=b.device, dtype=i32).view(1, 1, 4, 1)
        q = (qs[:, :, None, :] >> shifts) & 3                                       # [N,2,4,32]
        bit = torch.arange(8, device=b.device, dtype=i32).view(1, 2, 4, 1)         # mask bit = half*4 + j
        h = (hm[:, None, None, :] >> bit) & 1
        q = (q - (1 - h) * 4).reshape(n, 16, 16).float()
        out = q * (d[:, None] * scales)[:, :, None]
    elif t == GGMLType.Q4_K:
        d, dmin = _f16(b[:, 0:2]), _f16(b[:, 2:4])
        sc, mn = _scale_min_k4(b[:, 4:16])
        qs = b[:, 16:144].to(i32).view(n, 4, 32)
        q = torch.stack([qs & 15, qs >> 4], 2).reshape(n, 8, 32).float()
        out = q * (d[:, None] * sc)[:, :, None] - (dmin[:, None] * mn)[:, :, None]
    elif t == GGMLType.Q5_K:
        d, dmin = _f16(b[:, 0:2]), _f16(b[:, 2:4])
        sc, mn = _scale_min_k4(b[:, 4:16])
        qh = b[:, 16:48].to(i32)
        qs = b[:, 48:176].to(i32).view(n, 4, 32)
        q = torch.stack([qs & 15, qs >> 4], 2).reshape(n, 8, 32)
        bit = torch.arange(8, device=b.device, dtype=i32).view(1, 8, 1)
        q = (q + (((qh[:, None, :] >> bit) & 1) << 4)).float()
        out = q * (d[:, None] * sc)[:, :, None] - (dmin[:, None] * mn)[:, :, None]
    elif t == GGMLType.Q6_K:
        ql = b[:, 0:128].to(i32).view(n, 2, 64)
        qh = b[:, 128:192].to(i32).view(n, 2, 32)
        sc = b[:, 192:208].contiguous().view(torch.int8).float()
        d = _f16(b[:, 208:210])
        l0, l1 = ql[:, :, 0:32], ql[:, :, 32:64]
        q1 = (l0 & 15) | (((qh >> 0) & 3) << 4)
        q2 = (l1 & 15) | (((qh >> 2) & 3) << 4)
        q3 = (l0 >> 4) | (((qh >> 4) & 3) << 4)
        q4 = (l1 >> 4) | (((qh >> 6) & 3) << 4)
        q = torch.stack([q1, q2, q3, q4], 2).reshape(n, 16, 16).float() - 32.0   # [N, half*4*2, 16]
        out = q * (d[:, None] * sc)[:, :, None]
    elif t == GGMLType.Q8_K:
        d = b[:, 0:4].contiguous().view(torch.float32).squeeze(-1)
        q = b[:, 4:260].contiguous().view(torch.int8).float()
        out = q * d[:, None]
    elif t == GGMLType.MXFP4:
        e = b[:, 0].to(i32)
        scale = torch.exp2((e - 127).float())
        qs = b[:, 1:17].to(torch.int64)
        lut = torch.tensor(_MXFP4_VALUES, device=b.device, dtype=torch.float32)
        q = torch.cat([lut[qs & 15], lut[qs >> 4]], 1)
        out = q * scale[:, None]
    elif t == GGMLType.IQ4_NL:
        d = _f16(b[:, 0:2])
        qs = b[:, 2:18].to(torch.int64)
        lut = torch.tensor(_IQ4NL_VALUES, device=b.device, dtype=torch.float32)
        out = torch.cat([lut[qs & 15], lut[qs >> 4]], 1) * d[:, None]
    else:
        raise NotImplementedError(f"dequantisation of {t.name} is not supported")
    out = out.reshape(-1)
    if n_elements is not None and out.numel() != n_elements:
        raise ValueError(f"decoded {out.numel()} elements, expected {n_elements}")
    return out


def dequantize_tensor(raw: torch.Tensor, t: int, torch_shape: tuple[int, ...]) -> torch.Tensor:
    n = 1
    for d in torch_shape:
        n *= d
    return dequantize(raw, t, n).view(*torch_shape)


# ---------------------------------------------------------------------------------------------
# quantisers
# ---------------------------------------------------------------------------------------------

def _h(x: torch.Tensor) -> torch.Tensor:
    """float -> [N,2] uint8 holding IEEE half."""
    return x.to(torch.float16).contiguous().view(-1, 1).view(torch.uint8)


def _rne(x: torch.Tensor) -> torch.Tensor:
    return torch.round(x)


def quantize_q8_0(x: torch.Tensor) -> torch.Tensor:
    x = x.float().reshape(-1, 32)
    amax = x.abs().amax(1)
    d = amax / 127.0
    inv = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    q = _rne(x * inv[:, None]).clamp(-127, 127).to(torch.int8)
    return torch.cat([_h(d), q.view(torch.uint8)], 1).reshape(-1)


def quantize_q4_0(x: torch.Tensor) -> torch.Tensor:
    x = x.float().reshape(-1, 32)
    idx = x.abs().argmax(1, keepdim=True)
    mx = x.gather(1, idx).squeeze(1)
    d = mx / -8.0
    inv = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
    q = (x * inv[:, None] + 8.5).floor().clamp(0, 15).to(torch.uint8)
    packed = q[:, :16] | (q[:, 16:] << 4)
    return torch.cat([_h(d), packed], 1).reshape(-1)


def quantize_q4_1(x: torch.Tensor) -> torch.Tensor:
    x = x.float().reshape(-1, 32)
    mn, mx = x.amin(1), x.amax(1)
    d = (mx - mn) / 15.0
    inv = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    q = ((x - mn[:, None]) * inv[:, None] + 0.5).floor().clamp(0, 15).to(torch.uint8)
    packed = q[:, :16] | (q[:, 16:] << 4)
    return torch.cat([_h(d), _h(mn), packed], 1).reshape(-1)


def quantize_q5_0(x: torch.Tensor) -> torch.Tensor:
    x = x.float().reshape(-1, 32)
    idx = x.abs().argmax(1, keepdim=True)
    mx = x.gather(1, idx).squeeze(1)
    d = mx / -16.0
    inv = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
    q = (x * inv[:, None] + 16.5).floor().clamp(0, 31).to(torch.int32)
    packed = ((q[:, :16] & 15) | ((q[:, 16:] & 15) << 4)).to(torch.uint8)
    sh = torch.arange(32, device=x.device, dtype=torch.int64)[None, :]
    qh = (((q.to(torch.int64) >> 4) & 1) << sh).sum(1)
    qh = torch.stack([(qh >> (8 * k)) & 255 for k in range(4)], 1).to(torch.uint8)
    return torch.cat([_h(d), qh, packed], 1).reshape(-1)


def quantize_q4_k(x: torch.Tensor) -> torch.Tensor:
    """Q4_K with a closed-form (min/max) choice of the 6-bit sub-block scales and mins.

    The upstream tool refines the scales iteratively; the blocks produced here are valid
    Q4_K with slightly higher error, which is what a random-init benchmark checkpoint needs.
    """
    x = x.float().reshape(-1, 8, 32)
    n = x.shape[0]
    mn = x.amin(2).clamp(max=0.0)                      # sub-block minimum (<= 0)
    mx = x.amax(2)
    scale = (mx - mn) / 15.0
    mins = -mn
    d = scale.amax(1) / 63.0
    dmin = mins.amax(1) / 63.0
    # the stored super-scales are halves: quantise against the values the decoder will see
    d = d.to(torch.float16).float()
    dmin = dmin.to(torch.float16).float()
    inv_d = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    inv_dm = torch.where(dmin > 0, 1.0 / dmin, torch.zeros_like(dmin))
    sc = _rne(scale * inv_d[:, None]).clamp(0, 63)
    m = _rne(mins * inv_dm[:, None]).clamp(0, 63)
    eff = d[:, None] * sc
    inv_eff = torch.where(eff > 0, 1.0 / eff, torch.zeros_like(eff))
    q = _rne((x + (dmin[:, None] * m)[:, :, None]) * inv_eff[:, :, None]).clamp(0, 15).to(torch.uint8)
    q = q.view(n, 4, 2, 32)
    qs = (q[:, :, 0, :] | (q[:, :, 1, :] << 4)).reshape(n, 128)
    sci, mi = sc.to(torch.int32), m.to(torch.int32)
    b0 = (sci[:, 0:4] & 63) | ((sci[:, 4:8] >> 4) << 6)
    b1 = (mi[:, 0:4] & 63) | ((mi[:, 4:8] >> 4) << 6)
    b2 = (sci[:, 4:8] & 15) | ((mi[:, 4:8] & 15) << 4)
    scales = torch.cat([b0, b1, b2], 1).to(torch.uint8)
    return torch.cat([_h(d), _h(dmin), scales, qs], 1).reshape(-1)


def quantize_q5_k(x: torch.Tensor) -> torch.Tensor:
    x = x.float().reshape(-1, 8, 32)
    n = x.shape[0]
    mn = x.amin(2).clamp(max=0.0)
    mx = x.amax(2)
    scale = (mx - mn) / 31.0
    mins = -mn
    d = (scale.amax(1) / 63.0).to(torch.float16).float()
    dmin = (mins.amax(1) / 63.0).to(torch.float16).float()
    inv_d = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    inv_dm = torch.where(dmin > 0, 1.0 / dmin, torch.zeros_like(dmin))
    sc = _rne(scale * inv_d[:, None]).clamp(0, 63)
    m = _rne(mins * inv_dm[:, None]).clamp(0, 63)
    eff = d[:, None] * sc
    inv_eff = torch.where(eff > 0, 1.0 / eff, torch.zeros_like(eff))
    q = _rne((x + (dmin[:, None] * m)[:, :, None]) * inv_eff[:, :, None]).clamp(0, 31).to(torch.int32)
    lo = (q & 15).to(torch.uint8).view(n, 4, 2, 32)
    qs = (lo[:, :, 0, :] | (lo[:, :, 1, :] << 4)).reshape(n, 128)
    bit = torch.arange(8, device=x.device, dtype=torch.int32).view(1, 8, 1)
    qh = (((q >> 4) & 1) << bit).sum(1).to(torch.uint8)
    sci, mi = sc.to(torch.int32), m.to(torch.int32)
    b0 = (sci[:, 0:4] & 63) | ((sci[:, 4:8] >> 4) << 6)
    b1 = (mi[:, 0:4] & 63) | ((mi[:, 4:8] >> 4) << 6)
    b2 = (sci[:, 4:8] & 15) | ((mi[:, 4:8] & 15) << 4)
    scales = torch.cat([b0, b1, b2], 1).to(torch.uint8)
    return torch.cat([_h(d), _h(dmin), scales, qh, qs], 1).reshape(-1)


def quantize_q6_k(x: torch.Tensor) -> torch.Tensor:
    x = x.float().reshape(-1, 16, 16)
    n = x.shape[0]
    idx = x.abs().argmax(2, keepdim=True)
    mx = x.gather(2, idx).squeeze(2)
    s = mx / -32.0                                     # signed per-16 scale so that the extreme maps to -32
    sidx = s.abs().argmax(1, keepdim=True)
    smax = s.gather(1, sidx).squeeze(1)
    d = (smax / -128.0).to(torch.float16).float()
    inv_d = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
    sc = _rne(s * inv_d[:, None]).clamp(-128, 127)
    eff = d[:, None] * sc
    inv_eff = torch.where(eff != 0, 1.0 / eff, torch.zeros_like(eff))
    q = (_rne(x * inv_eff[:, :, None]).clamp(-32, 31) + 32).to(torch.int32)   # [N,16,16] in 0..63
    q = q.view(n, 2, 4, 32)                            # half, quarter(q1..q4), l
    l0 = (q[:, :, 0] & 15) | ((q[:, :, 2] & 15) << 4)
    l1 = (q[:, :, 1] & 15) | ((q[:, :, 3] & 15) << 4)
    ql = torch.cat([l0, l1], 2).reshape(n, 128).to(torch.uint8)
    qh = ((q[:, :, 0] >> 4) | ((q[:, :, 1] >> 4) << 2) | ((q[:, :, 2] >> 4) << 4) | ((q[:, :, 3] >> 4) << 6))
    qh = qh.reshape(n, 64).to(torch.uint8)
    return torch.cat([ql, qh, sc.to(torch.int8).view(torch.uint8), _h(d)], 1).reshape(-1)


def quantize_mxfp4(x: torch.Tensor) -> torch.Tensor:
    x = x.float().reshape(-1, 32)
    amax = x.abs().amax(1)
    # shared power-of-two scale so that the block maximum fits under 6.0
    e = torch.where(amax > 0, torch.floor(torch.log2(amax.clamp(min=1e-38))) - 2, torch.full_like(amax, -127.0))
    e = e.clamp(-127, 127)
    scaled = x / torch.exp2(e)[:, None]
    lut = torch.tensor(_MXFP4_VALUES[:8], device=x.device)
    mag = (scaled.abs()[:, :, None] - lut[None, None, :]).abs().argmin(2)
    q = (mag | ((scaled < 0).to(torch.int64) << 3)).to(torch.uint8)
    packed = q[:, :16] | (q[:, 16:] << 4)
    eb = (e + 127).to(torch.uint8)[:, None]
    return torch.cat([eb, packed], 1).reshape(-1)


_QUANTIZERS = {
    GGMLType.Q8_0: quantize_q8_0, GGMLType.Q4_0: quantize_q4_0, GGMLType.Q4_1: quantize_q4_1,
    GGMLType.Q5_0: quantize_q5_0, GGMLType.Q4_K: quantize_q4_k, GGMLType.Q5_K: quantize_q5_k,
    GGMLType.Q6_K: quantize_q6_k, GGMLType.MXFP4: quantize_mxfp4,
}


def quantize(x: torch.Tensor, t: int, native: bool = True) -> torch.Tensor:
    """Encode a float tensor (last dimension contiguous, multiple of the block size) to flat bytes.

    Host tensors are encoded by the C++ codecs, which make the same choices as the tensor-op encoders below
    (identical bytes); ``native=False`` forces the tensor ops."""
    t = GGMLType(t)
    if x.shape[-1] % block_size(t):
        raise ValueError(f"row length {x.shape[-1]} is not a multiple of the {t.name} block size")
    if native and t in _QUANTIZERS:
        y = _native_quantize(x, t)
        if y is not None:
            return y
    if t == GGMLType.F32:
        return x.float().contiguous().view(-1).view(torch.uint8)
    if t == GGMLType.F16:
        return x.to(torch.float16).contiguous().view(-1).view(torch.uint8)
    if t == GGMLType.BF16:
        return x.to(torch.bfloat16).contiguous().view(-1).view(torch.uint8)
    if t not in _QUANTIZERS:
        raise NotImplementedError(f"quantisation to {t.name} is not supported")
    return _QUANTIZERS[t](x.contiguous())


def can_quantize(t: int) -> bool:
    t = GGMLType(t)
    return t in _QUANTIZERS or t in (GGMLType.F32, GGMLType.F16, GGMLType.BF16)
