"""ctypes bindings of the sm_100a kernel library and the load-time weight re-layout.

The library (``ollama_b200/kernels/libb200ops.so``) exports plain C entry points that take raw
device pointers and a stream; tensors stay owned by torch.  If a CUDA device is present and the
library cannot be loaded this module raises: there is no silent fallback on a GPU box.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass, field

import torch

from ..gguf import quants
from ..gguf.types import GGMLType
from ..models.weights import QWeight

_LIB_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "kernels", "libb200ops.so")
_lib = None

WT_F32, WT_F16, WT_BF16, WT_Q8_0, WT_Q4_K, WT_Q6_K, WT_Q5_K, WT_MXFP4, WT_Q4_0 = range(9)
QUANT_INPUT_TYPES = {WT_Q8_0, WT_Q4_K, WT_Q6_K, WT_Q5_K, WT_MXFP4, WT_Q4_0}   # weights that consume int8 activations


class CudaKernelError(RuntimeError):
    pass


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            from ..kernels.build import build
            build()
        _lib = C.CDLL(_LIB_PATH)
    return _lib


def available() -> bool:
    return torch.cuda.is_available()


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise CudaKernelError(f"{what} failed with CUDA error {rc}")


def stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


class WDesc(C.Structure):
    _fields_ = [("p0", C.c_void_p), ("p1", C.c_void_p), ("p2", C.c_void_p), ("p3", C.c_void_p), ("bias", C.c_void_p),
                ("type", C.c_int), ("n", C.c_int), ("k", C.c_int), ("out_off", C.c_int)]


COMM_MAX_RANKS = 8


class CommSend(C.Structure):
    """Destinations and flags of one producer-side exchange (kernels/comm.cuh)."""
    _fields_ = [("n_dst", C.c_int), ("rank", C.c_int), ("local", C.c_void_p), ("peer_flag", C.c_void_p * COMM_MAX_RANKS),
                ("dst", C.c_void_p * COMM_MAX_RANKS), ("parity_stride", C.c_longlong), ("ll", C.c_int)]


class GemvArgs(C.Structure):
    _fields_ = [("seg", WDesc * 4), ("nseg", C.c_int), ("nb", C.c_int), ("xq", C.c_void_p), ("xds", C.c_void_p),
                ("xf", C.c_void_p), ("out", C.c_void_p), ("ldo", C.c_int), ("accumulate", C.c_int), ("cm", CommSend),
                ("ids", C.c_void_p), ("x_div", C.c_int), ("n_pairs", C.c_int)]


class GluArgs(C.Structure):
    _fields_ = [("gu", WDesc), ("nb", C.c_int), ("xq", C.c_void_p), ("xds", C.c_void_p), ("xf", C.c_void_p),
                ("act", C.c_int), ("alpha", C.c_float), ("limit", C.c_float), ("hq", C.c_void_p), ("hds", C.c_void_p),
                ("hf", C.c_void_p), ("ids", C.c_void_p), ("x_div", C.c_int), ("n_pairs", C.c_int)]


class MoeRouteArgs(C.Structure):
    _fields_ = [("logits", C.c_void_p), ("ld", C.c_int), ("n_experts", C.c_int), ("k", C.c_int), ("mode", C.c_int), ("norm_topk", C.c_int),
                ("e_lo", C.c_int), ("e_cnt", C.c_int), ("ids", C.c_void_p), ("lids", C.c_void_p), ("wts", C.c_void_p)]


class MoeCombineArgs(C.Structure):
    _fields_ = [("y", C.c_void_p), ("wts", C.c_void_p), ("k", C.c_int), ("d", C.c_int), ("x", C.c_void_p), ("cm", CommSend)]


class NormQuantArgs(C.Structure):
    _fields_ = [("x", C.c_void_p), ("w", C.c_void_p), ("eps", C.c_float), ("k", C.c_int), ("do_norm", C.c_int),
                ("xq", C.c_void_p), ("xds", C.c_void_p), ("xf", C.c_void_p), ("residual", C.c_void_p),
                ("parts", C.c_void_p), ("n_part", C.c_int), ("part_stride", C.c_longlong), ("parity_stride", C.c_longlong),
                ("chan", C.c_void_p)]


class RopeKvArgs(C.Structure):
    _fields_ = [("qkv", C.c_void_p), ("positions", C.c_void_p), ("slots", C.c_void_p), ("inv_freq", C.c_void_p),
                ("q_norm", C.c_void_p), ("k_norm", C.c_void_p), ("eps", C.c_float), ("mscale", C.c_float),
                ("n_heads", C.c_int), ("n_kv_heads", C.c_int), ("hd", C.c_int), ("n_rot", C.c_int), ("neox", C.c_int),
                ("n_ctx", C.c_int), ("q_out", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
                ("k_scale", C.c_void_p), ("v_scale", C.c_void_p)]


class EmbedArgs(C.Structure):
    _fields_ = [("table", WDesc), ("ids", C.c_void_p), ("scale", C.c_float), ("out", C.c_void_p)]


class DequantArgs(C.Structure):
    _fields_ = [("w", WDesc), ("row0", C.c_int), ("nrows", C.c_int), ("out", C.c_void_p)]


class NormCastArgs(C.Structure):
    _fields_ = [("x", C.c_void_p), ("w", C.c_void_p), ("eps", C.c_float), ("k", C.c_int), ("do_norm", C.c_int), ("out", C.c_void_p)]


class AttnDecodeArgs(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("positions", C.c_void_p),
                ("slots", C.c_void_p), ("n_heads", C.c_int), ("n_kv_heads", C.c_int), ("n_ctx", C.c_int), ("n_splits", C.c_int),
                ("scale", C.c_float), ("softcap", C.c_float), ("window", C.c_int), ("part_acc", C.c_void_p), ("part_ml", C.c_void_p),
                ("k_scale", C.c_void_p), ("v_scale", C.c_void_p)]


class AttnRopeArgs(C.Structure):
    _fields_ = [("qkv", C.c_void_p), ("inv_freq", C.c_void_p), ("mscale", C.c_float), ("n_rot", C.c_int), ("neox", C.c_int)]


class AttnCombineArgs(C.Structure):
    _fields_ = [("part_acc", C.c_void_p), ("part_ml", C.c_void_p), ("sinks", C.c_void_p), ("n_heads", C.c_int),
                ("n_splits", C.c_int), ("hd", C.c_int), ("out", C.c_void_p), ("out_q", C.c_void_p), ("out_ds", C.c_void_p)]


# ---------------------------------------------------------------------------------------------------
# device weights
# ---------------------------------------------------------------------------------------------------
@dataclass
class DevWeight:
    """A weight matrix [n, k] re-laid out into the planes the kernels read (see kernels/common.cuh)."""

    wtype: int
    n: int
    k: int
    planes: list[torch.Tensor]
    bias: torch.Tensor | None = None
    name: str = ""
    experts: int = 0          # > 0: planes hold `experts` stacked [n, k] matrices

    def desc(self, out_off: int = 0, row0: int = 0, rows: int | None = None) -> WDesc:
        """Descriptor of rows [row0, row0+rows) (used for expert slices of stacked tensors)."""
        if not self.planes:      # a kernel given null planes would fault on the device: refuse on the host
            raise CudaKernelError(f"{self.name or 'weight'}: the planes of this matrix were released (it runs on the streaming GEMV)")
        d = WDesc()
        ps = [0, 0, 0, 0]
        for i, p in enumerate(self.planes):
            ps[i] = p.data_ptr() + row0 * (p.numel() * p.element_size() // self.total_rows)
        d.p0, d.p1, d.p2, d.p3 = ps
        d.bias = (self.bias.data_ptr() + row0 * 4) if self.bias is not None else None
        d.type, d.n, d.k, d.out_off = self.wtype, (rows if rows is not None else self.n), self.k, out_off
        return d

    @property
    def total_rows(self) -> int:
        return self.n * max(self.experts, 1)

    @property
    def nbytes(self) -> int:
        return sum(p.numel() * p.element_size() for p in self.planes) + (self.bias.numel() * 4 if self.bias is not None else 0)

    @property
    def quant_input(self) -> bool:
        return self.wtype in QUANT_INPUT_TYPES


def repack(w: QWeight, device, bias: torch.Tensor | None = None) -> DevWeight:
    """GGUF block layout -> dense planes on ``device``.  Encodings without a native kernel become f16."""
    shape = w.shape
    experts = 0
    if len(shape) == 3:
        experts, n, k = shape
    elif len(shape) == 2:
        n, k = shape
    else:
        raise ValueError(f"{w.name}: expected a matrix, got shape {shape}")
    rows = n * max(experts, 1)
    raw = w.raw.to(device)
    t = w.dtype
    b = bias.to(device=device, dtype=torch.float32).contiguous() if bias is not None else None

    def mk(wt, planes):
        return DevWeight(wt, n, k, [p.contiguous() for p in planes], b, w.name, experts)

    if t == GGMLType.F32:
        return mk(WT_F32, [raw.view(torch.float32).view(rows, k)])
    if t == GGMLType.F16:
        return mk(WT_F16, [raw.view(torch.float16).view(rows, k)])
    if t == GGMLType.BF16:
        return mk(WT_BF16, [raw.view(torch.bfloat16).view(rows, k)])
    if t == GGMLType.Q8_0 and k % 32 == 0:
        blk = raw.view(rows, k // 32, 34)
        return mk(WT_Q8_0, [blk[:, :, 2:].reshape(rows, k).view(torch.int8), blk[:, :, :2].reshape(rows, k // 32 * 2).view(torch.float16)])
    if t == GGMLType.Q4_0 and k % 32 == 0:
        blk = raw.view(rows, k // 32, 18)
        return mk(WT_Q4_0, [blk[:, :, 2:].reshape(rows, k // 2), blk[:, :, :2].reshape(rows, k // 32 * 2).view(torch.float16)])
    if t == GGMLType.MXFP4 and k % 32 == 0:
        blk = raw.view(rows, k // 32, 17)
        return mk(WT_MXFP4, [blk[:, :, 1:].reshape(rows, k // 2), blk[:, :, 0].reshape(rows, k // 32)])
    if t in (GGMLType.Q4_K, GGMLType.Q5_K):
        q5 = t == GGMLType.Q5_K
        blk = raw.view(rows, k // 256, 176 if q5 else 144)
        sc, mn = quants._scale_min_k4(blk[:, :, 4:16].reshape(-1, 12))                # two [rows*nsb, 8] float tables
        sc, mn = sc.to(torch.uint8).view(-1, 4, 2), mn.to(torch.uint8).view(-1, 4, 2)
        sm = torch.cat([sc, mn], 2).reshape(rows, k // 256 * 16)                        # per 64-group: sc, sc, min, min
        dd = blk[:, :, :4].reshape(rows, k // 256 * 4)
        if q5:
            return mk(WT_Q5_K, [blk[:, :, 48:].reshape(rows, k // 2), sm, dd, blk[:, :, 16:48].reshape(rows, k // 8)])
        return mk(WT_Q4_K, [blk[:, :, 16:].reshape(rows, k // 2), sm, dd])
    if t == GGMLType.Q6_K:
        blk = raw.view(rows, k // 256, 210)
        return mk(WT_Q6_K, [blk[:, :, :128].reshape(rows, k // 2), blk[:, :, 128:192].reshape(rows, k // 4),
                            blk[:, :, 192:208].reshape(rows, k // 16).view(torch.int8),
                            blk[:, :, 208:210].reshape(rows, k // 256 * 2).view(torch.float16)])
    # anything else (Q2_K, Q3_K, Q4_1, Q5_0, Q5_1, IQ4_NL ...) is expanded once at load time
    deq = quants.dequantize(raw, t, rows * k).view(rows, k).to(torch.float16)
    return mk(WT_F16, [deq])


def dequant_to_bf16(w: DevWeight, row0: int = 0, nrows: int | None = None) -> torch.Tensor:
    nrows = w.total_rows - row0 if nrows is None else nrows
    out = torch.empty(nrows, w.k, device=w.planes[0].device, dtype=torch.bfloat16)
    a = DequantArgs()
    a.w = w.desc(rows=w.total_rows)
    a.row0, a.nrows, a.out = row0, nrows, out.data_ptr()
    _check(lib().b2_dequant_rows(C.byref(a), stream()), "dequant_rows")
    return out


# ---------------------------------------------------------------------------------------------------
# op wrappers (thin; the engine drives the same entry points with pre-built argument structs)
# ---------------------------------------------------------------------------------------------------
@dataclass
class QAct:
    """Activations quantised to int8 blocks of 32 (+ the fp32 copy for float-weight consumers)."""

    q: torch.Tensor            # int8 [nb, k]
    ds: torch.Tensor           # float32 [nb, k/32, 2]
    f: torch.Tensor | None     # float32 [nb, k]


def rmsnorm_quant(x: torch.Tensor, w: torch.Tensor | None, eps: float, do_norm: bool = True, want_f: bool = True,
                  residual: torch.Tensor | None = None, pdl: bool = False) -> QAct:
    nb, k = x.shape
    q = torch.empty(nb, k, device=x.device, dtype=torch.int8)
    ds = torch.empty(nb, k // 32, 2, device=x.device, dtype=torch.float32)
    f = torch.empty(nb, k, device=x.device, dtype=torch.float32) if want_f else None
    a = NormQuantArgs(ptr(x), ptr(w), eps, k, int(do_norm), ptr(q), ptr(ds), ptr(f), ptr(residual))
    _check(lib().b2_rmsnorm_quant(C.byref(a), nb, int(pdl), stream()), "rmsnorm_quant")
    return QAct(q, ds, f)


def gemv(weights: list[DevWeight], x: QAct, out: torch.Tensor | None = None, accumulate: bool = False, pdl: bool = False) -> torch.Tensor:
    """y[b] = concat_i(W_i x[b] + bias_i) for up to four weights sharing the input (1..8 tokens)."""
    nb = x.q.shape[0]
    total = sum(w.n for w in weights)
    if out is None:
        out = torch.empty(nb, total, device=x.q.device, dtype=torch.float32)
    a = GemvArgs()
    off = 0
    for i, w in enumerate(weights):
        a.seg[i] = w.desc(out_off=off)
        off += w.n
    a.nseg, a.nb = len(weights), nb
    a.xq, a.xds, a.xf = ptr(x.q), ptr(x.ds), ptr(x.f)
    a.out, a.ldo, a.accumulate = ptr(out), out.stride(0), int(accumulate)
    _check(lib().b2_gemv(C.byref(a), int(pdl), stream()), "gemv")
    return out


_ACT = {"silu": 0, "gelu_tanh": 1, "swiglu_oai": 2}


def interleave_rows(a: DevWeight, b: DevWeight) -> DevWeight:
    """Row-interleave two equally shaped weights (row 2i = a[i], row 2i+1 = b[i]): the FFN gate/up pair as one matrix."""
    if a.wtype != b.wtype or a.n != b.n or a.k != b.k or a.experts != b.experts:
        raise ValueError("interleave_rows needs two weights of the same encoding and shape")
    rows = a.total_rows
    planes = [torch.stack([pa.view(rows, -1), pb.view(rows, -1)], 1).reshape(2 * rows, -1).contiguous() for pa, pb in zip(a.planes, b.planes)]
    bias = None
    if a.bias is not None or b.bias is not None:
        za = a.bias if a.bias is not None else torch.zeros(rows, device=planes[0].device)
        zb = b.bias if b.bias is not None else torch.zeros(rows, device=planes[0].device)
        bias = torch.stack([za.view(-1), zb.view(-1)], 1).reshape(-1).contiguous()
    return DevWeight(a.wtype, 2 * a.n, a.k, planes, bias, a.name + "+" + b.name, a.experts)


def to_f16(w: DevWeight) -> DevWeight:
    """Expand any encoding to f16 planes (used when a fused pair does not share one encoding)."""
    deq = dequant_to_bf16(w).to(torch.float16)
    return DevWeight(WT_F16, w.n, w.k, [deq], w.bias, w.name, w.experts)


def gemv_glu_quant(gu: DevWeight, x: QAct, act: str, alpha: float = 1.702, limit: float = 7.0,
                   want_f: bool = False, pdl: bool = False) -> QAct:
    """h = act(gate x) * (up x) on the interleaved gate/up matrix, returned as int8 blocks (+ fp32 on request)."""
    nb = x.q.shape[0]
    n = gu.n // 2
    hq = torch.empty(nb, n, device=x.q.device, dtype=torch.int8)
    hds = torch.empty(nb, n // 32, 2, device=x.q.device, dtype=torch.float32)
    hf = torch.empty(nb, n, device=x.q.device, dtype=torch.float32) if want_f else None
    a = GluArgs()
    a.gu = gu.desc()
    a.nb, a.xq, a.xds, a.xf = nb, ptr(x.q), ptr(x.ds), ptr(x.f)
    a.act, a.alpha, a.limit = _ACT[act], alpha, limit
    a.hq, a.hds, a.hf = ptr(hq), ptr(hds), ptr(hf)
    _check(lib().b2_gemv_glu_quant(C.byref(a), int(pdl), stream()), "gemv_glu_quant")
    return QAct(hq, hds, hf)


def embed(table: DevWeight, ids: torch.Tensor, scale: float = 1.0, out: torch.Tensor | None = None) -> torch.Tensor:
    nt = ids.numel()
    if out is None:
        out = torch.empty(nt, table.k, device=ids.device, dtype=torch.float32)
    a = EmbedArgs()
    a.table, a.ids, a.scale, a.out = table.desc(), ptr(ids), scale, ptr(out)
    _check(lib().b2_embed(C.byref(a), nt, stream()), "embed")
    return out


def argmax(logits: torch.Tensor, out: torch.Tensor | None = None, tokens: torch.Tensor | None = None,
           positions: torch.Tensor | None = None) -> torch.Tensor:
    """Arg-max of every row (ties: lowest index).  With ``tokens`` and ``positions`` (int32, one per row) the winner also
    becomes the row's next input token and its position advances by one, in the same launch."""
    rows, n = logits.shape
    if out is None:
        out = torch.empty(rows, device=logits.device, dtype=torch.int32)
    if tokens is not None:
        lib().b2_argmax_advance.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        _check(lib().b2_argmax_advance(ptr(logits), rows, n, logits.stride(0), ptr(out), ptr(tokens), ptr(positions), stream()), "argmax")
        return out
    lib().b2_argmax.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
    _check(lib().b2_argmax(ptr(logits), rows, n, logits.stride(0), ptr(out), stream()), "argmax")
    return out


def rope_kv(qkv: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, inv_freq: torch.Tensor, *, n_heads: int,
            n_kv_heads: int, hd: int, n_rot: int, neox: bool, mscale: float, k_cache: torch.Tensor, v_cache: torch.Tensor,
            q_norm: torch.Tensor | None = None, k_norm: torch.Tensor | None = None, eps: float = 1e-6,
            q_out: torch.Tensor | None = None, pdl: bool = False, k_scale: torch.Tensor | None = None,
            v_scale: torch.Tensor | None = None) -> torch.Tensor:
    """``k_scale`` / ``v_scale`` (f16 [slots, Hkv, n_ctx, hd/32]) select a q8_0 cache: the caches then hold int8."""
    nt = qkv.shape[0]
    if q_out is None:
        q_out = torch.empty(nt, n_heads, hd, device=qkv.device, dtype=torch.float32)
    a = RopeKvArgs(ptr(qkv), ptr(positions), ptr(slots), ptr(inv_freq), ptr(q_norm), ptr(k_norm), eps, mscale, n_heads,
                   n_kv_heads, hd, n_rot, int(neox), k_cache.shape[2], ptr(q_out), ptr(k_cache), ptr(v_cache), ptr(k_scale), ptr(v_scale))
    _check(lib().b2_rope_kv(C.byref(a), nt, int(pdl), stream()), "rope_kv")
    return q_out


def attn_decode_mode(mode: int) -> None:
    """Kernel behind :func:`attn_decode`: 1 = tensor-core split-K kernel, 0 = scalar kernel, -1 = by shape (default)."""
    lib().b2_attn_decode_mode(int(mode))


def attn_decode_stages(n: int) -> int:
    """Pipeline depth of the tensor-core decode-attention kernel: 0 = chosen per launch (four stages when every SM gets at most one
    CTA, three when at most two, else two), 2, 3 or 4 = forced.  Returns the previous setting."""
    return int(lib().b2_attn_decode_stages(int(n)))


def attn_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, *,
                scale: float, n_splits: int, window: int = 0, softcap: float = 0.0, sinks: torch.Tensor | None = None,
                scratch: tuple[torch.Tensor, torch.Tensor] | None = None, quant_out: bool = True, pdl: bool = False,
                k_scale: torch.Tensor | None = None, v_scale: torch.Tensor | None = None):
    """q: [nb, H, hd] fp32; caches [slots, Hkv, n_ctx, hd] f16 (int8 + scales for q8_0).  Returns (out fp32 [nb, H*hd], QAct or None)."""
    nb, H, hd = q.shape
    Hkv, n_ctx = k_cache.shape[1], k_cache.shape[2]
    dev = q.device
    if scratch is None:
        scratch = (torch.empty(nb * H * n_splits * hd, device=dev, dtype=torch.float32),
                   torch.empty(nb * H * n_splits * 2, device=dev, dtype=torch.float32))
    out = torch.empty(nb, H * hd, device=dev, dtype=torch.float32)
    oq = torch.empty(nb, H * hd, device=dev, dtype=torch.int8) if quant_out else None
    ods = torch.empty(nb, H * hd // 32, 2, device=dev, dtype=torch.float32) if quant_out else None
    a = AttnDecodeArgs(ptr(q), ptr(k_cache), ptr(v_cache), ptr(positions), ptr(slots), H, Hkv, n_ctx, n_splits, scale, softcap,
                       window, ptr(scratch[0]), ptr(scratch[1]), ptr(k_scale), ptr(v_scale))
    c = AttnCombineArgs(ptr(scratch[0]), ptr(scratch[1]), ptr(sinks), H, n_splits, hd, ptr(out), ptr(oq), ptr(ods))
    _check(lib().b2_attn_decode(C.byref(a), C.byref(c), nb, hd, int(pdl), stream()), "attn_decode")
    return out, (QAct(oq, ods, out) if quant_out else None)


def attn_decode_rope(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor,
                     inv_freq: torch.Tensor, *, n_heads: int, n_rot: int, neox: bool, mscale: float, scale: float, n_splits: int,
                     window: int = 0, softcap: float = 0.0, sinks: torch.Tensor | None = None, pdl: bool = False) -> torch.Tensor | None:
    """Decode attention on raw projections ``qkv`` [nb, (H + 2 Hkv) * hd]: the kernel rotates the queries and the new key,
    appends key and value to the f16 caches at ``positions`` and attends over positions 0..position.  Returns the output
    [nb, H * hd], or None when the tensor-core kernel does not take the shape (nothing was launched)."""
    nb = qkv.shape[0]
    Hkv, n_ctx, hd = k_cache.shape[1], k_cache.shape[2], k_cache.shape[3]
    dev = qkv.device
    acc = torch.empty(nb * n_heads * n_splits * hd, device=dev, dtype=torch.float32)
    ml = torch.empty(nb * n_heads * n_splits * 2, device=dev, dtype=torch.float32)
    out = torch.empty(nb, n_heads * hd, device=dev, dtype=torch.float32)
    a = AttnDecodeArgs(None, ptr(k_cache), ptr(v_cache), ptr(positions), ptr(slots), n_heads, Hkv, n_ctx, n_splits, scale, softcap,
                       window, ptr(acc), ptr(ml), None, None)
    r = AttnRopeArgs(ptr(qkv), ptr(inv_freq), mscale, n_rot, int(neox))
    c = AttnCombineArgs(ptr(acc), ptr(ml), ptr(sinks), n_heads, n_splits, hd, ptr(out), None, None)
    f = lib().b2_attn_decode_rope
    f.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
    rc = f(C.byref(a), C.byref(r), C.byref(c), nb, hd, int(pdl), stream())
    if rc == 801:
        return None
    _check(rc, "attn_decode_rope")
    return out


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, bias: torch.Tensor | None = None, out: torch.Tensor | None = None,
              accumulate: bool = False) -> torch.Tensor:
    """out[m, n] (+)= a[m, k] @ b[n, k]^T + bias on the tcgen05 tensor-core kernel (bf16 operands, fp32 result)."""
    m, k = a.shape
    n = b.shape[0]
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16 or b.shape[1] != k:
        raise ValueError("gemm_bf16 needs bf16 operands [m, k] and [n, k]")
    a, b = a.contiguous(), b.contiguous()
    if out is None:
        out = torch.empty(m, n, device=a.device, dtype=torch.float32)
    f = lib().b2_gemm_bf16
    f.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p]
    _check(f(ptr(a), ptr(b), m, n, k, ptr(out), out.stride(0), ptr(bias), int(accumulate), stream()), "gemm_bf16")
    return out


def gemm_bf16_out16(a: torch.Tensor, b: torch.Tensor, bias: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """Same product as :func:`gemm_bf16` with a bf16 result (n % 8 == 0)."""
    m, k = a.shape
    n = b.shape[0]
    a, b = a.contiguous(), b.contiguous()
    if out is None:
        out = torch.empty(m, n, device=a.device, dtype=torch.bfloat16)
    f = lib().b2_gemm_bf16_out16
    f.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
    _check(f(ptr(a), ptr(b), m, n, k, ptr(out), out.stride(0), ptr(bias), stream()), "gemm_bf16_out16")
    return out


def gemm_bf16_scatter(a: torch.Tensor, b: torch.Tensor, ldo: int, cm: "CommSend", rows_per_rank: int, bias: torch.Tensor | None = None) -> None:
    """Row-parallel GEMM of a tensor-parallel group: partial rows go straight to their owners' buffers (kernels/gemm_tc.cu)."""
    m, k = a.shape
    n = b.shape[0]
    a, b = a.contiguous(), b.contiguous()
    f = lib().b2_gemm_bf16_scatter
    f.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
    _check(f(ptr(a), ptr(b), m, n, k, ldo, ptr(bias), C.addressof(cm), rows_per_rank, stream()), "gemm_bf16_scatter")


def gemm_q_scatter(x: torch.Tensor, w: DevWeight, ldo: int, cm: "CommSend", rows_per_rank: int) -> None:
    """Dequantisation-fused variant of :func:`gemm_bf16_scatter`."""
    m, k = x.shape
    x = x.contiguous()
    d = w.desc()
    f = lib().b2_gemm_q_scatter
    f.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p]
    _check(f(ptr(x), m, C.addressof(d), ldo, C.addressof(cm), rows_per_rank, stream()), "gemm_q_scatter")


class SampleRow(C.Structure):
    _fields_ = [("n_hist", C.c_int), ("hist_off", C.c_int), ("u", C.c_float)]


class SampleArgs(C.Structure):
    _fields_ = [("logits", C.c_void_p), ("ld", C.c_int), ("vocab", C.c_int), ("rows", C.c_void_p), ("hist_ids", C.c_void_p),
                ("hist_counts", C.c_void_p), ("repeat_penalty", C.c_float), ("freq_penalty", C.c_float), ("presence_penalty", C.c_float),
                ("top_k", C.c_int), ("top_p", C.c_float), ("min_p", C.c_float), ("temperature", C.c_float), ("out_token", C.c_void_p),
                ("out_prob", C.c_void_p), ("cand_idx", C.c_void_p), ("cand_prob", C.c_void_p), ("cand_n", C.c_void_p)]


SAMPLE_MAX_K = 256


def sample(logits: torch.Tensor, us: list[float], top_k: int, top_p: float, min_p: float, temperature: float,
           history: list[dict[int, int]] | None = None, repeat_penalty: float = 1.0, freq_penalty: float = 0.0, presence_penalty: float = 0.0,
           want_candidates: bool = False):
    """Draw one token per row of ``logits`` [rows, vocab] (fp32, modified in place by the penalties) on the device.

    ``us``: one uniform number per row; ``history``: per row, token id -> count inside the penalty window.
    Returns the ids (int32 tensor on the device) or, with ``want_candidates``, (ids, probs, cand_idx, cand_prob, cand_n).
    """
    rows, vocab = logits.shape
    dev = logits.device
    meta = torch.zeros(rows, 3, dtype=torch.int32)
    ids, cnts = [], []
    for r in range(rows):
        h = history[r] if history else {}
        meta[r, 0], meta[r, 1] = len(h), len(ids)
        ids += list(h.keys())
        cnts += list(h.values())
    meta[:, 2] = torch.tensor(us, dtype=torch.float32).view(torch.int32)
    meta_d = meta.to(dev)
    ids_d = torch.tensor(ids or [0], dtype=torch.int32, device=dev)
    cnt_d = torch.tensor(cnts or [0], dtype=torch.int32, device=dev)
    out = torch.empty(rows, dtype=torch.int32, device=dev)
    prob = torch.empty(rows, dtype=torch.float32, device=dev)
    ci = cp = cn = None
    if want_candidates:
        ci = torch.empty(rows, SAMPLE_MAX_K, dtype=torch.int32, device=dev)
        cp = torch.empty(rows, SAMPLE_MAX_K, dtype=torch.float32, device=dev)
        cn = torch.empty(rows, dtype=torch.int32, device=dev)
    a = SampleArgs(ptr(logits), logits.stride(0), vocab, ptr(meta_d), ptr(ids_d), ptr(cnt_d), repeat_penalty, freq_penalty, presence_penalty,
                   top_k, top_p, min_p, temperature, ptr(out), ptr(prob), ptr(ci), ptr(cp), ptr(cn))
    _check(lib().b2_sample(C.byref(a), rows, stream()), "sample")
    return (out, prob, ci, cp, cn) if want_candidates else out


class GluRowsArgs(C.Structure):
    _fields_ = [("gu", C.c_void_p), ("out", C.c_void_p), ("f", C.c_int), ("act", C.c_int), ("alpha", C.c_float), ("limit", C.c_float)]


def glu_rows(gu: torch.Tensor, act: str, alpha: float = 1.702, limit: float = 7.0) -> torch.Tensor:
    """Gated activation on a bf16 [rows, 2F] gate/up GEMM result with interleaved columns -> bf16 [rows, F]."""
    rows, f2 = gu.shape
    out = torch.empty(rows, f2 // 2, device=gu.device, dtype=torch.bfloat16)
    a = GluRowsArgs(ptr(gu), ptr(out), f2 // 2, _ACT[act], alpha, limit)
    _check(lib().b2_glu_rows(C.byref(a), rows, stream()), "glu_rows")
    return out


def rmsnorm_bf16(x: torch.Tensor, w: torch.Tensor | None, eps: float, do_norm: bool = True) -> torch.Tensor:
    """Row-wise RMSNorm of fp32 [rows, k] with a bf16 result (the A operand of the prefill GEMMs)."""
    rows, k = x.shape
    out = torch.empty(rows, k, device=x.device, dtype=torch.bfloat16)
    a = NormCastArgs(ptr(x), ptr(w), eps, k, int(do_norm), ptr(out))
    _check(lib().b2_rmsnorm_bf16(C.byref(a), rows, stream()), "rmsnorm_bf16")
    return out


class AttnPrefillArgs(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("out", C.c_void_p), ("sinks", C.c_void_p),
                ("T", C.c_int), ("H", C.c_int), ("Hkv", C.c_int), ("n_ctx", C.c_int), ("slot", C.c_int), ("pos0", C.c_int),
                ("kv_len", C.c_int), ("causal", C.c_int), ("window", C.c_int), ("scale", C.c_float), ("softcap", C.c_float),
                ("k_scale", C.c_void_p), ("v_scale", C.c_void_p)]


ATTN_PREFILL_HEAD_DIMS = (32, 64, 128, 256)
ATTN_PREFILL_DEFAULT = "auto"       # the kernel prefill attention runs on unless told otherwise (see attn_prefill)


def attn_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, slot: int, pos0: int, kv_len: int, scale: float,
                 causal: bool = True, window: int = 0, softcap: float = 0.0, sinks: torch.Tensor | None = None,
                 k_scale: torch.Tensor | None = None, v_scale: torch.Tensor | None = None, mode: str | None = None) -> torch.Tensor:
    """Flash attention of a prefill chunk: q [T, H, D] fp32 -> bf16 [T, H * D].  ``mode``: "tc" = the tcgen05 kernel
    (kernels/attn_prefill_tc.cu: f16 caches, head size 64 / 128), "mma" = the mma.sync kernel (kernels/attn_prefill.cu), "auto" =
    tcgen05 where it applies.  Default: B200_ATTN_PREFILL, else ATTN_PREFILL_DEFAULT."""
    T, H, D = q.shape
    n_slots, Hkv, n_ctx, _ = k_cache.shape
    out = torch.empty(T, H * D, device=q.device, dtype=torch.bfloat16)
    a = AttnPrefillArgs(ptr(q.contiguous()), ptr(k_cache), ptr(v_cache), ptr(out), ptr(sinks), T, H, Hkv, n_ctx, slot, pos0, kv_len,
                        int(causal), window, scale, softcap, ptr(k_scale), ptr(v_scale))
    mode = mode or os.environ.get("B200_ATTN_PREFILL", ATTN_PREFILL_DEFAULT)
    if mode in ("auto", "tc") and D in (64, 128) and k_scale is None and q.dtype == torch.float32:
        rc = lib().b2_attn_prefill_tc(C.byref(a), D, n_slots, stream())
        if rc == 0:
            return out
        if rc != 801 or mode == "tc":              # 801 = cudaErrorNotSupported: nothing was launched
            _check(rc, "attn_prefill_tc")
    elif mode == "tc":
        raise RuntimeError("attn_prefill: the tcgen05 kernel takes f16 caches and head size 64 or 128")
    _check(lib().b2_attn_prefill(C.byref(a), D, stream()), "attn_prefill")
    return out


def attn_prefill_tc_variant(v: int) -> int:
    """Where the tcgen05 attention kernel keeps the probabilities between its two products: 0 = a shared-memory tile,
    1 = TMEM (they overwrite the scores and feed the second product from there), 2 = the pipelined kernel (two score buffers and
    two output tiles in TMEM, the accumulation of a tile deferred behind the next tile's softmax).  Returns the previous setting."""
    return int(lib().b2_attn_prefill_tc_variant(int(v)))


def attn_prefill_tc_status(clear: bool = False) -> int:
    """0 = ok; 1 = a bounded wait inside the tcgen05 attention kernel expired (the result of that launch is not valid)."""
    v = int(lib().b2_attn_prefill_tc_status())
    if clear and v:
        lib().b2_attn_prefill_tc_clear_status()
    return v


def gemm_status() -> int:
    """0 = ok; 1 = a bounded wait inside a tensor-core kernel (the GEMMs, the tcgen05 attention) expired."""
    return int(lib().b2_gemm_status()) | int(lib().b2_gemm_q_status()) | int(lib().b2_attn_prefill_tc_status()) | int(lib().b2_gemm_q_grouped_status())


GEMM_Q_TYPES = {WT_Q4_K, WT_Q6_K, WT_Q8_0, WT_BF16, WT_F16}


def gemm_q_supported(w: DevWeight) -> bool:
    if w.wtype not in GEMM_Q_TYPES or w.n % 4:
        return False
    return w.k % (256 if w.wtype in (WT_Q4_K, WT_Q6_K) else 64) == 0


def gemm_q(x: torch.Tensor, w: DevWeight, out: torch.Tensor | None = None, accumulate: bool = False, out_off: int = 0) -> torch.Tensor:
    """out[:, out_off:out_off+n] (+)= x[m, k] (bf16) @ dequant(w)[n, k]^T + bias, weights expanded inside the tensor-core kernel."""
    m, k = x.shape
    if x.dtype != torch.bfloat16 or k != w.k:
        raise ValueError("gemm_q needs a bf16 activation matrix [m, k] matching the weight")
    x = x.contiguous()
    if out is None:
        out = torch.empty(m, w.n, device=x.device, dtype=torch.float32)
    d = w.desc(out_off=out_off)
    f = lib().b2_gemm_q
    f.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
    _check(f(ptr(x), m, C.addressof(d), ptr(out), out.stride(0), int(accumulate), stream()), "gemm_q")
    return out


# ---------------------------------------------------------------------------------------------------
# grouped mixture-of-experts prefill
# ---------------------------------------------------------------------------------------------------
class MoePlanArgs(C.Structure):
    _fields_ = [("lids", C.c_void_p), ("pairs", C.c_int), ("n_experts", C.c_int), ("row_of_pair", C.c_void_p), ("tile_expert", C.c_void_p),
                ("max_tiles", C.c_int)]


def moe_plan(lids: torch.Tensor, n_experts: int) -> tuple[torch.Tensor, torch.Tensor, int]:
    """Rows of a buffer sorted by expert for the (token, expert-slot) pairs ``lids`` (local expert or -1): returns
    (row_of_pair int32 [pairs], tile_expert int32 [tiles], padded row count).  Every expert's rows start at a multiple of 128."""
    pairs = lids.numel()
    max_tiles = (pairs + 127) // 128 + n_experts
    row = torch.empty(pairs, dtype=torch.int32, device=lids.device)
    te = torch.empty(max_tiles, dtype=torch.int32, device=lids.device)
    a = MoePlanArgs(ptr(lids), pairs, n_experts, ptr(row), ptr(te), max_tiles)
    _check(lib().b2_moe_plan(C.byref(a), stream()), "moe_plan")
    return row, te, max_tiles * 128


def moe_gather(h: torch.Tensor, row_of_pair: torch.Tensor, k: int, rows: int) -> torch.Tensor:
    """bf16 activation rows [T, d] -> [rows, d] sorted by expert (rows nobody owns are left as they are)."""
    xs = torch.empty(rows, h.shape[1], dtype=torch.bfloat16, device=h.device)
    f = lib().b2_moe_gather
    f.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
    _check(f(ptr(h), ptr(row_of_pair), row_of_pair.numel(), k, h.shape[1], ptr(xs), stream()), "moe_gather")
    return xs


def moe_scatter_combine(ys: torch.Tensor, row_of_pair: torch.Tensor, wts: torch.Tensor, tokens: int, k: int, out: torch.Tensor | None = None,
                        accumulate: bool = False) -> torch.Tensor:
    d = ys.shape[1]
    if out is None:
        out = torch.empty(tokens, d, dtype=torch.float32, device=ys.device)
    f = lib().b2_moe_scatter_combine
    f.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p]
    _check(f(ptr(ys), ptr(row_of_pair), ptr(wts), tokens, k, d, ptr(out), int(accumulate), stream()), "moe_scatter_combine")
    return out


def gemm_bf16_grouped(a: torch.Tensor, b: torch.Tensor, experts: int, tile_expert: torch.Tensor, bias: torch.Tensor | None = None,
                      glu: str | None = None, alpha: float = 1.702, limit: float = 7.0) -> torch.Tensor:
    """One launch over all experts: a [m, k] bf16 sorted by expert in 128-row tiles, b [experts * n, k] bf16.  Returns fp32 [m, n], or
    with ``glu`` (activation name) the gated activation of interleaved gate/up columns as bf16 [m, n / 2]."""
    m, k = a.shape
    n = b.shape[0] // experts
    a, b = a.contiguous(), b.contiguous()
    out = torch.empty(m, n // 2, device=a.device, dtype=torch.bfloat16) if glu else torch.empty(m, n, device=a.device, dtype=torch.float32)
    f = lib().b2_gemm_bf16_grouped
    f.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_float,
                  C.c_float, C.c_void_p]
    _check(f(ptr(a), ptr(b), m, n, k, experts, ptr(tile_expert), ptr(out), out.stride(0), ptr(bias), _ACT[glu] if glu else -1, alpha, limit,
             stream()), "gemm_bf16_grouped")
    return out


def gemm_q_grouped_supported(w: DevWeight) -> bool:
    """True when the expert stack ``w`` can be streamed in its own encoding by :func:`gemm_q_grouped` (MXFP4, k % 64 == 0)."""
    return w.wtype == WT_MXFP4 and w.k % 64 == 0 and w.n % 8 == 0


def gemm_q_grouped(a: torch.Tensor, w: DevWeight, tile_expert: torch.Tensor, glu: str | None = None, alpha: float = 1.702,
                   limit: float = 7.0) -> torch.Tensor | None:
    """The grouped product of :func:`gemm_bf16_grouped` with the experts read as MXFP4 blocks and expanded inside the kernel
    (kernels/gemm_q_grouped.cu).  ``w``: the stacked experts (``w.experts`` matrices of ``w.n`` rows, with their biases).
    Returns fp32 [m, n], with ``glu`` bf16 [m, n / 2], or None when the kernel does not take the encoding or shape (nothing
    was launched)."""
    m, k = a.shape
    n, experts = w.n, max(w.experts, 1)
    if a.dtype != torch.bfloat16 or k != w.k or m % 128 or not gemm_q_grouped_supported(w):
        return None
    a = a.contiguous()
    out = torch.empty(m, n // 2, device=a.device, dtype=torch.bfloat16) if glu else torch.empty(m, n, device=a.device, dtype=torch.float32)
    d = w.desc()
    f = lib().b2_gemm_q_grouped
    f.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_float, C.c_float, C.c_void_p]
    rc = f(ptr(a), m, C.addressof(d), experts, ptr(tile_expert), ptr(out), out.stride(0), d.bias, _ACT[glu] if glu else -1, alpha, limit, stream())
    if rc == 801:
        return None
    _check(rc, "gemm_q_grouped")
    return out


def gemm_bf16_glu(a: torch.Tensor, b: torch.Tensor, act: str, bias: torch.Tensor | None = None, alpha: float = 1.702, limit: float = 7.0) -> torch.Tensor:
    """Gate/up product of a dense FFN with the gated activation in the GEMM epilogue: bf16 [m, n / 2]."""
    m, k = a.shape
    n = b.shape[0]
    a, b = a.contiguous(), b.contiguous()
    out = torch.empty(m, n // 2, device=a.device, dtype=torch.bfloat16)
    f = lib().b2_gemm_bf16_glu
    f.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_float, C.c_float, C.c_void_p]
    _check(f(ptr(a), ptr(b), m, n, k, ptr(out), out.stride(0), ptr(bias), _ACT[act], alpha, limit, stream()), "gemm_bf16_glu")
    return out
