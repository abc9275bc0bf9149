"""Tile-major weight layout and bindings of the streaming decode GEMV (``kernels/gemv_sk.cu``).

A Q4_K / Q6_K matrix [n, k] (n % 16 == 0, k % 256 == 0) becomes ``[n / 16][k / 256]`` units.  A unit holds
one super-block of each of 16 rows in the order in which the lanes of a warp load their tensor-core A fragments,
followed by the rows' scales: 3360 bytes for Q6_K (the size of the 16 GGUF blocks it was made from) and 2368 bytes for Q4_K
(2304 in GGUF; the packed 6-bit scale table is stored as bytes).
``unit_weights`` restates the lane maps of the kernel in tensor ops and decodes units back to floats, so the layout
is checked on the CPU against the block codecs.

The reference's counterpart is the block layout consumed by ggml's mmvq kernels (fs/ggml/type.go type sizes).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from ..gguf import quants
from ..gguf.types import GGMLType
from ..models.weights import QWeight
from . import cuda as K

UNIT_BYTES = {K.WT_Q4_K: 2368, K.WT_Q6_K: 3360}
WS_FLOATS = 16 * 32
MAX_TOKENS = 32


class SkSeg(C.Structure):
    _fields_ = [("w", C.c_void_p), ("bias", C.c_void_p), ("type", C.c_int), ("n", C.c_int), ("out_off", C.c_int), ("unit0", C.c_int)]


class SkArgs(C.Structure):
    _fields_ = [("seg", SkSeg * 4), ("nseg", C.c_int), ("k", C.c_int), ("nb", C.c_int), ("total_units", C.c_int),
                ("x", C.c_void_p), ("ldx", C.c_int), ("norm_w", C.c_void_p), ("eps", C.c_float), ("xq", C.c_void_p), ("xd", C.c_void_p), ("xbs", C.c_void_p),
                ("mode", C.c_int), ("out", C.c_void_p), ("ldo", C.c_int), ("act", C.c_int), ("alpha", C.c_float), ("limit", C.c_float),
                ("ws", C.c_void_p), ("flags", C.c_void_p), ("status", C.c_void_p),
                ("off_red", C.c_int), ("off_xq", C.c_int), ("off_xd", C.c_int), ("off_xbs", C.c_int), ("off_ring", C.c_int), ("ring", C.c_int),
                ("slot_bytes", C.c_int), ("wpt_log2", C.c_int), ("n_groups", C.c_int),
                ("cm", K.CommSend)]


MAX_PHASES = 4
TUNE = int(__import__('os').environ.get('B200_SK_TUNE', '0'))      # kernel experiments (see SkChain.tune in kernels/gemv_sk.cu)


class SkChain(C.Structure):
    _fields_ = [("ph", SkArgs * MAX_PHASES), ("n", C.c_int), ("bar", C.c_void_p), ("tune", C.c_int), ("trace", C.c_void_p)]


class Quant256Args(C.Structure):
    _fields_ = [("x", C.c_void_p), ("ldx", C.c_int), ("norm_w", C.c_void_p), ("eps", C.c_float), ("k", C.c_int), ("xq", C.c_void_p),
                ("xd", C.c_void_p), ("xbs", C.c_void_p), ("perm", C.c_int)]


MODE_STORE, MODE_ACCUM, MODE_GLU = 0, 1, 2


@dataclass
class SkWeight:
    """A matrix in unit order: ``units`` is uint8 [n / 16, k / 256, unit bytes]."""

    wtype: int
    n: int
    k: int
    units: torch.Tensor
    bias: torch.Tensor | None = None
    name: str = ""

    @property
    def nbytes(self) -> int:
        return self.units.numel() + (self.bias.numel() * 4 if self.bias is not None else 0)

    def seg(self, out_off: int = 0) -> SkSeg:
        s = SkSeg()
        s.w, s.bias = self.units.data_ptr(), (self.bias.data_ptr() if self.bias is not None else None)
        s.type, s.n, s.out_off, s.unit0 = self.wtype, self.n, out_off, 0
        return s


def supported(dtype: GGMLType, n: int, k: int) -> bool:
    return dtype in (GGMLType.Q4_K, GGMLType.Q6_K) and n % 16 == 0 and k % 256 == 0 and n > 0


def _pack_q4k(raw: torch.Tensor, n: int, k: int) -> torch.Tensor:
    nsb, nt = k // 256, n // 16
    blk = raw.view(n, nsb, 144)
    sc, mn = quants._scale_min_k4(blk[:, :, 4:16].reshape(-1, 12))
    # row = 16 tile + 8 il + g, nibble byte = 32 p + 16 ih + 4 t + b  ->  [tile][sb][p][g][t][ih][il][b]: lane (g, t) reads 16 bytes,
    # word i = 2 ih + il
    q = blk[:, :, 16:].reshape(nt, 2, 8, nsb, 4, 2, 4, 4).permute(0, 3, 4, 2, 6, 5, 1, 7).reshape(nt, nsb, 2048)
    scm = torch.cat([sc.to(torch.uint8).view(n, nsb, 8), mn.to(torch.uint8).view(n, nsb, 8)], 2)
    scm = scm.view(nt, 16, nsb, 16).permute(0, 2, 1, 3).reshape(nt, nsb, 256)
    dd = blk[:, :, :4].reshape(nt, 16, nsb, 4).permute(0, 2, 1, 3).reshape(nt, nsb, 64)
    return torch.cat([q, scm, dd], 2).contiguous()


def _q6k_codes(blk: torch.Tensor) -> torch.Tensor:
    """Q6_K blocks [N, 210] -> the 6-bit codes q (0..63) in element order, int32 [N, 256]."""
    n = blk.shape[0]
    i32 = torch.int32
    ql = blk[:, 0:128].to(i32).view(n, 2, 64)
    qh = blk[:, 128:192].to(i32).view(n, 2, 32)
    l0, l1 = ql[:, :, 0:32], ql[:, :, 32:64]
    q1 = (l0 & 15) | (((qh >> 0) & 3) << 4)
    q2 = (l1 & 15) | (((qh >> 2) & 3) << 4)
    q3 = (l0 >> 4) | (((qh >> 4) & 3) << 4)
    q4 = (l1 >> 4) | (((qh >> 6) & 3) << 4)
    return torch.stack([q1, q2, q3, q4], 2).reshape(n, 256)


def _pack_q6k(raw: torch.Tensor, n: int, k: int) -> torch.Tensor:
    nsb, nt = k // 256, n // 16
    blk = raw.view(n * nsb, 210)
    s = ((_q6k_codes(blk) - 32) & 63).view(nt, 2, 8, nsb, 8, 2, 4, 4)          # [tile][il][g][sb][G][jj][t][b]; column = 32 G + 16 jj + 4 t + b
    r = s.permute(0, 3, 4, 2, 6, 5, 1, 7).reshape(nt, nsb, 8, 32, 4, 4)         # [tile][sb][G][lane][i = 2 jj + il][b]
    r3 = r[:, :, :, :, 3]
    words = torch.stack([(r[:, :, :, :, i] << 2) | ((r3 >> (4 - 2 * i)) & 3) for i in range(3)], 4)   # [tile][sb][G][lane][3][b]
    words = words.permute(0, 1, 3, 2, 4, 5).reshape(nt, nsb, 32, 6, 4, 4)       # lane-major: 24 words = 6 chunks of 4
    codes = words.permute(0, 1, 3, 2, 4, 5).reshape(nt, nsb, 3072).to(torch.uint8)
    blk3 = raw.view(n, nsb, 210)
    sc = blk3[:, :, 192:208].reshape(nt, 16, nsb, 16).permute(0, 2, 1, 3).reshape(nt, nsb, 256)
    d = blk3[:, :, 208:210].reshape(nt, 16, nsb, 2).permute(0, 2, 1, 3).reshape(nt, nsb, 32)
    return torch.cat([codes, sc, d], 2).contiguous()


def repack(w: QWeight, device, bias: torch.Tensor | None = None) -> SkWeight:
    """GGUF blocks of a Q4_K / Q6_K matrix -> units on ``device``."""
    if len(w.shape) != 2 or not supported(w.dtype, *w.shape):
        raise ValueError(f"{w.name}: {w.dtype.name} {w.shape} has no unit layout")
    n, k = w.shape
    raw = w.raw.to(device)
    b = bias.to(device=device, dtype=torch.float32).contiguous() if bias is not None else None
    if w.dtype == GGMLType.Q4_K:
        return SkWeight(K.WT_Q4_K, n, k, _pack_q4k(raw, n, k), b, w.name)
    # Q6_K goes through int32 intermediates: pack large matrices in slabs of rows
    step = max(16, (1 << 24) // k // 16 * 16)
    parts = [_pack_q6k(raw.view(n, -1)[r0:r0 + step].reshape(-1), min(step, n - r0), k) for r0 in range(0, n, step)]
    return SkWeight(K.WT_Q6_K, n, k, torch.cat(parts, 0).contiguous() if len(parts) > 1 else parts[0], b, w.name)


def interleave(a: QWeight, b: QWeight) -> QWeight:
    """Rows of two equally shaped and encoded matrices alternated (2i = a[i], 2i + 1 = b[i]): the FFN gate/up pair."""
    if a.dtype != b.dtype or a.shape != b.shape or len(a.shape) != 2:
        raise ValueError("interleave needs two matrices of the same encoding and shape")
    n = a.shape[0]
    raw = torch.stack([a.raw.view(n, -1), b.raw.view(n, -1)], 1).reshape(-1)
    return QWeight(a.name + "+" + b.name, a.dtype, (2 * n, a.shape[1]), raw)


def unit_weights(w: SkWeight) -> torch.Tensor:
    """Decode the units back to a float matrix [n, k] by following the kernel's lane maps (checks the layout, any device)."""
    u = w.units
    nt, nsb = u.shape[0], u.shape[1]
    i32 = torch.int32
    if w.wtype == K.WT_Q4_K:
        q = u[:, :, :2048].to(i32).view(nt, nsb, 4, 8, 4, 2, 2, 4)              # [tile][sb][p][g][t][ih][il][b]
        scm = u[:, :, 2048:2304].to(i32).view(nt, nsb, 16, 16)                   # [tile][sb][row][sc0..7 m0..7]
        dd = u[:, :, 2304:2368].contiguous().view(torch.float16).float().view(nt, nsb, 16, 2)
        out = torch.empty(nt, 16, nsb, 256, dtype=torch.float32, device=u.device)
        for p in range(4):
            for half, code in ((0, q[:, :, p] & 15), (1, q[:, :, p] >> 4)):      # sub-block 2p from the low, 2p + 1 from the high nibbles
                j = 2 * p + half
                # code: [tile][sb][g][t][ih][il][b] -> row 8 il + g, column 16 ih + 4 t + b of sub-block j
                c = code.permute(0, 5, 2, 1, 4, 3, 6).reshape(nt, 16, nsb, 32).float()
                sc = scm[:, :, :, j].permute(0, 2, 1).float()
                mn = scm[:, :, :, 8 + j].permute(0, 2, 1).float()
                d, dmin = dd[..., 0].permute(0, 2, 1), dd[..., 1].permute(0, 2, 1)
                out[:, :, :, 32 * j:32 * j + 32] = (d * sc)[..., None] * c - (dmin * mn)[..., None]
        return out.reshape(nt * 16, nsb * 256)
    words = u[:, :, :3072].to(i32).view(nt, nsb, 6, 32, 4, 4).permute(0, 1, 3, 2, 4, 5).reshape(nt, nsb, 32, 8, 3, 4)   # [..][lane][G][i][b]
    r = [words[..., i, :] >> 2 for i in range(3)]
    r.append(((words[..., 0, :] & 3) << 4) | ((words[..., 1, :] & 3) << 2) | (words[..., 2, :] & 3))
    code = torch.stack(r, 4)                                                     # [tile][sb][lane][G][i][b], 6-bit two's complement
    code = torch.where(code >= 32, code - 64, code).view(nt, nsb, 8, 4, 8, 2, 2, 4)   # [tile][sb][g][t][G][jj][il][b]
    vals = code.permute(0, 6, 2, 1, 4, 5, 3, 7).reshape(nt, 16, nsb, 256).float()  # row 8 il + g, column 32 G + 16 jj + 4 t + b
    sc = u[:, :, 3072:3328].contiguous().view(torch.int8).float().view(nt, nsb, 16, 16).permute(0, 2, 1, 3)            # [tile][row][sb][16]
    d = u[:, :, 3328:3360].contiguous().view(torch.float16).float().view(nt, nsb, 16).permute(0, 2, 1)
    out = vals.view(nt, 16, nsb, 16, 16) * (d[..., None] * sc)[..., None]
    return out.reshape(nt * 16, nsb * 256)


class Workspace:
    """Hand-over buffers of split tiles and the status word, one set per device (launches of one stream share it)."""

    def __init__(self, device):
        rows = int(K.lib().b2_gemv_sk_max_groups())
        self.ws = torch.zeros(rows * WS_FLOATS, device=device, dtype=torch.float32)
        self.flags = torch.zeros(rows, device=device, dtype=torch.int32)
        self.status = torch.zeros(1, device=device, dtype=torch.int32)
        self.bar = torch.zeros(2, device=device, dtype=torch.int32)          # arrival / exit counters of multi-phase launches

    def check(self) -> None:
        """Raise if a bounded wait inside a launch gave up; the flags are cleared so the next launch starts clean."""
        if int(self.status.item()) != 0:
            self.status.zero_()
            self.flags.zero_()
            self.bar.zero_()
            raise K.CudaKernelError("streaming GEMV: a bounded wait ran out")


_workspaces: dict = {}


def workspace(device) -> Workspace:
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    if key not in _workspaces:
        _workspaces[key] = Workspace(torch.device("cuda", key))
    return _workspaces[key]


def fits_fused_input(nb: int, k: int) -> bool:
    """True when the GEMV should normalise / quantise its nb x k fp32 input itself (every CTA repeats that work, so it only pays
    for small inputs: at most two rounds of loads per warp, and room left in shared memory for the weight rings)."""
    return nb * (k // 256) <= 32 and nb * (k + 16 + k // 64 + k // 16) <= 24 * 1024


def quant256(x: torch.Tensor, norm_w: torch.Tensor | None = None, eps: float = 0.0, out: tuple | None = None, pdl: bool = False) -> tuple:
    """int8 rows with one fp32 scale per 256 elements and the int16 sum of every 32 values (optionally RMS-normalised
    first): the pre-quantised GEMV input (xq, xd, xbs).  A single row is stored in the word order the one-token GEMV reads
    (inside every 256-block: [column quarter t][16-column group]); see :func:`natural_order`."""
    nb, k = x.shape
    xq, xd, xbs = out if out is not None else (torch.empty(nb, k, device=x.device, dtype=torch.int8),
                                               torch.empty(nb, k // 256, device=x.device, dtype=torch.float32),
                                               torch.empty(nb, k // 32, device=x.device, dtype=torch.int16))
    a = Quant256Args(K.ptr(x), x.stride(0), K.ptr(norm_w), eps, k, K.ptr(xq), K.ptr(xd), K.ptr(xbs), int(nb == 1))
    K._check(K.lib().b2_quant256(C.byref(a), nb, int(pdl), K.stream()), "quant256")
    return xq, xd, xbs


def natural_order(xq: torch.Tensor) -> torch.Tensor:
    """The int8 values of a one-row :func:`quant256` result in element order."""
    k = xq.shape[-1]
    return xq.view(-1, k // 256, 4, 16, 4).permute(0, 1, 3, 2, 4).reshape(-1, k)


def fill_args(a: SkArgs, weights: list[SkWeight], nb: int, ws: Workspace) -> None:
    off = 0
    for i, w in enumerate(weights):
        a.seg[i] = w.seg(out_off=off)
        off += w.n
    a.nseg, a.k, a.nb = len(weights), weights[0].k, nb
    a.ws, a.flags, a.status = ws.ws.data_ptr(), ws.flags.data_ptr(), ws.status.data_ptr()


def gemv(weights: list[SkWeight], x: torch.Tensor | tuple[torch.Tensor, torch.Tensor], *, norm_w: torch.Tensor | None = None, eps: float = 0.0,
         out: torch.Tensor | None = None, mode: int = MODE_STORE, act: str = "silu", alpha: float = 1.702, limit: float = 7.0,
         max_ctas: int = 0, split: int = 0, ring: int = 0, pdl: bool = False) -> torch.Tensor:
    """y[b] = concat_i(W_i x[b] + bias_i) for 1..32 tokens.

    ``x``: fp32 rows [nb, k] (normalised with ``norm_w`` and quantised inside the kernel) or the (int8, scales) pair of
    :func:`quant256`.  ``mode``: store, add to ``out``, or gated activation of interleaved gate/up rows ([nb, n / 2]).
    """
    pre = isinstance(x, tuple)
    nb = (x[0] if pre else x).shape[0]
    total = sum(w.n for w in weights)
    dev = weights[0].units.device
    if out is None:
        out = torch.empty(nb, total // 2 if mode == MODE_GLU else total, device=dev, dtype=torch.float32)
    a = SkArgs()
    fill_args(a, weights, nb, workspace(dev))
    if pre:
        a.xq, a.xd, a.xbs = x[0].data_ptr(), x[1].data_ptr(), x[2].data_ptr()
    else:
        a.x, a.ldx, a.norm_w, a.eps = x.data_ptr(), x.stride(0), K.ptr(norm_w), eps
    a.mode, a.out, a.ldo = mode, out.data_ptr(), out.stride(0)
    a.act, a.alpha, a.limit = K._ACT[act], alpha, limit
    K._check(K.lib().b2_gemv_sk(C.byref(a), max_ctas, split, ring, int(pdl), K.stream()), "gemv_sk")
    return out


def phase(weights: list[SkWeight], x: torch.Tensor, out: torch.Tensor, *, norm_w: torch.Tensor | None = None, eps: float = 0.0,
          mode: int = MODE_STORE, act: str = "silu", alpha: float = 1.702, limit: float = 7.0) -> SkArgs:
    """One product of a multi-phase launch: fp32 rows ``x`` [nb, k] in, ``out`` written / added to / gated (see :func:`gemv`)."""
    a = SkArgs()
    fill_args(a, weights, x.shape[0], workspace(weights[0].units.device))
    a.x, a.ldx, a.norm_w, a.eps = x.data_ptr(), x.stride(0), K.ptr(norm_w), eps
    a.mode, a.out, a.ldo = mode, out.data_ptr(), out.stride(0)
    a.act, a.alpha, a.limit = K._ACT[act], alpha, limit
    return a


def gemv_chain(phases: list[SkArgs], device, max_ctas: int = 0, split: int = 0, ring: int = 0, pdl: bool = False,
               trace: torch.Tensor | None = None) -> None:
    """Run up to four products back to back in one launch; every phase may read what earlier phases wrote."""
    if not 1 <= len(phases) <= MAX_PHASES:
        raise ValueError(f"a chain has 1..{MAX_PHASES} phases")
    c = SkChain()
    for i, a in enumerate(phases):
        c.ph[i] = a
    c.n, c.bar = len(phases), workspace(device).bar.data_ptr()
    c.tune = TUNE
    c.trace = trace.data_ptr() if trace is not None else None      # int64 [grid, 16]: time stamps of thread 0 of every CTA
    K._check(K.lib().b2_gemv_sk_chain(C.byref(c), max_ctas, split, ring, int(pdl), K.stream()), "gemv_sk_chain")
