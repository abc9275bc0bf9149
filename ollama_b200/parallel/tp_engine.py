"""Tensor-parallel execution of one model over the GPUs of an NVLink / NVSwitch node.

One process per GPU.  Attention heads, KV cache and FFN columns are split N ways (Q/K/V and gate/up are
column-parallel, attention-output and FFN-down are row-parallel), the vocabulary projection is split by
rows, norms and the token embedding are replicated.  Every rank runs the same sequence of calls (SPMD).

Decode (1..8 sequences per step): the row-parallel GEMV writes its partial output rows, each value tagged
with the exchange's epoch, straight into a receive buffer on every rank; the following fused add + RMSNorm
+ quantise kernel polls the words of that epoch, sums the N partial rows into its replica of the residual
stream and carries on.  There is no separate all-reduce kernel, no fence and no flag on this path, and the
whole step still replays as one CUDA graph per rank.

Prefill: the residual stream is sharded by token rows.  The row-parallel GEMM stores each partial tile
into the owner of those rows (GEMM + reduce-scatter in one kernel), and one kernel per exchange does
reduction + residual add + RMSNorm + bf16 conversion + all-gather into every rank's activation buffer.

Reference: multi-GPU placement and splits in llm/server.go (GPU layer assignment) and
ml/backend/ggml/ggml.go (tensor splits over devices); the measured baseline runs layer-split pipelines.
"""
from __future__ import annotations

import ctypes as C
import dataclasses
from typing import Sequence

import torch

from ..engine.b200 import MAX_DECODE_BATCH, B200Backend, supports
from ..gguf.types import GGMLType, block_size
from ..models.config import ModelConfig
from ..models.weights import QWeight
from ..ops import cuda as K
from ..ops import reference as R
from .comm import Layout, PeerRegion

CH_DEC, CH_LOGITS, CH_RS, CH_AG, CH_BAR = 0, 1, 2, 3, 4


class TpNormGatherArgs(C.Structure):
    _fields_ = [("x", C.c_void_p), ("parts", C.c_void_p), ("n_part", C.c_int), ("part_stride", C.c_longlong), ("rs_chan", C.c_void_p),
                ("w", C.c_void_p), ("eps", C.c_float), ("k", C.c_int), ("row0", C.c_int), ("ag", K.CommSend)]


def shard_plan(cfg: ModelConfig, world: int, types: dict[str, int] | None = None) -> dict:
    """Per-rank sizes of a tensor-parallel split, or a ValueError saying why ``world`` does not divide the model."""
    kv_rep = 1                     # ranks that share one KV head (its projection and cache are replicated on them)
    if cfg.n_kv_heads % world:
        if world % cfg.n_kv_heads:
            raise ValueError(f"{world} ranks neither divide nor are a multiple of {cfg.n_kv_heads} KV heads")
        kv_rep = world // cfg.n_kv_heads
    if cfg.n_heads % world:
        raise ValueError(f"{world} ranks do not divide {cfg.n_heads} heads")
    if cfg.d_ff % world:
        raise ValueError(f"{world} ranks do not divide the FFN width {cfg.d_ff}")
    if cfg.is_moe and cfg.n_experts % world:
        raise ValueError(f"{world} ranks do not divide {cfg.n_experts} experts")
    hl, kvl, fl = cfg.n_heads // world, max(cfg.n_kv_heads // world, 1), cfg.d_ff // world
    for name, cols in (("attn_output", hl * cfg.head_dim),) + (() if cfg.is_moe else (("ffn_down", fl),)):
        bs = max([block_size(t) for n, t in (types or {}).items() if n.endswith(name + ".weight")] or [256])
        if cols % bs:
            raise ValueError(f"{name}: {cols} columns per rank do not fall on {bs}-element quantisation blocks")
    if fl % 32 and not cfg.is_moe:       # expert models have no dense FFN to split
        raise ValueError(f"FFN width per rank {fl} is not a multiple of 32")
    vl = (cfg.vocab_size + world - 1) // world
    vl = (vl + 7) // 8 * 8
    return {"heads": hl, "kv_heads": kvl, "kv_rep": kv_rep, "d_ff": fl, "vocab_rows": vl, "experts": cfg.n_experts // world if cfg.is_moe else 0}


class ShardedTensors:
    """Presents one rank's slice of every tensor of ``src`` (a mapping name -> QWeight)."""

    def __init__(self, src, cfg: ModelConfig, rank: int, world: int):
        self.src, self.cfg, self.rank, self.world = src, cfg, rank, world
        types = {n: src.type_of(n) for n in src.keys()} if hasattr(src, "type_of") else None
        self.plan = shard_plan(cfg, world, types)

    def __contains__(self, name: str) -> bool:
        if name == "output.weight":
            return True
        if name.endswith(".bias") and name.rsplit(".", 2)[-2] in ("attn_output", "ffn_down") and self.rank != 0:
            return False                  # the bias of a row-parallel matrix is added once
        return name in self.src

    def __getitem__(self, name: str) -> QWeight:
        c, r, p = self.cfg, self.rank, self.plan
        if name == "output.weight":
            w = self.src[name] if name in self.src else self.src["token_embd.weight"]
            lo = min(r * p["vocab_rows"], c.vocab_size)
            return w.rows(lo, min(lo + p["vocab_rows"], c.vocab_size))
        w = self.src[name]
        leaf = name.rsplit(".", 2)[-2] if name.count(".") >= 2 else ""
        hd = c.head_dim
        if leaf == "attn_q":
            return w.rows(r * p["heads"] * hd, (r + 1) * p["heads"] * hd)
        if leaf in ("attn_k", "attn_v"):
            h0 = (r // p["kv_rep"]) * p["kv_heads"]
            return w.rows(h0 * hd, (h0 + p["kv_heads"]) * hd)
        if "_exps." in name:               # expert parallelism: whole experts, E / world per rank (weights [E, n, k], biases [E, n])
            return w.rows(r * p["experts"], (r + 1) * p["experts"])
        if leaf in ("ffn_gate", "ffn_up"):
            return w.rows(r * p["d_ff"], (r + 1) * p["d_ff"])
        if name.endswith(".weight") and leaf == "attn_output":
            return w.cols(r * p["heads"] * hd, (r + 1) * p["heads"] * hd)
        if name.endswith(".weight") and leaf == "ffn_down":
            return w.cols(r * p["d_ff"], (r + 1) * p["d_ff"])
        if leaf == "attn_sinks":
            return w.rows(r * p["heads"], (r + 1) * p["heads"])
        return w


class TPBackend(B200Backend):
    name = "b200-tp"
    supports_verify = False      # the verification pass of speculative decoding is not part of the follower protocol
    supports_embeds = False      # image rows are not part of the follower protocol either

    def __init__(self, cfg: ModelConfig, tensors, device: str = "cuda", rank: int = 0, world: int = 1, group=None,
                 max_chunk: int = 2048, keep_bf16: bool | None = None, kv_type: str | None = None):
        if cfg.sandwich_norm:
            raise NotImplementedError("tensor parallelism is implemented for pre-norm models")
        if cfg.d_model > 8192:
            raise NotImplementedError("tensor parallelism keeps one row of the residual stream in registers: d_model <= 8192")
        self.full_cfg, self.rank, self.world, self.group, self.max_chunk = cfg, rank, world, group, max_chunk
        self.region: PeerRegion | None = None
        sh = ShardedTensors(tensors, cfg, rank, world)
        self.plan = sh.plan
        local = dataclasses.replace(cfg, n_heads=sh.plan["heads"], n_kv_heads=sh.plan["kv_heads"], d_ff=sh.plan["d_ff"])
        self.e_lo, self.e_cnt = rank * sh.plan["experts"], sh.plan["experts"]      # expert parallelism: this rank's experts
        super().__init__(None, device=device, cfg=local, tensors=sh, keep_bf16=keep_bf16, kv_type=kv_type)
        self.v_lo = min(rank * sh.plan["vocab_rows"], cfg.vocab_size)
        if self.head.n != min(self.v_lo + sh.plan["vocab_rows"], cfg.vocab_size) - self.v_lo:
            raise RuntimeError("vocabulary shard has an unexpected number of rows")

    # -- buffers --------------------------------------------------------------------------------------
    def alloc(self, n_slots: int, n_ctx: int) -> None:
        super().alloc(n_slots, n_ctx)
        c, N, MB = self.cfg, self.world, MAX_DECODE_BATCH
        if self.region is not None:
            self.region.close()
        lay = Layout()
        self.rpr_max = (self.max_chunk + N - 1) // N
        self.b_dec = lay.add("dec_parts", 2 * N * MB * c.d_model * 8)          # (value, epoch) pairs, two halves
        self.b_logits = lay.add("logits", MB * c.vocab_size * 4)
        self.b_parts = lay.add("pre_parts", N * self.rpr_max * c.d_model * 2)       # bf16 partial rows
        self.b_h = lay.add("h_full", self.max_chunk * c.d_model * 2)
        self.region = reg = PeerRegion(lay.size, self.rank, N, self.device, self.group)
        b = self.buf
        b.logits = reg.tensor(self.b_logits, (MB, c.vocab_size), torch.float32)
        self.h_full = reg.tensor(self.b_h, (self.max_chunk, c.d_model), torch.bfloat16)
        self.xs = torch.zeros(self.rpr_max, c.d_model, device=self.device, dtype=torch.float32)
        slab = MB * c.d_model * 8
        # partial rows of a decode exchange land in slab `rank` of every rank's receive buffer (low-latency protocol)
        self.cm_dec = reg.send(CH_DEC, [reg.addr(self.b_dec, r, self.rank * slab) for r in range(N)], parity_stride=N * MB * c.d_model)
        self.cm_dec.ll = 1
        # logits: this rank's vocabulary rows are columns [v_lo, v_lo + n) of every rank's logits buffer
        self.cm_logits = reg.send(CH_LOGITS, [reg.addr(self.b_logits, r, self.v_lo * 4) for r in range(N)])
        self.cm_ag = reg.send(CH_AG, [reg.addr(self.b_h, r) for r in range(N)])
        pslab = self.rpr_max * c.d_model * 2
        self.cm_rs = reg.send(CH_RS, [reg.addr(self.b_parts, r, self.rank * pslab) for r in range(N)])

    def close(self) -> None:
        super().close()
        if self.region is not None:
            self.region.close()
            self.region = None

    def comm_status(self) -> int:
        return max(self.region.status(ch) for ch in (CH_DEC, CH_LOGITS, CH_RS, CH_AG, CH_BAR))

    def check_exchanges(self) -> None:
        """Raise if a bounded wait of an exchange ran out on this rank (a peer is late, gone or out of step).

        The kernels that waited contributed zeros and returned, so the step's result is unusable; the status words are
        cleared so that the group can be torn down or retried by the caller.
        """
        bad = self.region.failed_channels()
        if bad:
            for ch in bad:
                self.region.clear_status(ch)
            names = {CH_DEC: "decode all-reduce", CH_LOGITS: "logits gather", CH_RS: "prefill reduce-scatter", CH_AG: "prefill all-gather",
                     CH_BAR: "chunk barrier"}
            raise RuntimeError("tensor-parallel exchange timed out on rank %d: %s" % (self.rank, ", ".join(names.get(c, str(c)) for c in bad)))

    def decode_argmax(self, slots, tokens, positions):
        out = super().decode_argmax(slots, tokens, positions)
        self.check_exchanges()
        return out

    def decode(self, slots, tokens, positions):
        out = super().decode(slots, tokens, positions)
        self.check_exchanges()
        return out

    def decode_loop(self, slots, tokens, positions, n_steps, first_tokens=None):
        # after a wait has run out every later wait of that channel returns at once with zeros: without this check the rest
        # of the loop would be fast garbage
        out = super().decode_loop(slots, tokens, positions, n_steps, first_tokens)
        self.check_exchanges()
        return out

    # -- decode ---------------------------------------------------------------------------------------
    def _norm_quant_reduce(self, w, nb):
        """x += sum of the partial rows of the last exchange; then RMSNorm + int8 quantisation of x."""
        b, c, N = self.buf, self.cfg, self.world
        a = K.NormQuantArgs(K.ptr(b.x), K.ptr(w), c.norm_eps, c.d_model, 1, K.ptr(b.xq), K.ptr(b.xds), K.ptr(b.xf), None)
        a.parts = self.region.addr(self.b_dec)
        a.n_part, a.part_stride, a.parity_stride = N, MAX_DECODE_BATCH * c.d_model, N * MAX_DECODE_BATCH * c.d_model
        a.chan = self.region.chan(CH_DEC)
        K._check(K.lib().b2_rmsnorm_quant(C.byref(a), nb, int(self.pdl), K.stream()), "rmsnorm_quant(reduce)")
        self._n += 1

    def _gemv_send(self, w, nb, xq, xds, xf, cm, ldo):
        a = K.GemvArgs()
        a.seg[0] = w.desc()
        a.nseg, a.nb = 1, nb
        a.xq, a.xds, a.xf, a.out, a.ldo, a.accumulate = K.ptr(xq), K.ptr(xds), K.ptr(xf), None, ldo, 0
        a.cm = cm
        K._check(K.lib().b2_gemv(C.byref(a), int(self.pdl), K.stream()), "gemv(send)")
        self._n += 1

    def _decode_kernels(self, nb: int, want_argmax) -> None:
        c, b, lib, st = self.cfg, self.buf, K.lib(), K.stream
        self._n = 0
        K.embed(self.embd, b.tokens[:nb], c.embed_scale, out=b.x)
        self._n += 1
        act = K._ACT[c.act]
        for i, L in enumerate(self.layers):
            if i == 0:
                self._norm_quant(b.x, L.attn_norm, nb, c.d_model)
            else:
                self._norm_quant_reduce(L.attn_norm, nb)            # completes the previous layer's FFN
            self._gemv([L.wq, L.wk, L.wv], nb, b.xq, b.xds, b.xf, b.qkv, b.qkv.stride(0))
            local = L.swa and c.rope_base_local > 0
            inv_freq, mscale = (self.inv_freq_local, 1.0) if local else (self.inv_freq, self.mscale)
            fused = self.fuse_rope and L.q_norm is None and L.k_norm is None and self.k_scale[i] is None and not self.fuse_attn_combine
            aa = K.AttnDecodeArgs(None if fused else K.ptr(b.q), K.ptr(self.k_cache[i]), K.ptr(self.v_cache[i]), K.ptr(b.positions), K.ptr(b.slots),
                                  c.n_heads, c.n_kv_heads, self.n_ctx, self.n_splits, self.attn_scale, c.attn_softcap,
                                  c.sliding_window if L.swa else 0, K.ptr(b.part_acc), K.ptr(b.part_ml), K.ptr(self.k_scale[i]),
                                  K.ptr(self.v_scale[i]))
            ca = K.AttnCombineArgs(K.ptr(b.part_acc), K.ptr(b.part_ml), K.ptr(L.sinks), c.n_heads, self.n_splits, c.head_dim,
                                   K.ptr(b.ao), K.ptr(b.aq), K.ptr(b.ads))
            if fused:
                # rotary embedding of the queries, rotation + cache append of the new key / value and the attention in one launch
                rr = K.AttnRopeArgs(K.ptr(b.qkv), K.ptr(inv_freq), mscale, c.rope_dim, int(c.rope_style == "neox"))
                lib.b2_attn_decode_rope.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
                rc = lib.b2_attn_decode_rope(C.byref(aa), C.byref(rr), C.byref(ca), nb, c.head_dim, int(self.pdl), st())
                if rc == 801:           # cudaErrorNotSupported: nothing was launched; this model keeps the separate kernel
                    self.fuse_rope = fused = False
                    aa.q = K.ptr(b.q)
                else:
                    K._check(rc, "attn_decode_rope")
                    self._n += 2
            if not fused:
                ra = K.RopeKvArgs(K.ptr(b.qkv), K.ptr(b.positions), K.ptr(b.slots), K.ptr(inv_freq),
                                  K.ptr(L.q_norm), K.ptr(L.k_norm), c.norm_eps, mscale, c.n_heads, c.n_kv_heads,
                                  c.head_dim, c.rope_dim, int(c.rope_style == "neox"), self.n_ctx, K.ptr(b.q), K.ptr(self.k_cache[i]),
                                  K.ptr(self.v_cache[i]), K.ptr(self.k_scale[i]), K.ptr(self.v_scale[i]))
                K._check(lib.b2_rope_kv(C.byref(ra), nb, int(self.pdl), st()), "rope_kv")
                if self.fuse_attn_combine:      # the last CTA of every head group merges the splits: one launch instead of two
                    K._check(lib.b2_attn_decode_fused(C.byref(aa), C.byref(ca), C.c_void_p(K.ptr(b.attn_tickets)), nb, c.head_dim, int(self.pdl), st()),
                             "attn_decode_fused")
                    self._n += 2
                else:
                    K._check(lib.b2_attn_decode(C.byref(aa), C.byref(ca), nb, c.head_dim, int(self.pdl), st()), "attn_decode")
                    self._n += 3
            self._gemv_send(L.wo, nb, b.aq, b.ads, b.ao, self.cm_dec, c.d_model)
            self._norm_quant_reduce(L.ffn_norm, nb)
            if L.moe:      # expert parallel: local experts only; the weighted partial sum goes to every rank like a row-parallel GEMV
                self._moe_decode(L, nb, act, cm=self.cm_dec)
                continue
            ga = K.GluArgs()
            ga.gu = L.gu.desc()
            ga.nb, ga.xq, ga.xds, ga.xf = nb, K.ptr(b.xq), K.ptr(b.xds), K.ptr(b.xf)
            ga.act, ga.alpha, ga.limit = act, c.swiglu_alpha, c.swiglu_limit
            ga.hq, ga.hds, ga.hf = K.ptr(b.hq), K.ptr(b.hds), K.ptr(b.hf) if not L.down.quant_input else None
            K._check(lib.b2_gemv_glu_quant(C.byref(ga), int(self.pdl), st()), "gemv_glu_quant")
            self._n += 1
            self._gemv_send(L.down, nb, b.hq, b.hds, b.hf, self.cm_dec, c.d_model)
        self._norm_quant_reduce(self.out_norm, nb)
        self._gemv_send(self.head, nb, b.xq, b.xds, b.xf, self.cm_logits, c.vocab_size)
        self.region.wait(CH_LOGITS, self.pdl)
        self._n += 1
        if want_argmax:
            loop = want_argmax == "loop"      # the winner is fed back on the device: no host round trip between steps
            K.argmax(b.logits[:nb], out=b.sampled, tokens=b.tokens if loop else None, positions=b.positions if loop else None)
            self._n += 1
        self.launches_per_step = self._n

    # -- prefill --------------------------------------------------------------------------------------
    def _norm_gather(self, w, rows: int, row0: int, reduce: bool) -> None:
        c, reg = self.cfg, self.region
        a = TpNormGatherArgs()
        a.x, a.w, a.eps, a.k, a.row0 = K.ptr(self.xs), K.ptr(w), c.norm_eps, c.d_model, row0
        a.parts, a.n_part, a.part_stride = reg.addr(self.b_parts), (self.world if reduce else 0), self.rpr_max * c.d_model
        a.rs_chan = reg.chan(CH_RS)
        a.ag = self.cm_ag
        f = K.lib().b2_tp_norm_gather
        f.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        K._check(f(C.addressof(a), rows, K.stream()), "tp_norm_gather")
        reg.wait(CH_AG)
        self.kernel_launches += 2

    def _mm_scatter(self, x_bf16: torch.Tensor, w: K.DevWeight, rpr: int) -> None:
        """Row-parallel product: partial rows go to the parts buffer of the rank that owns them."""
        wb = getattr(w, "bf16", None)
        if wb is None:
            wb = K.dequant_to_bf16(w)
            self.kernel_launches += 1
        K.gemm_bf16_scatter(x_bf16, wb, self.cfg.d_model, self.cm_rs, rpr, w.bias)
        self.kernel_launches += 1

    @torch.no_grad()
    def _forward_chunk(self, slot: int, tokens: Sequence[int], pos0: int) -> torch.Tensor:
        """Chunked prefill; returns the final hidden states after the output norm, [T, d_model] bf16, on every rank."""
        c, dev, N = self.cfg, self.device, self.world
        T = len(tokens)
        if T > self.max_chunk:
            raise ValueError(f"prefill chunk of {T} tokens exceeds {self.max_chunk}")
        rpr = (T + N - 1) // N
        row0 = min(self.rank * rpr, T)
        rows = min(rpr, T - row0)
        ids = torch.tensor(list(tokens), device=dev, dtype=torch.int32)
        pos = torch.arange(pos0, pos0 + T, device=dev, dtype=torch.int32)
        slots = torch.full((T,), slot, device=dev, dtype=torch.int32)
        self.region.barrier(CH_BAR)          # the previous chunk's readers of h_full / parts are done on every rank
        if rows > 0:
            K.embed(self.embd, ids[row0:row0 + rows], c.embed_scale, out=self.xs)
        p_end = pos0 + T
        h = self.h_full[:T]
        for i, L in enumerate(self.layers):
            self._norm_gather(L.attn_norm, rows, row0, reduce=i > 0)
            qkv = torch.empty(T, (c.n_heads + 2 * c.n_kv_heads) * c.head_dim, device=dev, dtype=torch.float32)
            if L.wqkv16 is not None:
                K.gemm_bf16(h, L.wqkv16, L.bqkv, out=qkv)
                self.kernel_launches += 1
            else:
                self._mm(h, L.wq, qkv, 0)
                self._mm(h, L.wk, qkv, c.q_dim)
                self._mm(h, L.wv, qkv, c.q_dim + c.kv_dim)
            local = L.swa and c.rope_base_local > 0
            q = K.rope_kv(qkv, pos, slots, self.inv_freq_local if local else self.inv_freq, n_heads=c.n_heads, n_kv_heads=c.n_kv_heads,
                          hd=c.head_dim, n_rot=c.rope_dim, neox=c.rope_style == "neox", mscale=1.0 if local else self.mscale,
                          k_cache=self.k_cache[i], v_cache=self.v_cache[i], q_norm=L.q_norm, k_norm=L.k_norm, eps=c.norm_eps,
                          k_scale=self.k_scale[i], v_scale=self.v_scale[i])
            self._mm_scatter(self._attn_prefill(q, i, L, slot, pos0, p_end), L.wo, rpr)
            self._norm_gather(L.ffn_norm, rows, row0, reduce=True)
            if L.moe:
                # every rank holds all rows of h (the all-gather was the dispatch); its experts' partial output rows go to their owners
                part = self._moe_prefill(h, L).contiguous()
                f_sc = K.lib().b2_tp_scatter_rows
                f_sc.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
                K._check(f_sc(K.ptr(part), T, c.d_model, rpr, C.addressof(self.cm_rs), K.stream()), "tp_scatter_rows")
                self.kernel_launches += 1
                continue
            self._mm_scatter(self._mm_glu(h, L.gu), L.down, rpr)
        self._norm_gather(self.out_norm, rows, row0, reduce=True)
        return h

    @torch.no_grad()
    def prefill(self, slot: int, tokens: Sequence[int], pos0: int, need_logits: bool = True):
        h = self._forward_chunk(slot, tokens, pos0)
        if not need_logits:
            return None
        # vocabulary rows are split over the ranks: every rank multiplies the last row with its shard and
        # writes the result into every rank's logits buffer (the decode-side gather)
        b, c = self.buf, self.cfg
        x = h[len(tokens) - 1:len(tokens)].float()
        a = K.NormQuantArgs(K.ptr(x), None, c.norm_eps, c.d_model, 0, K.ptr(b.xq), K.ptr(b.xds), K.ptr(b.xf), None)
        K._check(K.lib().b2_rmsnorm_quant(C.byref(a), 1, 0, K.stream()), "quant")
        self._n = 0
        self._gemv_send(self.head, 1, b.xq, b.xds, b.xf, self.cm_logits, c.vocab_size)
        self.region.wait(CH_LOGITS)
        self.kernel_launches += 3
        out = R.softcap(b.logits[0].clone(), c.final_softcap)
        self.check_exchanges()
        return out

    @torch.no_grad()
    def hidden(self, slot: int, tokens: Sequence[int]) -> torch.Tensor:
        return self._forward_chunk(slot, tokens, 0).float()
