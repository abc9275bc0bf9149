"""The sm_100a execution engine.

One process drives one GPU.  Weights stay in their GGUF quantisation, re-laid out into aligned planes
(``ops/cuda.py``); the KV cache is f16, partitioned by slot: ``[slot][kv_head][position][dim]`` per
layer.  A decode step for up to eight sequences is a fixed sequence of hand-written kernels

    embed -> L x [ rmsnorm+quant -> QKV GEMV -> qk-norm+RoPE+cache append -> split-K attention
                   -> O GEMV (+residual) -> rmsnorm+quant -> gate/up GEMV + GLU + quant
                   -> down GEMV (+residual) ] -> rmsnorm+quant -> LM-head GEMV -> arg-max

captured once per batch size into a CUDA graph (kernels are launched with programmatic dependent
launch so that the launch latency of kernel i+1 hides behind kernel i) and replayed with device-side
token / position / slot arrays.  Prefill runs chunked through the tensor-core GEMM path.

In the reference this layer is the external engine process (its runner interface:
llm/server.go:59-78); its kernels are ggml-cuda's mmvq / mmq / fattn / norm / rope families.
"""
from __future__ import annotations

import ctypes as C
import math
import os
from typing import Sequence

import torch

from .. import envconfig
from ..gguf.reader import GGUFFile
from ..models.config import ModelConfig, config_from_gguf
from ..models.weights import QWeight, load_tensor
from ..ops import cuda as K
from ..ops import reference as R
from ..ops import sk as SK

MAX_DECODE_BATCH = 8             # sequences per launch of the dp4a kernels (kernels/gemv.cu)
MAX_STREAM_BATCH = 32            # sequences per step when every matrix runs on the streaming kernel (kernels/gemv_sk.cu)


def supports(cfg: ModelConfig) -> bool:
    if cfg.is_moe and (cfg.n_experts > 512 or cfg.n_experts_used > 16 or cfg.d_ff_expert % 32):
        return False
    return cfg.arch in ("llama", "mistral", "qwen2", "qwen3", "qwen3moe", "gpt-oss", "gemma", "gemma2", "gemma3", "phi3") \
        and cfg.head_dim in (32, 64, 128, 256) and cfg.head_dim == cfg.v_head_dim and cfg.d_model % 32 == 0 \
        and (cfg.d_ff % 32 == 0 or cfg.is_moe)       # expert models have no dense FFN: its width (per rank, under a split) plays no part


class _Layer:
    pass


class B200Backend:
    name = "b200"
    supports_verify = True

    def __init__(self, g: GGUFFile | None, device: str = "cuda", opts=None, cfg: ModelConfig | None = None,
                 tensors: dict[str, QWeight] | None = None, keep_bf16: bool | None = None, prefill_gemm: str = "bf16",
                 kv_type: str | None = None, layers: tuple[int, int] | None = None):
        """Load from an opened GGUF, or from ``cfg`` + an iterable source of :class:`QWeight` (synthetic checkpoints).

        ``keep_bf16``: keep a resident 16-bit copy of every matrix for prefill (None: when it fits in 40% of the free HBM;
        otherwise each matrix is expanded into scratch right before its GEMM).  ``prefill_gemm``: "bf16" (expand, then the
        bf16 tensor-core GEMM) or "fused" (weights expanded inside the GEMM kernel; no 16-bit copy anywhere).
        ``kv_type``: "f16" or "q8_0" (int8 values with one f16 scale per 32 dims, written by the rope kernel and expanded
        inside the attention kernels; "q4_0" is served as q8_0); default: ``opts.kv_cache_type``
        (envconfig/config.go:183 OLLAMA_KV_CACHE_TYPE).  ``layers`` = (lo, hi): this object is one stage of a layer
        pipeline and holds blocks lo..hi-1 only; the first stage also holds the embedding, the last one the output
        norm and head, and the residual stream enters / leaves through ``buf.x`` (decode) or the ``x`` argument (prefill).
        """
        self.device = torch.device(device if device != "cuda" else f"cuda:{torch.cuda.current_device()}")
        self.cfg = cfg if cfg is not None else config_from_gguf(g)
        if not supports(self.cfg):
            raise NotImplementedError(f"{self.cfg.arch} is not supported by the sm_100a engine")
        K.lib()
        self.prefill_gemm = prefill_gemm
        self.l_lo, self.l_hi = layers if layers is not None else (0, self.cfg.n_layers)
        if not 0 <= self.l_lo < self.l_hi <= self.cfg.n_layers:
            raise ValueError(f"layer range {layers} outside 0..{self.cfg.n_layers}")
        self.first, self.last = self.l_lo == 0, self.l_hi == self.cfg.n_layers
        kv_type = (kv_type or getattr(opts, "kv_cache_type", None) or "f16").lower()
        if kv_type not in ("f16", "q8_0", "q4_0"):
            raise ValueError(f"unknown K/V cache type {kv_type!r}")
        # quantised blocks cover 32 dims; head sizes outside the flash-attention kernel read the cache through torch
        self.kv_q8 = kv_type != "f16" and self.cfg.head_dim % 32 == 0 and self.cfg.head_dim in K.ATTN_PREFILL_HEAD_DIMS
        self.kv_type = "q8_0" if self.kv_q8 else "f16"
        if kv_type != self.kv_type:       # say so: the cache costs what the stored encoding costs, not what was asked for
            import logging
            logging.getLogger("ollama_b200.engine").warning("K/V cache type %s is stored as %s (%s)", kv_type, self.kv_type,
                                                            "there is no 4-bit cache encoding" if self.kv_q8 else "this head size has no quantised cache")
        if keep_bf16 is None:
            c = self.cfg
            est = 2 * (c.n_layers * (c.d_model * (2 * c.q_dim + 2 * c.kv_dim) + 3 * c.d_model * c.d_ff) + c.vocab_size * c.d_model)
            keep_bf16 = prefill_gemm == "bf16" and est < 0.4 * torch.cuda.mem_get_info(self.device)[0]
        self.keep_bf16 = keep_bf16
        if not hasattr(self, "e_lo"):       # experts resident on this GPU (a tensor-parallel subclass narrows the range)
            self.e_lo, self.e_cnt = 0, self.cfg.n_experts
        self.n_slots = self.n_ctx = 0
        self._graphs: dict[tuple[int, bool], torch.cuda.CUDAGraph] = {}
        self._capture_stream = None
        self.pdl = True
        # Decode matrices in unit order for the streaming GEMV (Q4_K / Q6_K layers without experts or sandwich norms); B200_SK=0
        # keeps every layer on the dp4a kernels.
        # Subclasses that enqueue their own decode kernels (tensor parallelism) keep the dp4a planes.
        if os.environ.get("B200_ATTN_DECODE_STAGES", "") in ("2", "3", "4"):      # pipeline depth of the tensor-core decode attention (default: per launch)
            K.attn_decode_stages(int(os.environ["B200_ATTN_DECODE_STAGES"]))
        # decode steps of at least this many sequences run their 16-bit matrices (bf16 weights, or resident bf16 copies of matrices
        # that have no streaming-GEMV form) on the tcgen05 GEMM instead of the plane GEMV; 0 = never
        # (tensor-parallel ranks keep the GEMV unless the variable asks otherwise)
        env = os.environ.get("B200_TC_DECODE_MIN", "")
        self.tc_decode_min = int(env) if env else (4 if type(self) is B200Backend else 0)
        self.moe_stream_q = os.environ.get("B200_MOE_STREAM_Q", "1") != "0"    # MoE prefill reads MXFP4 experts as they are (no 16-bit expansion per chunk)
        self.fuse_rope = os.environ.get("B200_FUSE_ROPE", "1") != "0"      # decode attention rotates Q / K and appends K / V itself
        self.use_sk = os.environ.get("B200_SK", "1") != "0" and not self.cfg.sandwich_norm and type(self) is B200Backend
        self.max_batch = MAX_DECODE_BATCH
        self.fuse_attn_combine = False    # one launch (last CTA merges the splits) measured slower than two launches joined by PDL
        self.use_graphs = True
        self.launches_per_step = 0
        self.launches_by_key: dict = {}
        self._warm: set = set()
        self.kernel_launches = 0          # kernels of this library executed so far (graph nodes count individually)
        self.h2d_bytes = self.d2h_bytes = 0
        self._load(g, tensors)

    # -- loading ------------------------------------------------------------------------------------
    def _load(self, g: GGUFFile | None, tensors) -> None:
        c, dev = self.cfg, self.device

        def has(name):
            return (name in tensors) if tensors is not None else g.has(name)

        def get(name) -> QWeight:
            return tensors[name] if tensors is not None else load_tensor(g, name)

        def vec(name) -> torch.Tensor | None:
            if not has(name):
                return None
            return get(name).dequant().to(dev).contiguous()

        def mat(name, keep=True) -> K.DevWeight:
            w = K.repack(get(name + ".weight"), dev, bias=vec(name + ".bias"))
            if self.keep_bf16 and keep:
                w.bf16 = K.dequant_to_bf16(w)
            return w

        tied = not has("output.weight")
        self.embd = K.repack(get("token_embd.weight"), dev) if self.first or (self.last and tied) else None
        self.out_norm = self.head = None
        if self.last:
            self.out_norm = vec("output_norm.weight")
            self.head = mat("output") if not tied else self.embd
            if self.keep_bf16 and not hasattr(self.head, "bf16"):
                self.head.bf16 = K.dequant_to_bf16(self.head)
        self.layers: list[_Layer] = []
        for i in range(self.l_lo, self.l_hi):
            p, L = f"blk.{i}.", _Layer()
            L.attn_norm = vec(p + "attn_norm.weight")
            L.wq, L.wk, L.wv, L.wo = mat(p + "attn_q"), mat(p + "attn_k"), mat(p + "attn_v"), mat(p + "attn_output")
            L.wqkv16 = L.bqkv = None
            if self.keep_bf16:          # prefill multiplies Q, K and V in one GEMM
                L.wqkv16 = torch.cat([L.wq.bf16, L.wk.bf16, L.wv.bf16])
                del L.wq.bf16, L.wk.bf16, L.wv.bf16
                if any(w.bias is not None for w in (L.wq, L.wk, L.wv)):
                    L.bqkv = torch.cat([w.bias if w.bias is not None else torch.zeros(w.n, device=dev) for w in (L.wq, L.wk, L.wv)])
            L.q_norm, L.k_norm = vec(p + "attn_q_norm.weight"), vec(p + "attn_k_norm.weight")
            L.post_attn_norm = vec(p + "post_attention_norm.weight") if c.sandwich_norm else None
            L.ffn_norm = vec(p + "ffn_norm.weight")
            if L.ffn_norm is None:
                L.ffn_norm = vec(p + "post_attention_norm.weight")
            L.post_ffw_norm = vec(p + "post_ffw_norm.weight") if c.sandwich_norm else None
            L.moe = c.is_moe and has(p + "ffn_gate_inp.weight")
            if L.moe:
                # experts stay stacked: [E][n][k] planes, the expert index selects a row range inside the kernels
                L.router = mat(p + "ffn_gate_inp", False)
                L.router_f32 = get(p + "ffn_gate_inp.weight").dequant().to(dev).contiguous()

                def exps(kind):
                    b = vec(p + f"ffn_{kind}_exps.bias")
                    return K.repack(get(p + f"ffn_{kind}_exps.weight"), dev, bias=b.reshape(-1) if b is not None else None)

                L.gate, L.up, L.down = exps("gate"), exps("up"), exps("down")
            else:
                L.gate, L.up, L.down = mat(p + "ffn_gate", False), mat(p + "ffn_up", False), mat(p + "ffn_down")
            if L.gate.wtype != L.up.wtype:
                L.gu = K.interleave_rows(K.to_f16(L.gate), K.to_f16(L.up))
            else:
                L.gu = K.interleave_rows(L.gate, L.up)
            L.gate.planes, L.up.planes = [], []      # the interleaved matrix serves decode and prefill
            if self.keep_bf16 and not L.moe:
                L.gu.bf16 = K.dequant_to_bf16(L.gu)
            L.sinks = vec(p + "attn_sinks.weight")
            L.swa = c.layer_is_swa(i)
            L.sk = self._load_sk_layer(p, L, get, vec) if self.use_sk and not L.moe else None
            self.layers.append(L)
        # Expert matrices as 16-bit copies for the grouped prefill GEMM when they fit into a third of the free memory (EP shards
        # of the large models do: 30 to 60 GB per GPU); otherwise every chunk expands the layer's experts into scratch.
        moe_layers = [L for L in self.layers if L.moe]
        if moe_layers and self.keep_bf16 is not False:
            need = sum(2 * (L.gu.total_rows * L.gu.k + L.down.total_rows * L.down.k) for L in moe_layers)
            if need < 0.33 * torch.cuda.mem_get_info(dev)[0]:
                for L in moe_layers:
                    L.gu.bf16, L.down.bf16 = K.dequant_to_bf16(L.gu), K.dequant_to_bf16(L.down)
        self.sk_head = None
        if self.use_sk and self.last and all(L.sk is not None for L in self.layers):
            hw = get("output.weight" if not tied else "token_embd.weight")
            if SK.supported(hw.dtype, *hw.shape) and self.head.bias is None:
                self.sk_head = SK.repack(hw, dev)
        # a step takes up to 32 sequences only when no layer falls back to the dp4a kernels (eight per launch)
        if all(L.sk is not None for L in self.layers) and (self.sk_head is not None or not self.last) and type(self) is B200Backend:
            self.max_batch = MAX_STREAM_BATCH
        # ... and up to 32 when every layer is a mixture of experts (its kernels run one grid row per token-expert pair) whose dense
        # matrices are 16-bit and multiply on the tensor-core GEMM; the router's GEMV then runs eight rows per launch
        if (type(self) is B200Backend and 0 < self.tc_decode_min <= MAX_DECODE_BATCH and self.layers and all(L.moe for L in self.layers)
                and all(self._bf16_of(w) is not None for L in self.layers for w in ((L.wo,) if L.wqkv16 is not None else (L.wq, L.wk, L.wv, L.wo)))
                and all(w.wtype in (K.WT_BF16, K.WT_F16) for L in self.layers for w in (L.wq, L.wk, L.wv))
                and (not self.last or self._bf16_of(self.head) is not None)):
            self.max_batch = MAX_STREAM_BATCH
        ff = vec("rope_freqs.weight")
        kw = dict(scaling=c.rope_scaling_type if c.rope_scaling_type != "llama3" else "none", factor=c.rope_scaling_factor,
                  orig_ctx=c.rope_orig_ctx, beta_fast=c.yarn_beta_fast, beta_slow=c.yarn_beta_slow, device=dev)
        self.inv_freq, self.mscale = R.rope_inv_freq(c.rope_dim, c.rope_base, freq_factors=ff, **kw)
        if c.rope_attn_factor > 0:
            self.mscale = c.rope_attn_factor
        self.inv_freq = self.inv_freq.contiguous()
        self.inv_freq_local = self.inv_freq
        if c.rope_base_local > 0:
            self.inv_freq_local = R.rope_inv_freq(c.rope_dim, c.rope_base_local, device=dev)[0].contiguous()
        self.attn_scale = c.scale
        if c.arch in ("gemma2", "gemma3") and c.n_layers in (46, 62):
            self.attn_scale = 1.0 / math.sqrt(c.d_model / c.n_heads)
        torch.cuda.synchronize(dev)

    def _load_sk_layer(self, p: str, L, get, vec):
        """Unit-ordered copies of a layer's seven matrices for the streaming decode GEMV, or None when one of them has no unit
        layout (other encodings, odd shapes).  With a resident 16-bit copy for prefill the dp4a planes are dropped."""
        names = ("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down")
        qs = {n: get(p + n + ".weight") for n in names}
        if any(len(q.shape) != 2 or not SK.supported(q.dtype, *q.shape) for q in qs.values()) or qs["ffn_gate"].dtype != qs["ffn_up"].dtype:
            return None
        dev, o = self.device, _Layer()
        o.qkv = [SK.repack(qs[n], dev, bias=vec(p + n + ".bias")) for n in ("attn_q", "attn_k", "attn_v")]
        o.o = SK.repack(qs["attn_output"], dev, bias=vec(p + "attn_output.bias"))
        bg, bu = vec(p + "ffn_gate.bias"), vec(p + "ffn_up.bias")
        gub = None
        if bg is not None or bu is not None:
            z = torch.zeros(qs["ffn_gate"].shape[0], device=dev)
            gub = torch.stack([bg if bg is not None else z, bu if bu is not None else z], 1).reshape(-1)
        o.gu = SK.repack(SK.interleave(qs["ffn_gate"], qs["ffn_up"]), dev, bias=gub)
        o.down = SK.repack(qs["ffn_down"], dev, bias=vec(p + "ffn_down.bias"))
        if self.keep_bf16:
            for w in (L.wq, L.wk, L.wv, L.wo, L.gu, L.down):
                w.planes = []
        return o

    def weight_bytes(self) -> int:
        ws = [w for w in (self.embd, self.head if self.head is not self.embd else None) if w is not None]
        for L in self.layers:
            ws += [L.wq, L.wk, L.wv, L.wo, L.gu, L.down]
            if L.sk is not None:
                ws += L.sk.qkv + [L.sk.o, L.sk.gu, L.sk.down]
        if self.sk_head is not None:
            ws.append(self.sk_head)
        return sum(w.nbytes for w in ws)

    def kv_bytes(self) -> int:
        n = sum(t.numel() * t.element_size() for t in getattr(self, "k_cache", [])) * 2
        return n + sum(t.numel() * 2 for t in getattr(self, "k_scale", []) if t is not None) * 2

    # -- buffers --------------------------------------------------------------------------------------
    def alloc(self, n_slots: int, n_ctx: int) -> None:
        c, dev = self.cfg, self.device
        self.n_slots, self.n_ctx = n_slots, n_ctx
        kv_dt = torch.int8 if self.kv_q8 else torch.float16
        self.k_cache = [torch.zeros(n_slots, c.n_kv_heads, n_ctx, c.head_dim, device=dev, dtype=kv_dt) for _ in self.layers]
        self.v_cache = [torch.zeros(n_slots, c.n_kv_heads, n_ctx, c.head_dim, device=dev, dtype=kv_dt) for _ in self.layers]
        self.k_scale = self.v_scale = [None] * len(self.layers)
        if self.kv_q8:
            def sc():
                return [torch.zeros(n_slots, c.n_kv_heads, n_ctx, c.head_dim // 32, device=dev, dtype=torch.float16) for _ in self.layers]
            self.k_scale, self.v_scale = sc(), sc()
        MB = self.max_batch
        f32, i8, i32 = torch.float32, torch.int8, torch.int32
        qkv_dim = (c.n_heads + 2 * c.n_kv_heads) * c.head_dim
        kmax = max(c.d_model, c.q_dim)
        # split-K width of decode attention: one CTA per (sequence, KV head, split).  Measured on Llama-8B (num_ctx 8192,
        # tensor-core kernel): 16 splits give 442 tok/s at 640 tokens of context and 382 at 6272; 32 splits 428 and 396;
        # 64 splits 409 and 371
        self.n_splits = max(1, min(envconfig.attn_splits(), n_ctx // envconfig.attn_split_len()))
        b = self.buf = _Layer()
        b.x = torch.zeros(MB, c.d_model, device=dev, dtype=f32)
        b.tmp = torch.zeros(MB, c.d_model, device=dev, dtype=f32)
        b.xq = torch.zeros(MB, kmax, device=dev, dtype=i8)
        b.xds = torch.zeros(MB, kmax // 32, 2, device=dev, dtype=f32)
        b.xf = torch.zeros(MB, kmax, device=dev, dtype=f32)
        b.qkv = torch.zeros(MB, qkv_dim, device=dev, dtype=f32)
        b.q = torch.zeros(MB, c.n_heads, c.head_dim, device=dev, dtype=f32)
        b.ao = torch.zeros(MB, c.q_dim, device=dev, dtype=f32)
        b.aq = torch.zeros(MB, c.q_dim, device=dev, dtype=i8)
        b.ads = torch.zeros(MB, c.q_dim // 32, 2, device=dev, dtype=f32)
        ff = max(c.d_ff_expert, c.d_ff) if c.is_moe else c.d_ff
        hr = MB * max(c.n_experts_used, 1) if c.is_moe else MB          # MoE: one row per (token, expert-slot) pair
        b.hq = torch.zeros(hr, ff, device=dev, dtype=i8)
        b.hds = torch.zeros(hr, ff // 32, 2, device=dev, dtype=f32)
        b.hf = torch.zeros(hr, ff, device=dev, dtype=f32)
        if c.is_moe:
            b.rlogits = torch.zeros(MB, c.n_experts, device=dev, dtype=f32)
            b.moe_ids = torch.zeros(hr, device=dev, dtype=i32)
            b.moe_lids = torch.zeros(hr, device=dev, dtype=i32)
            b.moe_w = torch.zeros(hr, device=dev, dtype=f32)
            b.ey = torch.zeros(hr, c.d_model, device=dev, dtype=f32)
        b.logits = torch.zeros(MB, c.vocab_size, device=dev, dtype=f32)
        b.part_acc = torch.zeros(MB * c.n_heads * self.n_splits * c.head_dim, device=dev, dtype=f32)
        b.part_ml = torch.zeros(MB * c.n_heads * self.n_splits * 2, device=dev, dtype=f32)
        b.attn_tickets = torch.zeros(MB * c.n_heads, device=dev, dtype=i32)
        b.meta = torch.zeros(3, MB, device=dev, dtype=i32)          # tokens | positions | slots of the decode batch
        b.tokens, b.positions, b.slots = b.meta[0], b.meta[1], b.meta[2]
        b.sampled = torch.zeros(MB, device=dev, dtype=i32)
        if any(L.sk is not None for L in self.layers):      # pre-quantised inputs of the streaming GEMV (rows too wide to quantise in place)
            kq = max(kmax, ff)
            b.sk_x = (torch.zeros(MB * kq, device=dev, dtype=i8), torch.zeros(MB * (kq // 256 + 1), device=dev, dtype=f32),
                      torch.zeros(MB * (kq // 32 + 1), device=dev, dtype=torch.int16))
        b.host_in = torch.zeros(3, MB, dtype=i32).pin_memory()
        b.host_out = torch.zeros(MB, dtype=i32).pin_memory()
        b.host_np, b.host_out_np = b.host_in.numpy(), b.host_out.numpy()
        self._graphs.clear()
        self._warm.clear()

    def close(self) -> None:
        self._graphs.clear()
        self.k_cache = self.v_cache = self.k_scale = self.v_scale = []
        self.buf = None

    # -- decode ---------------------------------------------------------------------------------------
    def _norm_quant(self, x, w, nb, k, *, do_norm=True, residual=None, src=None):
        b = self.buf
        a = K.NormQuantArgs(K.ptr(x if src is None else src), K.ptr(w), self.cfg.norm_eps, k, int(do_norm), K.ptr(b.xq), K.ptr(b.xds),
                            K.ptr(b.xf), K.ptr(residual))
        K._check(K.lib().b2_rmsnorm_quant(C.byref(a), nb, int(self.pdl), K.stream()), "rmsnorm_quant")
        self._n += 1

    @staticmethod
    def _bf16_of(w):
        """The 16-bit form of a matrix when one is resident: its bf16 copy, or the planes of a bf16 matrix."""
        if w.experts or w.wtype not in (K.WT_BF16, K.WT_F16):      # quantised matrices stream fewer bytes through the GEMV
            return None
        b16 = getattr(w, "bf16", None)
        if b16 is None and w.wtype == K.WT_BF16 and w.planes:
            b16 = w.planes[0]
        return b16 if b16 is not None and w.k % 8 == 0 and w.n % 4 == 0 else None

    def _gemm_step(self, ws, b16s, nb, xf, out, accumulate=False, bias=None) -> None:
        """A projection of a decode step on the tcgen05 GEMM: fp32 activation rows -> bf16, one product per matrix (the rows
        beyond ``nb`` of the 128-row tile are the tensor map's zero fill).  Steps of several sequences on 16-bit matrices:
        a dp4a / FMA GEMV over a 16-bit matrix costs one multiply-add per weight and token, the tensor core does not care."""
        k = b16s[0].shape[1]
        a16 = xf.view(-1)[:nb * k].view(nb, k).to(torch.bfloat16)      # activation rows are packed at the matrix's row length
        off = 0
        for w, b16 in zip(ws, b16s):
            K.gemm_bf16(a16, b16, w.bias if bias is None else bias, out=out[:nb, off:off + b16.shape[0]], accumulate=accumulate)
            off += b16.shape[0]
        self._n += 1 + len(ws)

    def _gemv(self, ws, nb, xq, xds, xf, out, ldo, accumulate=False, tc=True):
        if tc and self.tc_decode_min and nb >= self.tc_decode_min and xf is not None and out.dim() == 2:
            b16s = [self._bf16_of(w) for w in ws]
            if all(b is not None for b in b16s):
                self._gemm_step(ws, b16s, nb, xf, out, accumulate)
                return
        a = K.GemvArgs()
        off = 0
        for i, w in enumerate(ws):
            a.seg[i] = w.desc(out_off=off)
            off += w.n
        k = ws[0].k
        for r0 in range(0, nb, MAX_DECODE_BATCH):      # the kernel takes eight rows; rows are packed at the matrix's row length
            a.nseg, a.nb = len(ws), min(MAX_DECODE_BATCH, nb - r0)
            a.xq, a.xds = K.ptr(xq) + r0 * k, K.ptr(xds) + r0 * (k // 32) * 8
            a.xf = K.ptr(xf) + r0 * k * 4 if xf is not None else None
            a.out, a.ldo, a.accumulate = K.ptr(out) + r0 * ldo * 4, ldo, int(accumulate)
            K._check(K.lib().b2_gemv(C.byref(a), int(self.pdl), K.stream()), "gemv")
            self._n += 1

    def _route(self, logits: torch.Tensor, tokens: int, ids, lids, wts, pdl: bool) -> None:
        c = self.cfg
        a = K.MoeRouteArgs(K.ptr(logits), logits.stride(0), c.n_experts, c.n_experts_used, 0 if c.moe_router == "softmax_topk" else 1,
                           int(c.moe_norm_topk), self.e_lo, self.e_cnt, K.ptr(ids), K.ptr(lids), K.ptr(wts))
        K._check(K.lib().b2_moe_route(C.byref(a), tokens, int(pdl), K.stream()), "moe_route")

    def _moe_decode(self, L, nb: int, act: int, cm=None) -> None:
        """Router -> top-k -> expert gate/up + GLU -> expert down -> weighted sum into the residual stream.

        Every (token, expert-slot) pair is one grid row of the indirect GEMV kernels; experts that live on another
        GPU produce zero rows.  With ``cm`` the weighted sum is sent to the tensor-parallel group instead of being added.
        """
        c, b, lib, st = self.cfg, self.buf, K.lib(), K.stream
        k = c.n_experts_used
        pairs = nb * k
        # the router stays on fp32 activations: its matrix is small and the choice of experts is sensitive to rounding
        self._gemv([L.router], nb, b.xq, b.xds, b.xf, b.rlogits, b.rlogits.stride(0), tc=False)
        self._route(b.rlogits, nb, b.moe_ids, b.moe_lids, b.moe_w, self.pdl)
        ga = K.GluArgs()
        ga.gu = L.gu.desc()
        ga.nb, ga.xq, ga.xds, ga.xf = 1, K.ptr(b.xq), K.ptr(b.xds), K.ptr(b.xf)
        ga.act, ga.alpha, ga.limit = act, c.swiglu_alpha, c.swiglu_limit
        ga.hq, ga.hds, ga.hf = K.ptr(b.hq), K.ptr(b.hds), K.ptr(b.hf) if not L.down.quant_input else None
        ga.ids, ga.x_div, ga.n_pairs = K.ptr(b.moe_lids), k, pairs
        K._check(lib.b2_gemv_glu_quant(C.byref(ga), int(self.pdl), st()), "gemv_glu_quant(moe)")
        a = K.GemvArgs()
        a.seg[0] = L.down.desc()
        a.nseg, a.nb = 1, 1
        a.xq, a.xds, a.xf, a.out, a.ldo, a.accumulate = K.ptr(b.hq), K.ptr(b.hds), K.ptr(b.hf), K.ptr(b.ey), c.d_model, 0
        a.ids, a.x_div, a.n_pairs = K.ptr(b.moe_lids), 1, pairs
        K._check(lib.b2_gemv(C.byref(a), int(self.pdl), st()), "gemv(moe down)")
        ca = K.MoeCombineArgs(K.ptr(b.ey), K.ptr(b.moe_w), k, c.d_model, K.ptr(b.x))
        if cm is not None:
            ca.cm = cm
        K._check(lib.b2_moe_combine(C.byref(ca), nb, int(self.pdl), st()), "moe_combine")
        self._n += 4

    def _moe_prefill(self, h: torch.Tensor, L) -> torch.Tensor:
        """Expert FFN of a prefill chunk without leaving the device: the (token, expert-slot) pairs are sorted by expert into
        128-row tiles, one grouped tensor-core GEMM runs gate/up with the gated activation in its epilogue, a second one the
        down projection, and the weighted rows are added back per token.

        ``h``: [T, d_model] bf16.  Returns this GPU's (partial, under expert parallelism) FFN output [T, d_model] fp32.
        """
        c = self.cfg
        T, k = h.shape[0], c.n_experts_used
        logits = h.float() @ L.router_f32.t()                       # [T, E]: tiny; kept in fp32 so that near-ties select as the fp32 graph does
        if L.router.bias is not None:
            logits = logits + L.router.bias
        ids = torch.empty(T * k, device=self.device, dtype=torch.int32)
        lids, wts = torch.empty_like(ids), torch.empty(T * k, device=self.device, dtype=torch.float32)
        self._route(logits.contiguous(), T, ids, lids, wts, False)
        row, tile_expert, rows = K.moe_plan(lids, self.e_cnt)
        xs = K.moe_gather(h, row, k, rows)
        if self.moe_stream_q and getattr(L.gu, "bf16", None) is None and K.gemm_q_grouped_supported(L.gu) and K.gemm_q_grouped_supported(L.down):
            # experts without a resident 16-bit copy: the grouped kernel streams their 4-bit blocks and expands them itself
            f = K.gemm_q_grouped(xs, L.gu, tile_expert, glu=c.act, alpha=c.swiglu_alpha, limit=c.swiglu_limit)
            ys = K.gemm_q_grouped(f, L.down, tile_expert) if f is not None else None
            if ys is not None:
                self.kernel_launches += 6
                return K.moe_scatter_combine(ys, row, wts, T, k)
        gu16 = getattr(L.gu, "bf16", None)
        if gu16 is None:
            gu16 = K.dequant_to_bf16(L.gu)                        # all resident experts at once: scratch until the call returns
            self.kernel_launches += 1
        f = K.gemm_bf16_grouped(xs, gu16, self.e_cnt, tile_expert, L.gu.bias, glu=c.act, alpha=c.swiglu_alpha, limit=c.swiglu_limit)
        del gu16
        dn16 = getattr(L.down, "bf16", None)
        if dn16 is None:
            dn16 = K.dequant_to_bf16(L.down)
            self.kernel_launches += 1
        ys = K.gemm_bf16_grouped(f, dn16, self.e_cnt, tile_expert, L.down.bias)
        del dn16
        self.kernel_launches += 6
        return K.moe_scatter_combine(ys, row, wts, T, k)

    def _sk(self, ws, x: torch.Tensor, out: torch.Tensor, nb: int, norm_w=None, mode: int = SK.MODE_STORE) -> None:
        """One streaming GEMV of the decode step: fp32 rows in (normalised with ``norm_w``), ``out`` stored / added to / gated."""
        c, b = self.cfg, self.buf
        k = ws[0].k
        xin = x[:nb, :k]
        if not SK.fits_fused_input(nb, k):      # wide or many rows: one CTA per row quantises, the GEMV reads int8 from global memory
            xq, xd, xbs = b.sk_x          # flat buffers, used as dense [nb, k] rows
            xin = SK.quant256(xin, norm_w, c.norm_eps, pdl=self.pdl,
                              out=(xq[:nb * k].view(nb, k), xd[:nb * (k // 256)].view(nb, k // 256), xbs[:nb * (k // 32)].view(nb, k // 32)))
            norm_w = None
            self._n += 1
        SK.gemv(ws, xin, norm_w=norm_w, eps=c.norm_eps, out=out, mode=mode, act=c.act, alpha=c.swiglu_alpha, limit=c.swiglu_limit, pdl=self.pdl)
        self._n += 1

    def _decode_layer_sk(self, i: int, L, nb: int) -> None:
        """A layer on the streaming GEMV: both RMSNorms, both residual adds, the gated activation and every activation
        quantisation happen inside the four matrix kernels; attention keeps its own kernels."""
        c, b, lib, st = self.cfg, self.buf, K.lib(), K.stream
        self._sk(L.sk.qkv, b.x, b.qkv, nb, norm_w=L.attn_norm)
        local = L.swa and c.rope_base_local > 0
        inv_freq, mscale = (self.inv_freq_local, 1.0) if local else (self.inv_freq, self.mscale)
        ca = K.AttnCombineArgs(K.ptr(b.part_acc), K.ptr(b.part_ml), K.ptr(L.sinks), c.n_heads, self.n_splits, c.head_dim,
                               K.ptr(b.ao), None, None)
        fused = self.fuse_rope and L.q_norm is None and L.k_norm is None and self.k_scale[i] is None
        aa = K.AttnDecodeArgs(None if fused else K.ptr(b.q), K.ptr(self.k_cache[i]), K.ptr(self.v_cache[i]), K.ptr(b.positions), K.ptr(b.slots),
                              c.n_heads, c.n_kv_heads, self.n_ctx, self.n_splits, self.attn_scale, c.attn_softcap,
                              c.sliding_window if L.swa else 0, K.ptr(b.part_acc), K.ptr(b.part_ml), K.ptr(self.k_scale[i]),
                              K.ptr(self.v_scale[i]))
        if fused:
            # rotary embedding of the queries, rotation + cache append of the new key / value and the attention in one launch
            rr = K.AttnRopeArgs(K.ptr(b.qkv), K.ptr(inv_freq), mscale, c.rope_dim, int(c.rope_style == "neox"))
            lib.b2_attn_decode_rope.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
            rc = lib.b2_attn_decode_rope(C.byref(aa), C.byref(rr), C.byref(ca), nb, c.head_dim, int(self.pdl), st())
            if rc == 801:               # cudaErrorNotSupported: nothing was launched; this model keeps the separate kernel
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
            K._check(lib.b2_attn_decode(C.byref(aa), C.byref(ca), nb, c.head_dim, int(self.pdl), st()), "attn_decode")
            self._n += 3
        self._sk([L.sk.o], b.ao, b.x, nb, mode=SK.MODE_ACCUM)
        self._sk([L.sk.gu], b.x, b.hf, nb, norm_w=L.ffn_norm, mode=SK.MODE_GLU)
        self._sk([L.sk.down], b.hf, b.x, nb, mode=SK.MODE_ACCUM)

    def _decode_kernels(self, nb: int, want_argmax: bool) -> None:
        """Enqueue one decode step for ``nb`` sequences on the current stream (inputs: buf.tokens/positions/slots)."""
        c, b, lib, st = self.cfg, self.buf, K.lib(), K.stream
        self._n = 0
        if self.first:      # later pipeline stages find the residual stream of the previous stage in b.x
            K.embed(self.embd, b.tokens[:nb], c.embed_scale, out=b.x)
            self._n += 1
        act = K._ACT[c.act]
        for i, L in enumerate(self.layers):
            if L.sk is not None:
                self._decode_layer_sk(i, L, nb)
                continue
            self._norm_quant(b.x, L.attn_norm, nb, c.d_model)
            if (self.tc_decode_min and nb >= self.tc_decode_min and L.wqkv16 is not None
                    and all(w.wtype in (K.WT_BF16, K.WT_F16) for w in (L.wq, L.wk, L.wv))):
                self._gemm_step([L.wq], [L.wqkv16], nb, b.xf, b.qkv, bias=L.bqkv)      # Q, K and V in one product
            else:
                self._gemv([L.wq, L.wk, L.wv], nb, b.xq, b.xds, b.xf, b.qkv, b.qkv.stride(0))
            local = L.swa and c.rope_base_local > 0
            ra = K.RopeKvArgs(K.ptr(b.qkv), K.ptr(b.positions), K.ptr(b.slots), K.ptr(self.inv_freq_local if local else self.inv_freq),
                              K.ptr(L.q_norm), K.ptr(L.k_norm), c.norm_eps, 1.0 if local else self.mscale, c.n_heads, c.n_kv_heads,
                              c.head_dim, c.rope_dim, int(c.rope_style == "neox"), self.n_ctx, K.ptr(b.q), K.ptr(self.k_cache[i]),
                              K.ptr(self.v_cache[i]), K.ptr(self.k_scale[i]), K.ptr(self.v_scale[i]))
            K._check(lib.b2_rope_kv(C.byref(ra), nb, int(self.pdl), st()), "rope_kv")
            aa = K.AttnDecodeArgs(K.ptr(b.q), K.ptr(self.k_cache[i]), K.ptr(self.v_cache[i]), K.ptr(b.positions), K.ptr(b.slots),
                                  c.n_heads, c.n_kv_heads, self.n_ctx, self.n_splits, self.attn_scale, c.attn_softcap,
                                  c.sliding_window if L.swa else 0, K.ptr(b.part_acc), K.ptr(b.part_ml), K.ptr(self.k_scale[i]),
                                  K.ptr(self.v_scale[i]))
            ca = K.AttnCombineArgs(K.ptr(b.part_acc), K.ptr(b.part_ml), K.ptr(L.sinks), c.n_heads, self.n_splits, c.head_dim,
                                   K.ptr(b.ao), K.ptr(b.aq), K.ptr(b.ads))
            if self.fuse_attn_combine:      # the last CTA of every head group merges the splits: one launch instead of two
                K._check(lib.b2_attn_decode_fused(C.byref(aa), C.byref(ca), C.c_void_p(K.ptr(b.attn_tickets)), nb, c.head_dim, int(self.pdl), st()),
                         "attn_decode_fused")
                self._n += 2
            else:
                K._check(lib.b2_attn_decode(C.byref(aa), C.byref(ca), nb, c.head_dim, int(self.pdl), st()), "attn_decode")
                self._n += 3
            if c.sandwich_norm:
                self._gemv([L.wo], nb, b.aq, b.ads, b.ao, b.tmp, b.tmp.stride(0))
                self._norm_quant(b.tmp, L.post_attn_norm, nb, c.d_model, residual=b.x)
            else:
                self._gemv([L.wo], nb, b.aq, b.ads, b.ao, b.x, b.x.stride(0), accumulate=True)
            self._norm_quant(b.x, L.ffn_norm, nb, c.d_model)
            if L.moe:
                self._moe_decode(L, nb, act)
                continue
            ga = K.GluArgs()
            ga.gu = L.gu.desc()
            ga.nb, ga.xq, ga.xds, ga.xf = nb, K.ptr(b.xq), K.ptr(b.xds), K.ptr(b.xf)
            ga.act, ga.alpha, ga.limit = act, c.swiglu_alpha, c.swiglu_limit
            ga.hq, ga.hds, ga.hf = K.ptr(b.hq), K.ptr(b.hds), K.ptr(b.hf) if not L.down.quant_input else None
            K._check(lib.b2_gemv_glu_quant(C.byref(ga), int(self.pdl), st()), "gemv_glu_quant")
            self._n += 1
            if c.sandwich_norm:
                self._gemv([L.down], nb, b.hq, b.hds, b.hf, b.tmp, b.tmp.stride(0))
                self._norm_quant(b.tmp, L.post_ffw_norm, nb, c.d_model, residual=b.x)
            else:
                self._gemv([L.down], nb, b.hq, b.hds, b.hf, b.x, b.x.stride(0), accumulate=True)
        if not self.last:
            self.launches_per_step = self._n
            return
        if self.sk_head is not None:
            self._sk([self.sk_head], b.x, b.logits, nb, norm_w=self.out_norm)
        else:
            self._norm_quant(b.x, self.out_norm, nb, c.d_model)
            self._gemv([self.head], nb, b.xq, b.xds, b.xf, b.logits, b.logits.stride(0))
        if want_argmax:
            loop = want_argmax == "loop"      # the winner is fed back on the device: no host round trip between steps
            K.argmax(b.logits[:nb], out=b.sampled, tokens=b.tokens if loop else None, positions=b.positions if loop else None)
            self._n += 1
        self.launches_per_step = self._n

    def _run_step(self, nb: int, mode) -> None:
        """mode: False = logits only, True = + arg-max, "loop" = + arg-max and on-device token feedback."""
        key = (nb, mode)
        self.kernel_launches += self.launches_by_key.get(key, 0)
        if not self.use_graphs:
            self._decode_kernels(nb, mode)
            self.launches_by_key[key] = self.launches_per_step
            return
        g = self._graphs.get(key)
        if g is None:
            # the first call runs eagerly (loads the kernels); the second call records the graph
            if key not in self._warm:
                self._warm.add(key)
                self._decode_kernels(nb, mode)
                self.launches_by_key[key] = self.launches_per_step
                return
            g = torch.cuda.CUDAGraph()
            if self._capture_stream is None:      # torch's default capture stream belongs to whichever device captured first
                self._capture_stream = torch.cuda.Stream(device=self.device)
            with torch.cuda.device(self.device), torch.cuda.graph(g, stream=self._capture_stream):
                self._decode_kernels(nb, mode)
            self._graphs[key] = g
        g.replay()

    def _stage(self, slots, tokens, positions) -> int:
        nb = len(slots)
        if nb > self.max_batch:
            raise ValueError(f"decode batch {nb} exceeds {self.max_batch}")
        b = self.buf
        h = b.host_np
        h[0, :nb] = tokens
        h[1, :nb] = positions
        h[2, :nb] = slots
        b.meta.copy_(b.host_in, non_blocking=True)        # one pinned host -> device copy per step
        self.h2d_bytes += b.host_in.numel() * 4
        return nb

    @torch.no_grad()
    def decode_argmax(self, slots: Sequence[int], tokens: Sequence[int], positions: Sequence[int]) -> list[int]:
        if len(slots) > self.max_batch:      # more sequences than one step takes: consecutive steps
            out: list[int] = []
            for i in range(0, len(slots), self.max_batch):
                j = i + self.max_batch
                out += self.decode_argmax(slots[i:j], tokens[i:j], positions[i:j])
            return out
        nb = self._stage(slots, tokens, positions)
        self._run_step(nb, True)
        self.buf.host_out.copy_(self.buf.sampled, non_blocking=True)
        self.d2h_bytes += self.buf.host_out.numel() * 4
        torch.cuda.current_stream().synchronize()
        return self.buf.host_out_np[:nb].tolist()

    @torch.no_grad()
    def decode(self, slots, tokens, positions) -> torch.Tensor:
        if len(slots) > self.max_batch:
            mb = self.max_batch
            return torch.cat([self.decode(slots[i:i + mb], tokens[i:i + mb], positions[i:i + mb]) for i in range(0, len(slots), mb)])
        nb = self._stage(slots, tokens, positions)
        self._run_step(nb, False)
        return R.softcap(self.buf.logits[:nb].clone(), self.cfg.final_softcap)

    @torch.no_grad()
    def decode_loop(self, slots: Sequence[int], tokens: Sequence[int], positions: Sequence[int], n_steps: int,
                    first_tokens: torch.Tensor | None = None) -> torch.Tensor:
        """Greedy-decode ``n_steps`` tokens for every sequence without leaving the device.

        Returns the sampled ids as an int32 tensor [n_steps, nb] (still on the device).  Used by the
        benchmark's kernel-only measurement and by speculative prefixes where no stop condition can fire.
        """
        if len(slots) > self.max_batch:      # one group of sequences after the other
            parts = []
            for i in range(0, len(slots), self.max_batch):
                j = i + self.max_batch
                parts.append(self.decode_loop(slots[i:j], tokens[i:j], positions[i:j], n_steps,
                                              None if first_tokens is None else first_tokens[i:j]))
            return torch.cat(parts, 1)
        nb = self._stage(slots, tokens, positions)
        if first_tokens is not None:          # ids that are already on the device (e.g. the arg-max of the prefill logits)
            self.buf.tokens[:nb].copy_(first_tokens.to(torch.int32))
        out = torch.empty(n_steps, nb, device=self.device, dtype=torch.int32)
        for i in range(n_steps):
            self._run_step(nb, "loop")
            out[i].copy_(self.buf.sampled[:nb])
        return out

    # -- prefill --------------------------------------------------------------------------------------
    def _mm(self, x_bf16: torch.Tensor, w: K.DevWeight, out: torch.Tensor | None = None, out_off: int = 0, accumulate: bool = False,
            out16: bool = False) -> torch.Tensor:
        """x @ W^T + bias for a prefill chunk on the tcgen05 GEMM.

        ``out`` / ``out_off`` place the fp32 result in a column window of a wider buffer, ``accumulate`` adds to it (the
        residual add of the output and down projections happens in the GEMM epilogue), ``out16`` returns bf16 instead.
        """
        if self.prefill_gemm == "fused" and K.gemm_q_supported(w):
            self.kernel_launches += 1
            y = K.gemm_q(x_bf16, w, out=out, accumulate=accumulate, out_off=out_off)
            return y.to(torch.bfloat16) if out16 else y
        wb = getattr(w, "bf16", None)
        if wb is None:
            wb = K.dequant_to_bf16(w)        # scratch: freed (back to the caching allocator) when this call returns
            self.kernel_launches += 1
        self.kernel_launches += 1
        if out16:
            return K.gemm_bf16_out16(x_bf16, wb, w.bias)
        if out is not None:
            return K.gemm_bf16(x_bf16, wb, w.bias, out=out[:, out_off:out_off + w.n], accumulate=accumulate)
        return K.gemm_bf16(x_bf16, wb, w.bias)

    def _mm_glu(self, x_bf16: torch.Tensor, w: K.DevWeight) -> torch.Tensor:
        """act(gate) * up of the interleaved gate/up matrix for a prefill chunk, bf16 [T, d_ff]."""
        c = self.cfg
        if self.prefill_gemm == "fused" and K.gemm_q_supported(w):
            self.kernel_launches += 2
            gu = K.gemm_q(x_bf16, w).to(torch.bfloat16)                  # columns interleaved: even = gate, odd = up
            return K.glu_rows(gu, c.act, c.swiglu_alpha, c.swiglu_limit)
        wb = getattr(w, "bf16", None)
        if wb is None:
            wb = K.dequant_to_bf16(w)
            self.kernel_launches += 1
        self.kernel_launches += 1
        return K.gemm_bf16_glu(x_bf16, wb, c.act, w.bias, c.swiglu_alpha, c.swiglu_limit)

    def _attn_prefill(self, q: torch.Tensor, i: int, L, slot: int, pos0: int, p_end: int, spans=()) -> torch.Tensor:
        """Attention of a prefill chunk over cache positions [0, p_end): q [T, H, hd] fp32 -> bf16 [T, H * hd].  ``spans``
        (position ranges that attend to themselves in both directions: the rows of an image) take the plain tensor-op path,
        the kernels know the causal and windowed masks only; such chunks occur once per image."""
        c = self.cfg
        T = q.shape[0]
        window = c.sliding_window if L.swa else 0
        spans = [(lo, hi) for lo, hi in spans if lo < p_end and hi > pos0]
        if c.head_dim in K.ATTN_PREFILL_HEAD_DIMS and not spans:
            self.kernel_launches += 1
            return K.attn_prefill(q, self.k_cache[i], self.v_cache[i], slot, pos0, p_end, self.attn_scale, c.causal, window,
                                  c.attn_softcap, L.sinks, k_scale=self.k_scale[i], v_scale=self.v_scale[i])
        # head sizes without a flash-attention instantiation (32, 256): plain torch attention over the same cache rows
        kk = self.k_cache[i][slot, :, :p_end].transpose(0, 1).float()        # [S, Hkv, hd]
        vv = self.v_cache[i][slot, :, :p_end].transpose(0, 1).float()
        if self.k_scale[i] is not None:         # int8 cache: one f16 scale per 32 dims
            kk = (kk.reshape(*kk.shape[:2], -1, 32) * self.k_scale[i][slot, :, :p_end].transpose(0, 1).float()[..., None]).reshape(kk.shape)
            vv = (vv.reshape(*vv.shape[:2], -1, 32) * self.v_scale[i][slot, :, :p_end].transpose(0, 1).float()[..., None]).reshape(vv.shape)
        pos = torch.arange(pos0, p_end, device=q.device)
        o = R.attention(q, kk, vv, pos, torch.arange(p_end, device=q.device), scale=self.attn_scale, causal=c.causal, window=window,
                        softcap=c.attn_softcap, sinks=L.sinks, spans=spans)
        return o.reshape(T, -1).to(torch.bfloat16)

    @torch.no_grad()
    def _forward_chunk(self, slot: int, tokens: Sequence[int], pos0: int, x: torch.Tensor | None = None, embeds=None, spans=()) -> torch.Tensor:
        """Chunked prefill: returns the final hidden states [T, d_model] (fp32, before the output norm).

        ``x``: residual stream handed over by the previous pipeline stage (the token ids then only give the chunk length).
        ``embeds`` = (rows, [n, d_model] values): rows whose input embedding is given (image positions); ``spans``: position
        ranges that attend to themselves in both directions.
        """
        return self._forward_rows([(slot, tokens, pos0)], x, embeds, spans)

    @torch.no_grad()
    def _forward_rows(self, segs: Sequence[tuple[int, Sequence[int], int]], x: torch.Tensor | None = None, embeds=None, spans=()) -> torch.Tensor:
        """One pass over the rows of several chunks, each ``(slot, tokens, first position)`` of a different sequence: the
        projections, the feed-forward block and the cache append see one matrix of all rows, attention runs per sequence
        over its own cache rows.  Returns the hidden states of all rows in the order given."""
        c, dev = self.cfg, self.device
        flat = [max(int(t), 0) for _, toks, _ in segs for t in toks]      # negative ids stand for rows whose input comes from ``embeds``
        T = len(flat)
        ids = torch.tensor(flat, device=dev, dtype=torch.int32)
        if len(segs) == 1:
            slot, toks, pos0 = segs[0]
            pos = torch.arange(pos0, pos0 + T, device=dev, dtype=torch.int32)
            slots = torch.full((T,), slot, device=dev, dtype=torch.int32)
        else:
            pos = torch.tensor([p0 + j for _, toks, p0 in segs for j in range(len(toks))], device=dev, dtype=torch.int32)
            slots = torch.tensor([sl for sl, toks, _ in segs for _ in toks], device=dev, dtype=torch.int32)
        bounds, at = [], 0
        for sl, toks, p0 in segs:
            bounds.append((at, at + len(toks), sl, p0))
            at += len(toks)
        if x is None:
            x = K.embed(self.embd, ids, c.embed_scale)
            if embeds is not None and len(embeds[0]):      # image rows: projected features, not scaled like token embeddings
                x[torch.as_tensor(list(embeds[0]), device=dev)] = embeds[1].to(dev, x.dtype)
        for i, L in enumerate(self.layers):
            h = K.rmsnorm_bf16(x, L.attn_norm, c.norm_eps)
            qkv = torch.empty(T, (c.n_heads + 2 * c.n_kv_heads) * c.head_dim, device=dev, dtype=torch.float32)
            if getattr(L, "wqkv16", None) is not None:      # resident 16-bit copies: one GEMM for Q, K and V
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
            if len(bounds) == 1:
                o = self._attn_prefill(q, i, L, bounds[0][2], bounds[0][3], bounds[0][3] + T, spans)
            else:
                o = torch.cat([self._attn_prefill(q[r0:r1], i, L, sl, p0, p0 + r1 - r0) for r0, r1, sl, p0 in bounds])
            if c.sandwich_norm:
                x = x + R.rmsnorm(self._mm(o, L.wo), L.post_attn_norm, c.norm_eps)
            else:
                self._mm(o, L.wo, x, 0, accumulate=True)                  # residual add in the GEMM epilogue
            h = K.rmsnorm_bf16(x, L.ffn_norm, c.norm_eps)
            if L.moe:
                x = x + self._moe_prefill(h, L)
                continue
            f = self._mm_glu(h, L.gu)                                     # gate/up with the gated activation in the GEMM epilogue
            if c.sandwich_norm:
                x = x + R.rmsnorm(self._mm(f, L.down), L.post_ffw_norm, c.norm_eps)
            else:
                self._mm(f, L.down, x, 0, accumulate=True)
            self.kernel_launches += 3
        return x

    @torch.no_grad()
    def copy_rows(self, src: int, dst: int, n: int) -> None:
        """Cache rows [0, n) of slot ``src`` become rows [0, n) of slot ``dst``: a prompt prefix that another request already
        evaluated is copied on the device (a few MB per thousand tokens) instead of being evaluated again."""
        for i in range(len(self.layers)):
            for t in (self.k_cache[i], self.v_cache[i], self.k_scale[i], self.v_scale[i]):
                if t is not None:
                    t[dst, :, :n].copy_(t[src, :, :n])

    @torch.no_grad()
    def shift(self, slot: int, keep: int, discard: int, n: int) -> None:
        """Context shift in place: cache rows [keep, keep + discard) of ``slot`` are dropped, the rows behind them (up to
        ``n``) move down by ``discard`` and their keys, stored rotated, are turned back by ``discard`` positions
        (kvcache/causal.go:640-700).  int8 caches are expanded, rotated and quantised again with fresh block scales.  Runs
        once per ``n_ctx / 2`` generated tokens, so it is written with tensor ops rather than a kernel of its own."""
        c = self.cfg
        src, dst = slice(keep + discard, n), slice(keep, n - discard)
        back = torch.full((n - keep - discard,), -discard, device=self.device)
        for i, L in enumerate(self.layers):
            inv = self.inv_freq_local if (L.swa and c.rope_base_local > 0) else self.inv_freq
            kc, vc, ks, vs = self.k_cache[i], self.v_cache[i], self.k_scale[i], self.v_scale[i]
            k = kc[slot, :, src].float()                                   # [Hkv, S, hd]
            if ks is not None:
                k = (k.view(*k.shape[:2], -1, 32) * ks[slot, :, src].float()[..., None]).view_as(k)
            k = R.rope(k.transpose(0, 1), back, inv[: c.rope_dim // 2], c.rope_style, 1.0).transpose(0, 1)
            if ks is not None:
                blocks = k.reshape(*k.shape[:2], -1, 32)
                d = blocks.abs().amax(-1) / 127.0
                q = torch.where(d[..., None] > 0, blocks / d[..., None], torch.zeros_like(blocks)).round().clamp(-127, 127)
                kc[slot, :, dst] = q.view_as(k).to(torch.int8)
                ks[slot, :, dst] = d.to(torch.float16)
                vs[slot, :, dst] = vs[slot, :, src].clone()
            else:
                kc[slot, :, dst] = k.to(kc.dtype)
            vc[slot, :, dst] = vc[slot, :, src].clone()

    @torch.no_grad()
    def prefill_many(self, segs: Sequence[tuple[int, Sequence[int], int]], need_logits: Sequence[bool]) -> list:
        """Prefill chunks of several sequences in one pass (one set of GEMMs over all their rows).  Returns, per chunk, the
        logits after its last token where asked for, else None."""
        x = self._forward_rows(segs)
        ends, at = [], 0
        for _, toks, _ in segs:
            at += len(toks)
            ends.append(at - 1)
        want = [e for e, need in zip(ends, need_logits) if need]
        out: list = [None] * len(segs)
        if want:
            h = R.rmsnorm(x[torch.tensor(want, device=x.device)], self.out_norm, self.cfg.norm_eps).to(torch.bfloat16)
            logits = R.softcap(self._mm(h, self.head), self.cfg.final_softcap)
            for j, i in enumerate([i for i, need in enumerate(need_logits) if need]):
                out[i] = logits[j]
        return out

    supports_embeds = True

    @torch.no_grad()
    def prefill(self, slot: int, tokens: Sequence[int], pos0: int, need_logits: bool = True, embeds=None, spans=()):
        x = self._forward_chunk(slot, tokens, pos0, embeds=embeds, spans=spans)
        if not need_logits:
            return None
        h = R.rmsnorm(x[-1:], self.out_norm, self.cfg.norm_eps).to(torch.bfloat16)
        logits = self._mm(h, self.head)[0]
        return R.softcap(logits, self.cfg.final_softcap)

    @torch.no_grad()
    def verify(self, slot: int, tokens: Sequence[int], pos0: int) -> torch.Tensor:
        """Logits of every token of the chunk, [T, vocab]: the target-model pass of speculative decoding (one prefill-style
        pass over the drafted tokens instead of one decode step per token)."""
        x = self._forward_chunk(slot, tokens, pos0)
        h = R.rmsnorm(x, self.out_norm, self.cfg.norm_eps).to(torch.bfloat16)
        return R.softcap(self._mm(h, self.head), self.cfg.final_softcap)

    @torch.no_grad()
    def hidden(self, slot: int, tokens: Sequence[int]) -> torch.Tensor:
        x = self._forward_chunk(slot, tokens, 0)
        return R.rmsnorm(x, self.out_norm, self.cfg.norm_eps)
