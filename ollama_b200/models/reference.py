"""Reference decoder graph in plain PyTorch.

Runs any supported GGUF (llama, qwen2, qwen3, qwen3moe, gemma/2/3, gpt-oss, mixtral) on any torch
device in fp32.  It is both the CPU execution path and the oracle that the sm_100a engine is
checked against.  Block structure per family follows the graphs the reference keeps in source
(x/models/llama/llama.go:240-316, x/models/qwen3/qwen3.go:300-335,
x/models/gemma3/gemma3.go:199-202,442-466,511) and the GGUF conventions of its converters
(interleaved RoPE for llama because Q/K rows are permuted at conversion,
convert/convert_llama.go:189-232; gemma norm weights already hold 1+w, convert/convert_gemma.go:47-50).
"""
from __future__ import annotations

import math

import torch

from ..ops import reference as R
from .config import ModelConfig
from .weights import QWeight

_DEQUANT_CACHE_LIMIT = 1 << 28   # cache dequantised copies only for small models (elements)


class RefKVCache:
    """Slot-partitioned cache: k/v[layer] has shape [n_slots, n_ctx, n_kv_heads, head_dim]."""

    def __init__(self, cfg: ModelConfig, n_slots: int, n_ctx: int, device="cpu", dtype=torch.float32):
        self.n_slots, self.n_ctx = n_slots, n_ctx
        self.k = [torch.zeros(n_slots, n_ctx, cfg.n_kv_heads, cfg.head_dim, device=device, dtype=dtype) for _ in range(cfg.n_layers)]
        self.v = [torch.zeros(n_slots, n_ctx, cfg.n_kv_heads, cfg.v_head_dim, device=device, dtype=dtype) for _ in range(cfg.n_layers)]

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.k + self.v)


class ReferenceModel:
    def __init__(self, cfg: ModelConfig, weights: dict[str, QWeight], device="cpu"):
        self.cfg, self.w, self.device = cfg, weights, torch.device(device)
        self._dq: dict[str, torch.Tensor] = {}
        total = sum(int(math.prod(q.shape)) for q in weights.values())
        self._cache_ok = total <= _DEQUANT_CACHE_LIMIT
        c = cfg
        ff = self._f("rope_freqs.weight") if "rope_freqs.weight" in weights else None
        kw = dict(scaling=c.rope_scaling_type if c.rope_scaling_type != "llama3" else "none", factor=c.rope_scaling_factor,
                  orig_ctx=c.rope_orig_ctx, beta_fast=c.yarn_beta_fast, beta_slow=c.yarn_beta_slow, device=self.device)
        self.inv_freq, self.mscale = R.rope_inv_freq(c.rope_dim, c.rope_base, freq_factors=ff, **kw)
        if c.rope_attn_factor > 0:
            self.mscale = c.rope_attn_factor
        if c.rope_base_local > 0:
            # sliding-window layers of gemma3 use their own base and no context scaling
            self.inv_freq_local, _ = R.rope_inv_freq(c.rope_dim, c.rope_base_local, device=self.device)
        else:
            self.inv_freq_local = self.inv_freq
        self.attn_scale = c.scale
        if c.arch in ("gemma2", "gemma3") and c.n_layers in (46, 62):   # 27B variants scale by d_model / n_heads
            self.attn_scale = 1.0 / math.sqrt(c.d_model / c.n_heads)

    # -- weight access ------------------------------------------------------------------------
    def _f(self, name: str) -> torch.Tensor:
        t = self._dq.get(name)
        if t is None:
            t = self.w[name].dequant().to(self.device)
            if self._cache_ok or t.numel() < (1 << 22):
                self._dq[name] = t
        return t

    def _has(self, name: str) -> bool:
        return name in self.w

    def _linear(self, x: torch.Tensor, name: str) -> torch.Tensor:
        y = x.float() @ self._f(name + ".weight").t()
        if self._has(name + ".bias"):
            y = y + self._f(name + ".bias")
        return y

    def new_cache(self, n_slots: int, n_ctx: int) -> RefKVCache:
        return RefKVCache(self.cfg, n_slots, n_ctx, self.device)

    # -- blocks ---------------------------------------------------------------------------------
    def layer_rope(self, i: int) -> torch.Tensor:
        """Rotary frequencies of layer ``i`` (sliding-window layers of gemma3 have their own)."""
        return self.inv_freq_local if (self.cfg.layer_is_swa(i) and self.cfg.rope_base_local > 0) else self.inv_freq

    @torch.no_grad()
    def shift_cache(self, cache: RefKVCache, slot: int, keep: int, discard: int, n: int) -> None:
        """Drop cache rows [keep, keep + discard) of ``slot``: rows [keep + discard, n) move down by ``discard`` and their
        keys, stored rotated, are turned back by ``discard`` positions so that they carry their new positions
        (kvcache/causal.go:640-700 does the same with a RoPE-shift graph).  Values only move."""
        src, dst = slice(keep + discard, n), slice(keep, n - discard)
        back = torch.full((n - keep - discard,), -discard, device=self.device)
        for i in range(self.cfg.n_layers):
            k = R.rope(cache.k[i][slot, src], back, self.layer_rope(i), self.cfg.rope_style, 1.0)
            cache.k[i][slot, dst] = k.to(cache.k[i].dtype)
            cache.v[i][slot, dst] = cache.v[i][slot, src].clone()

    def _mlp(self, h: torch.Tensor, p: str) -> torch.Tensor:
        c = self.cfg
        if not c.is_moe or not self._has(p + "ffn_gate_inp.weight"):
            g = self._linear(h, p + "ffn_gate")
            u = self._linear(h, p + "ffn_up")
            return self._linear(R.glu(g, u, c.act, c.swiglu_alpha, c.swiglu_limit), p + "ffn_down")
        logits = self._linear(h, p + "ffn_gate_inp")
        ids, wts = R.moe_route(logits, c.n_experts_used, c.moe_router, c.moe_norm_topk)
        out = torch.zeros(h.shape[0], c.d_model, device=h.device)
        wg, wu, wd = self.w[p + "ffn_gate_exps.weight"], self.w[p + "ffn_up_exps.weight"], self.w[p + "ffn_down_exps.weight"]
        bias = {k: self._f(p + f"ffn_{k}_exps.bias") for k in ("gate", "up", "down") if self._has(p + f"ffn_{k}_exps.bias")}
        for e in ids.unique().tolist():
            tok, slot = (ids == e).nonzero(as_tuple=True)
            x = h[tok].float()
            g = x @ self._expert(wg, e).t()
            u = x @ self._expert(wu, e).t()
            if "gate" in bias:
                g, u = g + bias["gate"][e], u + bias["up"][e]
            y = R.glu(g, u, c.act, c.swiglu_alpha, c.swiglu_limit) @ self._expert(wd, e).t()
            if "down" in bias:
                y = y + bias["down"][e]
            out.index_add_(0, tok, y * wts[tok, slot][:, None])
        return out

    def _expert(self, w: QWeight, e: int) -> torch.Tensor:
        key = f"{w.name}#{e}"
        t = self._dq.get(key)
        if t is None:
            t = w.expert(e).dequant().to(self.device)
            if self._cache_ok:
                self._dq[key] = t
        return t

    def embed_tokens(self, tokens: torch.Tensor) -> torch.Tensor:
        w = self.w["token_embd.weight"]
        if "token_embd.weight" in self._dq or self._cache_ok:
            x = self._f("token_embd.weight")[tokens]
        else:  # gather quantised rows, then decode only those
            rb = w.row_nbytes
            rows = w.raw.view(w.shape[0], rb)[tokens.cpu()]
            from ..gguf import quants
            x = quants.dequantize(rows.reshape(-1), w.dtype).view(len(tokens), w.shape[1]).to(self.device)
        return x * self.cfg.embed_scale

    def forward(self, tokens: torch.Tensor, positions: torch.Tensor, cache: RefKVCache, slot: int,
                logit_rows: torch.Tensor | None = None, return_hidden: bool = False, embeds=None, spans=()) -> torch.Tensor:
        """Run ``tokens`` ([T]) at ``positions`` ([T]) for one slot; writes K/V at those positions.

        Returns logits for ``logit_rows`` (default: the last token) as [R, vocab], or the final normed
        hidden states [T, d_model] when ``return_hidden``.  ``embeds`` = (rows, values): rows of the chunk whose input is the
        given embedding (an image position; not scaled like a token embedding) instead of the token's; ``spans``: position
        ranges [lo, hi) that attend to themselves in both directions.
        """
        c = self.cfg
        tokens = tokens.to(self.device)
        positions = positions.to(self.device)
        T = tokens.shape[0]
        x = self.embed_tokens(tokens.clamp(min=0))
        if embeds is not None and len(embeds[0]):
            x[torch.as_tensor(embeds[0], device=self.device)] = embeds[1].to(self.device, x.dtype)
        p_end = int(positions.max().item()) + 1
        k_pos = torch.arange(p_end, device=self.device)
        for i in range(c.n_layers):
            p = f"blk.{i}."
            h = R.rmsnorm(x, self._f(p + "attn_norm.weight"), c.norm_eps)
            q = self._linear(h, p + "attn_q").view(T, c.n_heads, c.head_dim)
            k = self._linear(h, p + "attn_k").view(T, c.n_kv_heads, c.head_dim)
            v = self._linear(h, p + "attn_v").view(T, c.n_kv_heads, c.v_head_dim)
            if c.qk_norm:
                q = R.rmsnorm(q, self._f(p + "attn_q_norm.weight"), c.norm_eps)
                k = R.rmsnorm(k, self._f(p + "attn_k_norm.weight"), c.norm_eps)
            swa = c.layer_is_swa(i)
            inv = self.inv_freq_local if (swa and c.rope_base_local > 0) else self.inv_freq
            ms = 1.0 if (swa and c.rope_base_local > 0) else self.mscale
            q = R.rope(q, positions, inv, c.rope_style, ms)
            k = R.rope(k, positions, inv, c.rope_style, ms)
            cache.k[i][slot, positions] = k.to(cache.k[i].dtype)
            cache.v[i][slot, positions] = v.to(cache.v[i].dtype)
            sinks = self._f(p + "attn_sinks.weight") if c.attn_sinks and self._has(p + "attn_sinks.weight") else None
            o = R.attention(q, cache.k[i][slot, :p_end], cache.v[i][slot, :p_end], positions, k_pos,
                            scale=self.attn_scale, causal=c.causal, window=c.sliding_window if swa else 0,
                            softcap=c.attn_softcap, sinks=sinks, spans=spans)
            o = self._linear(o.reshape(T, -1), p + "attn_output")
            if c.sandwich_norm:
                o = R.rmsnorm(o, self._f(p + "post_attention_norm.weight"), c.norm_eps)
            x = x + o
            ffn_norm = p + "ffn_norm.weight"
            if not self._has(ffn_norm):
                ffn_norm = p + "post_attention_norm.weight"     # gpt-oss names its pre-FFN norm this way
            h = R.rmsnorm(x, self._f(ffn_norm), c.norm_eps)
            f = self._mlp(h, p)
            if c.sandwich_norm:
                f = R.rmsnorm(f, self._f(p + "post_ffw_norm.weight"), c.norm_eps)
            x = x + f
        x = R.rmsnorm(x, self._f("output_norm.weight"), c.norm_eps)
        if return_hidden:
            return x
        rows = x[-1:] if logit_rows is None else x[logit_rows]
        head = "output" if self._has("output.weight") else "token_embd"
        logits = rows @ self._f(head + ".weight").t()
        if self._has("output.bias"):
            logits = logits + self._f("output.bias")
        return R.softcap(logits, c.final_softcap)
