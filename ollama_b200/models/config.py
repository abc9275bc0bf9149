"""Architecture description derived from GGUF metadata.

One dataclass covers every decoder family served here (llama / mistral / mixtral, qwen2,
qwen3, qwen3moe, gemma, gemma2, gemma3, gpt-oss).  The keys read are the ones the reference
converters write (convert/convert_llama.go:49-104, convert_qwen3.go:35-73,
convert_gemma2.go:10-30, convert_gemma3.go:58-150, convert_gptoss.go:44-82) with the
defaults of the accessors in fs/ggml/ggml.go:35-185.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any

import numpy as np

SUPPORTED_ARCHS = ("llama", "mistral", "qwen2", "qwen3", "qwen3moe", "gemma", "gemma2", "gemma3", "gpt-oss", "phi3",
                   "bert", "nomic-bert")


@dataclass
class ModelConfig:
    arch: str = "llama"
    name: str = ""
    vocab_size: int = 0
    n_layers: int = 0
    d_model: int = 0
    n_heads: int = 0
    n_kv_heads: int = 0
    head_dim: int = 0              # key length
    v_head_dim: int = 0            # value length
    d_ff: int = 0
    ctx_train: int = 0
    norm_eps: float = 1e-5
    # rotary embedding
    rope_dim: int = 0
    rope_attn_factor: float = 0.0      # > 0: cos / sin are multiplied by this instead of the scale the rope scaling type implies
    rope_base: float = 10000.0
    rope_base_local: float = 0.0   # gemma3 sliding layers
    rope_style: str = "norm"       # "norm" = interleaved pairs (llama), "neox" = half-split
    rope_scaling_type: str = "none"  # none | linear | yarn | llama3(freq factors tensor)
    rope_scaling_factor: float = 1.0
    rope_orig_ctx: int = 0
    yarn_beta_fast: float = 32.0
    yarn_beta_slow: float = 1.0
    yarn_attn_factor: float = 1.0
    # block structure
    qk_norm: bool = False
    attn_bias: bool = False
    attn_out_bias: bool = False
    sandwich_norm: bool = False    # gemma2/3 post-attention and post-ffw norms
    act: str = "silu"              # silu | gelu_tanh | swiglu_oai
    embed_scale: float = 1.0
    attn_scale: float = 0.0        # 0 -> 1/sqrt(head_dim)
    attn_softcap: float = 0.0
    final_softcap: float = 0.0
    sliding_window: int = 0
    swa_layers: list[bool] = field(default_factory=list)   # per layer: True = sliding window
    attn_sinks: bool = False
    tied_embeddings: bool = False
    # mixture of experts
    n_experts: int = 0
    n_experts_used: int = 0
    d_ff_expert: int = 0
    moe_router: str = ""           # softmax_topk (qwen3moe, mixtral) | topk_softmax (gpt-oss)
    moe_norm_topk: bool = True
    moe_bias: bool = False
    swiglu_alpha: float = 1.702
    swiglu_limit: float = 7.0
    # pooling (embedding models)
    pooling: str = "none"          # none | mean | cls | last
    causal: bool = True

    @property
    def is_moe(self) -> bool:
        return self.n_experts > 0

    @property
    def scale(self) -> float:
        return self.attn_scale if self.attn_scale > 0 else 1.0 / math.sqrt(self.head_dim)

    @property
    def q_dim(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.n_kv_heads * self.head_dim

    def layer_is_swa(self, i: int) -> bool:
        return bool(self.swa_layers[i]) if self.swa_layers else False

    def layer_rope_base(self, i: int) -> float:
        if self.rope_base_local > 0 and self.layer_is_swa(i):
            return self.rope_base_local
        return self.rope_base

    def kv_bytes_per_token(self, elem_bytes: int = 2) -> int:
        return self.n_layers * (self.n_kv_heads * (self.head_dim + self.v_head_dim)) * elem_bytes


def _first(v: Any, default: int) -> int:
    if v is None:
        return default
    if isinstance(v, (list, np.ndarray)):
        vals = [int(x) for x in v if int(x) > 0]
        return vals[0] if vals else default
    return int(v)


def config_from_gguf(g) -> ModelConfig:
    """Build a :class:`ModelConfig` from an opened :class:`GGUFFile`."""
    arch = g.architecture
    if arch == "gptoss":          # legacy spelling used by older blobs (llama/compat/llama-ollama-compat.cpp:1510-1555)
        arch = "gpt-oss"
    c = ModelConfig(arch=arch, name=g.kv.get("general.name", ""))
    u, f = g.uint, g.float
    c.n_layers = u("block_count")
    c.d_model = u("embedding_length")
    c.n_heads = _first(g.get("attention.head_count"), 0)
    c.n_kv_heads = _first(g.get("attention.head_count_kv"), c.n_heads)
    c.head_dim = u("attention.key_length", c.d_model // max(c.n_heads, 1))
    c.v_head_dim = u("attention.value_length", c.head_dim)
    c.d_ff = _first(g.get("feed_forward_length"), 0)
    c.ctx_train = u("context_length", 2048)
    c.norm_eps = f("attention.layer_norm_rms_epsilon", f("attention.layer_norm_epsilon", 1e-5))
    c.rope_dim = u("rope.dimension_count", c.head_dim)
    c.rope_base = f("rope.freq_base", 10000.0)
    c.rope_scaling_type = g.string("rope.scaling.type", "none")
    c.rope_scaling_factor = f("rope.scaling.factor", 1.0)
    c.rope_orig_ctx = u("rope.scaling.original_context_length", 0)
    c.yarn_beta_fast = f("rope.scaling.yarn_beta_fast", 32.0)
    c.yarn_beta_slow = f("rope.scaling.yarn_beta_slow", 1.0)
    c.n_experts = u("expert_count", 0)
    c.n_experts_used = u("expert_used_count", 0)
    c.d_ff_expert = u("expert_feed_forward_length", c.d_ff)
    toks = g.kv.get("tokenizer.ggml.tokens")
    c.vocab_size = u("vocab_size", len(toks) if toks is not None else 0)
    if c.vocab_size == 0 and g.has("token_embd.weight"):
        c.vocab_size = g.tensors["token_embd.weight"].shape[-1]
    c.tied_embeddings = not g.has("output.weight")
    c.sliding_window = u("attention.sliding_window", 0)

    if arch in ("llama", "mistral"):
        c.rope_style = "norm"
        if c.is_moe:
            c.moe_router, c.moe_norm_topk = "softmax_topk", True
        if g.has("rope_freqs.weight"):
            c.rope_scaling_type = "llama3"
    elif arch == "phi3":
        # llama-shaped once the fused matrices are split into views (gguf/compat.py); rotary pairs in the half-split order,
        # per-frequency divisors in rope_freqs.weight, cos / sin scaled by the attention factor of the long-context recipe
        c.rope_style = "neox"
        c.rope_attn_factor = f("rope.scaling.attn_factor", 0.0) if g.has("rope_freqs.weight") else 0.0
        c.rope_scaling_type = "none"
        if 0 < c.sliding_window < c.ctx_train:
            c.swa_layers = [True] * c.n_layers          # every layer attends within the window
    elif arch == "qwen2":
        c.rope_style, c.attn_bias = "neox", True
    elif arch in ("qwen3", "qwen3moe"):
        c.rope_style, c.qk_norm = "neox", True
        if arch == "qwen3moe":
            c.moe_router = "softmax_topk"
            c.moe_norm_topk = g.bool("norm_top_k_prob", True)
    elif arch in ("gemma", "gemma2", "gemma3"):
        c.rope_style, c.act = "neox", "gelu_tanh"
        c.embed_scale = math.sqrt(c.d_model)
        c.tied_embeddings = not g.has("output.weight")
        if arch in ("gemma2", "gemma3"):
            c.sandwich_norm = True
        if arch == "gemma2":
            c.attn_softcap = f("attn_logit_softcapping", 50.0)
            c.final_softcap = f("final_logit_softcapping", 30.0)
            if c.sliding_window:
                c.swa_layers = [i % 2 == 0 for i in range(c.n_layers)]
        if arch == "gemma3":
            c.qk_norm = True
            c.final_softcap = f("final_logit_softcapping", 0.0)
            c.rope_base_local = f("rope.local.freq_base", 10000.0)
            pat = g.get("attention.sliding_window_pattern")
            if isinstance(pat, (list, np.ndarray)) and len(pat) >= c.n_layers:
                c.swa_layers = [bool(x) for x in pat[: c.n_layers]]
            else:
                period = int(pat) if pat is not None and not isinstance(pat, (list, np.ndarray)) else 6
                c.swa_layers = [(i + 1) % period != 0 for i in range(c.n_layers)]
            if c.sliding_window == 0:
                c.sliding_window = 1024
    elif arch == "gpt-oss":
        c.rope_style, c.act = "neox", "swiglu_oai"
        c.attn_bias = c.attn_out_bias = True
        c.attn_sinks = True
        c.moe_router, c.moe_bias = "topk_softmax", True
        if c.rope_scaling_type in ("", "none") and c.rope_scaling_factor > 1.0:
            c.rope_scaling_type = "yarn"
        if c.sliding_window == 0:
            c.sliding_window = 128
        # alternating window / full layers, even layers use the window (fs/ggml/ggml.go:877-886)
        c.swa_layers = [i % 2 == 0 for i in range(c.n_layers)]
    elif arch in ("bert", "nomic-bert"):
        c.causal = False
        c.pooling = {0: "none", 1: "mean", 2: "cls", 3: "last"}.get(u("pooling_type", 1), "mean")
    else:
        raise NotImplementedError(f"unsupported model architecture {arch!r}")
    pt = g.get("pooling_type")
    if pt is not None and arch not in ("bert", "nomic-bert"):
        c.pooling = {0: "none", 1: "mean", 2: "cls", 3: "last"}.get(int(pt), "none")
    if c.rope_scaling_type == "yarn":
        # attention temperature used with YaRN: 0.1 ln(s) + 1
        c.yarn_attn_factor = 0.1 * math.log(max(c.rope_scaling_factor, 1.0)) + 1.0
    return c
