"""In-memory normalisation of legacy GGUF spellings to the current conventions.

Older published blobs differ from today's key and tensor names; the reference fixes them while
loading (llama/compat/llama-ollama-compat.cpp:3239-3286 dispatches per architecture; gpt-oss rules
at :1510-1555, gemma3 at :237-275, llama3 tokenizer metadata at :1334-1355, mistral3 at :1643-1665, qwen2.5-vl at :1776-1840, qwen3-vl at
:1846-1868).  Here the same rules are a table applied to the opened :class:`GGUFFile` (nothing is written back to disk).
Vision-language checkpoints of the Qwen family are read as their text model: the decoder has the tensor names and key
names of qwen2 / qwen3 / qwen3moe under another prefix, and its multi-axis rotary embedding gives every axis the same
position for text tokens, which is the ordinary rotary embedding; the ``v.*`` / ``mm.*`` tensors stay in the file unread.  Set
``OLLAMA_LLAMA_CPP_COMPAT=0`` to switch the normaliser off (llama/compat/README.md:64-66).
"""
from __future__ import annotations

import os

from .reader import GGUFFile, TensorInfo
from .types import row_bytes

_GEMMA3_TEMPLATE = (
    "{{ bos_token }}{% for message in messages %}{% if message['role'] == 'assistant' %}{% set role = 'model' %}"
    "{% else %}{% set role = message['role'] %}{% endif %}<start_of_turn>{{ role }}\n{{ message['content'] | trim }}"
    "<end_of_turn>\n{% endfor %}{% if add_generation_prompt %}<start_of_turn>model\n{% endif %}"
)

# arch -> list of (needle, replacement) applied once per tensor name
_TENSOR_RENAMES = {
    "gpt-oss": [(".attn_out.", ".attn_output."), (".attn_sinks", ".attn_sinks.weight"), (".ffn_norm.", ".post_attention_norm.")],
}


def _rename_prefix(g: GGUFFile, old: str, new: str) -> None:
    for k in [k for k in g.kv if k.startswith(old)]:
        nk = new + k[len(old):]
        g.kv.setdefault(nk, g.kv[k])
        if k in g.kv_types:
            g.kv_types.setdefault(nk, g.kv_types[k])


def _rename_tensors(g: GGUFFile, rules) -> None:
    out = {}
    for name, ti in g.tensors.items():
        new = name
        for needle, repl in rules:
            if needle in new and repl not in new:
                new = new.replace(needle, repl, 1)
        if new.endswith(".weight.weight"):
            new = new[: -len(".weight")]
        ti.name = new
        out[new] = ti
    g.tensors.clear()
    g.tensors.update(out)


# architecture of a vision-language checkpoint -> the text architecture its decoder is
_TEXT_ARCH = {"qwen25vl": "qwen2", "qwen2vl": "qwen2", "qwen3vl": "qwen3", "qwen3vlmoe": "qwen3moe", "mistral3": "llama"}


def _row_views(g: GGUFFile, fused: str, parts: list[tuple[str, int]]) -> None:
    """Register ``parts`` (name, rows) as tensors that are consecutive row ranges of the stored tensor ``fused``: rows are the
    quantisation axis, so a row range of any encoding is a contiguous byte range of the stored data."""
    t = g.tensors.get(fused)
    if t is None or sum(n for _, n in parts) != t.shape[-1] or len(t.shape) != 2:
        return
    per_row = row_bytes(t.dtype, t.shape[0])
    at = 0
    for name, n in parts:
        if name not in g.tensors:
            g.tensors[name] = TensorInfo(name, (t.shape[0], n), t.dtype, t.offset + at * per_row, n * per_row)
        at += n


def _phi3(g: GGUFFile) -> None:
    """Phi-3 stores Q | K | V and gate | up as one matrix each (convert/convert_phi3.go:103-117); the decoder here reads the llama
    names, which become views into the fused tensors.  The per-frequency rotary divisors are the long set when the checkpoint's
    context is larger than the window it was trained on, else the short set."""
    u = lambda k, d=0: int(g.kv.get("phi3." + k, d) or d)                    # noqa: E731
    layers, d, heads = u("block_count"), u("embedding_length"), u("attention.head_count")
    kvh, ff = u("attention.head_count_kv", heads), u("feed_forward_length")
    if not (layers and d and heads):
        return
    hd = d // heads
    for i in range(layers):
        _row_views(g, f"blk.{i}.attn_qkv.weight", [(f"blk.{i}.attn_q.weight", heads * hd), (f"blk.{i}.attn_k.weight", kvh * hd), (f"blk.{i}.attn_v.weight", kvh * hd)])
        if f"blk.{i}.ffn_gate.weight" not in g.tensors and f"blk.{i}.ffn_up.weight" in g.tensors and g.tensors[f"blk.{i}.ffn_up.weight"].shape[-1] == 2 * ff:
            fused = g.tensors.pop(f"blk.{i}.ffn_up.weight")
            g.tensors[f"blk.{i}.ffn_gate_up.weight"] = fused
            _row_views(g, f"blk.{i}.ffn_gate_up.weight", [(f"blk.{i}.ffn_gate.weight", ff), (f"blk.{i}.ffn_up.weight", ff)])
        g.tensors.pop(f"blk.{i}.attn_qkv.weight", None)
        g.tensors.pop(f"blk.{i}.ffn_gate_up.weight", None)
    long_ctx = u("context_length") > u("rope.scaling.original_context_length", u("context_length"))
    pick = "rope_factors_long.weight" if long_ctx else "rope_factors_short.weight"
    if pick in g.tensors and "rope_freqs.weight" not in g.tensors:
        src = g.tensors[pick]
        g.tensors["rope_freqs.weight"] = TensorInfo("rope_freqs.weight", src.shape, src.dtype, src.offset, src.nbytes)
    if not long_ctx:
        g.kv.pop("phi3.rope.scaling.attn_factor", None)
    for name in ("rope_factors_long.weight", "rope_factors_short.weight"):
        g.tensors.pop(name, None)


def normalise(g: GGUFFile) -> GGUFFile:
    if os.environ.get("OLLAMA_LLAMA_CPP_COMPAT", "1") == "0":
        return g
    arch = g.kv.get("general.architecture", "")
    if arch == "phi3":
        _phi3(g)
    if arch == "mistral3":
        # llama/compat/llama-ollama-compat.cpp:1643-1665: YaRN keys under their current names, the tekken pre-tokenizer as default.
        # The decoder is llama's; its attention temperature (a factor on the queries that grows with log(position / trained
        # context)) is 1 inside the trained context and is not applied beyond it.
        for old, new in (("beta_fast", "yarn_beta_fast"), ("beta_slow", "yarn_beta_slow")):
            if f"mistral3.rope.scaling.{old}" in g.kv:
                g.kv.setdefault(f"mistral3.rope.scaling.{new}", g.kv[f"mistral3.rope.scaling.{old}"])
        if g.kv.get("tokenizer.ggml.pre", "default") in ("", "default"):
            g.kv["tokenizer.ggml.pre"] = "tekken"
    if arch in _TEXT_ARCH:
        text = _TEXT_ARCH[arch]
        g.kv["general.source_architecture"] = arch
        g.kv["general.architecture"] = text
        _rename_prefix(g, arch + ".", text + ".")
        for name in [n for n in g.tensors if n.startswith(("v.", "mm."))]:
            g.tensors.pop(name)                    # the vision tower and projector are not part of the text graph
        arch = text
    if arch == "gptoss":
        g.kv["general.architecture"] = "gpt-oss"
        _rename_prefix(g, "gptoss.", "gpt-oss.")
        if "gpt-oss.expert_feed_forward_length" not in g.kv and "blk.0.ffn_gate_exps.weight" in g.tensors:
            g.kv["gpt-oss.expert_feed_forward_length"] = int(g.tensors["blk.0.ffn_gate_exps.weight"].shape[1])
        g.kv.setdefault("gpt-oss.rope.scaling.type", "yarn")
        g.kv["tokenizer.ggml.pre"] = "gpt-4o"
        _rename_tensors(g, _TENSOR_RENAMES["gpt-oss"])
    elif arch == "gemma3":
        if "gemma3.rope.global.freq_base" in g.kv:
            g.kv.setdefault("gemma3.rope.freq_base", g.kv["gemma3.rope.global.freq_base"])
        if "gemma3.rope.freq_base_swa" in g.kv:
            g.kv.setdefault("gemma3.rope.local.freq_base", g.kv["gemma3.rope.freq_base_swa"])
        g.kv.setdefault("gemma3.attention.layer_norm_rms_epsilon", 1e-6)
        g.kv.setdefault("gemma3.rope.freq_base", 1000000.0)
        g.kv.setdefault("gemma3.rope.local.freq_base", 10000.0)
        g.kv.setdefault("tokenizer.chat_template", _GEMMA3_TEMPLATE)
        if int(g.kv.get("gemma3.context_length", 0)) >= 131072:
            g.kv.setdefault("gemma3.rope.scaling.type", "linear")
            g.kv.setdefault("gemma3.rope.scaling.factor", 8.0)
        # extra multimodal tokens beyond the embedding rows are dropped from the vocabulary arrays
        if "token_embd.weight" in g.tensors:
            rows = int(g.tensors["token_embd.weight"].shape[-1])
            for k in ("tokenizer.ggml.tokens", "tokenizer.ggml.scores", "tokenizer.ggml.token_type"):
                v = g.kv.get(k)
                if v is not None and hasattr(v, "__len__") and len(v) > rows:
                    g.kv[k] = v[:rows]
    elif arch == "llama":
        # Llama-3 blobs whose tokenizer block lacks the pre-tokenizer id / end-of-turn ids
        toks = g.kv.get("tokenizer.ggml.tokens")
        is_l3 = g.kv.get("tokenizer.ggml.model") == "gpt2" and toks is not None and len(toks) >= 128256
        if is_l3:
            if g.kv.get("tokenizer.ggml.pre", "default") in ("", "default"):
                g.kv["tokenizer.ggml.pre"] = "llama-bpe"
            if int(g.kv.get("tokenizer.ggml.eos_token_id", 128001)) == 128001:
                g.kv["tokenizer.ggml.eos_token_id"] = 128009
                g.kv["tokenizer.ggml.eos_token_ids"] = [128009]
    return g
