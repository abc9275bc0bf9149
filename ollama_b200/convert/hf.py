"""Hugging Face checkpoint directory (config.json + *.safetensors + tokenizer files) -> GGUF.

Covers the decoder families this runtime executes: Llama / Mistral, Mixtral, Qwen2, Qwen3, Qwen3-MoE,
Gemma, Gemma 2 and Gemma 3 (text tower), gpt-oss (16-bit expert tensors, or experts packed as
MXFP4 blocks + scales, which are re-ordered into GGML MXFP4 blocks without re-quantising).  Mirrors convert/convert.go:279-379 (dispatch by
``architectures[0]``), convert/convert_llama.go (key/value metadata, the Q/K row permutation that turns the
checkpoint's half-split rotary layout into the interleaved one llama-arch GGUFs use:189-232),
convert/convert_qwen3.go, convert_gemma*.go, convert_mixtral.go (expert stacking) and convert/tokenizer.go
(vocabulary, merges, token types, pretokenizer identification, special token ids, chat template).

Tensors keep their source precision (F16/BF16 matrices, F32 vectors) unless ``outtype`` asks otherwise;
quantisation is a separate pass (store/create.py quantize_gguf).
"""
from __future__ import annotations

import json
import math
import os
import re
from typing import Any, Callable, Iterator

import torch

from ..gguf import quants
from ..gguf.types import GGMLType
from ..gguf.writer import WriteTensor, write_gguf
from .safetensors import ModelDir


class ConvertError(ValueError):
    pass


ARCHS = {
    "LlamaForCausalLM": "llama", "MistralForCausalLM": "llama", "MixtralForCausalLM": "llama", "Qwen2ForCausalLM": "qwen2",
    "Qwen3ForCausalLM": "qwen3", "Qwen3MoeForCausalLM": "qwen3moe", "GemmaForCausalLM": "gemma", "Gemma2ForCausalLM": "gemma2",
    "Gemma3ForCausalLM": "gemma3", "Gemma3ForConditionalGeneration": "gemma3", "GptOssForCausalLM": "gpt-oss",
    "Phi3ForCausalLM": "phi3",
}

# (pattern on the checkpoint name, GGUF name); {n} = layer index, {e} = expert index
_LAYER = r"(?:model\.)?(?:language_model\.)?(?:model\.)?layers\.(\d+)\."
_RULES: list[tuple[str, str]] = [
    (r"(?:model\.)?(?:language_model\.)?(?:model\.)?embed_tokens\.weight", "token_embd.weight"),
    (r"(?:model\.)?(?:language_model\.)?(?:model\.)?norm\.weight", "output_norm.weight"),
    (r"(?:model\.)?(?:language_model\.)?lm_head\.weight", "output.weight"),
    (_LAYER + r"input_layernorm\.weight", "blk.{n}.attn_norm.weight"),
    (_LAYER + r"self_attn\.q_proj\.(weight|bias)", "blk.{n}.attn_q.{1}"),
    (_LAYER + r"self_attn\.k_proj\.(weight|bias)", "blk.{n}.attn_k.{1}"),
    (_LAYER + r"self_attn\.v_proj\.(weight|bias)", "blk.{n}.attn_v.{1}"),
    (_LAYER + r"self_attn\.o_proj\.(weight|bias)", "blk.{n}.attn_output.{1}"),
    # phi3: Q, K and V in one matrix, gate and up in one matrix (convert/convert_phi3.go:103-117); split into views at load
    (_LAYER + r"self_attn\.qkv_proj\.weight", "blk.{n}.attn_qkv.weight"),
    (_LAYER + r"mlp\.gate_up_proj\.weight", "blk.{n}.ffn_up.weight"),
    (_LAYER + r"self_attn\.q_norm\.weight", "blk.{n}.attn_q_norm.weight"),
    (_LAYER + r"self_attn\.k_norm\.weight", "blk.{n}.attn_k_norm.weight"),
    (_LAYER + r"mlp\.gate_proj\.weight", "blk.{n}.ffn_gate.weight"),
    (_LAYER + r"mlp\.up_proj\.weight", "blk.{n}.ffn_up.weight"),
    (_LAYER + r"mlp\.down_proj\.weight", "blk.{n}.ffn_down.weight"),
    (_LAYER + r"mlp\.gate\.weight", "blk.{n}.ffn_gate_inp.weight"),
    (_LAYER + r"block_sparse_moe\.gate\.weight", "blk.{n}.ffn_gate_inp.weight"),
    (_LAYER + r"mlp\.experts\.(\d+)\.gate_proj\.weight", "blk.{n}.ffn_gate_exps.weight#{1}"),
    (_LAYER + r"mlp\.experts\.(\d+)\.up_proj\.weight", "blk.{n}.ffn_up_exps.weight#{1}"),
    (_LAYER + r"mlp\.experts\.(\d+)\.down_proj\.weight", "blk.{n}.ffn_down_exps.weight#{1}"),
    (_LAYER + r"block_sparse_moe\.experts\.(\d+)\.w1\.weight", "blk.{n}.ffn_gate_exps.weight#{1}"),
    (_LAYER + r"block_sparse_moe\.experts\.(\d+)\.w3\.weight", "blk.{n}.ffn_up_exps.weight#{1}"),
    (_LAYER + r"block_sparse_moe\.experts\.(\d+)\.w2\.weight", "blk.{n}.ffn_down_exps.weight#{1}"),
    # gpt-oss: stacked experts stored [expert, in, out] with gate / up interleaved along `out` (split and transposed in convert_tensors)
    (_LAYER + r"self_attn\.sinks", "blk.{n}.attn_sinks.weight"),
    (_LAYER + r"mlp\.router\.(weight|bias)", "blk.{n}.ffn_gate_inp.{1}"),
    (_LAYER + r"mlp\.experts\.gate_up_proj", "blk.{n}.ffn_gate_up_exps.weight"),
    (_LAYER + r"mlp\.experts\.gate_up_proj_bias", "blk.{n}.ffn_gate_up_exps.bias"),
    (_LAYER + r"mlp\.experts\.down_proj", "blk.{n}.ffn_down_exps.weight@T"),
    (_LAYER + r"mlp\.experts\.down_proj_bias", "blk.{n}.ffn_down_exps.bias"),
    # gpt-oss checkpoints with MXFP4-packed experts: [expert, out, in / 32, 16] nibble bytes + [expert, out, in / 32] e8m0 scales
    (_LAYER + r"mlp\.experts\.gate_up_proj_(blocks|scales)", "blk.{n}.ffn_gate_up_exps.{1}"),
    (_LAYER + r"mlp\.experts\.down_proj_(blocks|scales)", "blk.{n}.ffn_down_exps.{1}"),
]
# post_attention_layernorm is the FFN pre-norm for llama/qwen but a sandwich post-norm for gemma 2/3
_RULES_PRENORM = [(_LAYER + r"post_attention_layernorm\.weight", "blk.{n}.ffn_norm.weight")]
_RULES_SANDWICH = [(_LAYER + r"post_attention_layernorm\.weight", "blk.{n}.post_attention_norm.weight"),
                   (_LAYER + r"pre_feedforward_layernorm\.weight", "blk.{n}.ffn_norm.weight"),
                   (_LAYER + r"post_feedforward_layernorm\.weight", "blk.{n}.post_ffw_norm.weight")]
_SKIP = re.compile(r".*(rotary_emb\.inv_freq|vision_tower|multi_modal_projector|vision_model|audio_tower).*")


# SigLIP tower and projector of a multimodal gemma3 checkpoint (convert/convert_gemma3.go:155-188)
_VISION_PREFIX = re.compile(r"(?:model\.)?(?:vision_tower|vision_model)\.vision_model\.(.*)")
_VISION_RULES = [
    (r"embeddings\.patch_embedding\.(weight|bias)", r"v.patch_embedding.\1"),
    (r"embeddings\.position_embedding\.weight", "v.position_embedding.weight"),
    (r"encoder\.layers\.(\d+)\.layer_norm([12])\.(weight|bias)", r"v.blk.\1.layer_norm\2.\3"),
    (r"encoder\.layers\.(\d+)\.self_attn\.q_proj\.(weight|bias)", r"v.blk.\1.attn_q.\2"),
    (r"encoder\.layers\.(\d+)\.self_attn\.k_proj\.(weight|bias)", r"v.blk.\1.attn_k.\2"),
    (r"encoder\.layers\.(\d+)\.self_attn\.v_proj\.(weight|bias)", r"v.blk.\1.attn_v.\2"),
    (r"encoder\.layers\.(\d+)\.self_attn\.out_proj\.(weight|bias)", r"v.blk.\1.attn_output.\2"),
    (r"encoder\.layers\.(\d+)\.mlp\.fc([12])\.(weight|bias)", r"v.blk.\1.mlp.fc\2.\3"),
    (r"post_layernorm\.(weight|bias)", r"v.post_layernorm.\1"),
]


def map_vision_name(name: str) -> str | None:
    """GGUF name of a vision-tower / projector tensor of a multimodal gemma3 checkpoint, or None."""
    m = re.fullmatch(r"(?:model\.)?multi_modal_projector\.mm_input_projection_weight", name)
    if m:
        return "mm.mm_input_projection.weight"
    if re.fullmatch(r"(?:model\.)?multi_modal_projector\.mm_soft_emb_norm\.weight", name):
        return "mm.mm_soft_emb_norm.weight"
    m = _VISION_PREFIX.fullmatch(name)
    if not m:
        return None
    for pat, repl in _VISION_RULES:
        if re.fullmatch(pat, m.group(1)):
            return re.sub(pat, repl, m.group(1))
    return None


def map_name(name: str, arch: str) -> str | None:
    rules = _RULES + (_RULES_SANDWICH if arch in ("gemma2", "gemma3") else _RULES_PRENORM)
    for pat, repl in rules:
        m = re.fullmatch(pat, name)
        if m:
            groups = m.groups()
            out = repl
            if "{n}" in repl:
                out = out.replace("{n}", groups[0])
                groups = groups[1:]
            for i, g in enumerate(groups, 1):
                out = out.replace("{%d}" % i, g)
            return out
    return None


def permute_qk(w: torch.Tensor, n_head: int) -> torch.Tensor:
    """Rows of a Q or K projection: half-split rotary order (HF) -> interleaved pairs (llama-arch GGUF)."""
    rows = w.shape[0]
    hd = rows // n_head
    rest = w.shape[1:]
    return w.reshape(n_head, 2, hd // 2, *rest).transpose(1, 2).reshape(rows, *rest)


def _kv(cfg: dict[str, Any], arch: str, name: str) -> dict[str, Any]:
    c = cfg.get("text_config", cfg) if arch == "gemma3" else cfg
    n_head = c["num_attention_heads"]
    hd = c.get("head_dim") or c["hidden_size"] // n_head
    kv: dict[str, Any] = {
        "general.architecture": arch, "general.name": name, "general.file_type": 1,
        f"{arch}.context_length": c.get("max_position_embeddings", 8192), f"{arch}.embedding_length": c["hidden_size"],
        f"{arch}.block_count": c["num_hidden_layers"], f"{arch}.feed_forward_length": c.get("intermediate_size", 0),
        f"{arch}.attention.head_count": n_head, f"{arch}.attention.head_count_kv": c.get("num_key_value_heads", n_head),
        f"{arch}.attention.layer_norm_rms_epsilon": float(c.get("rms_norm_eps", 1e-6)),
        f"{arch}.rope.freq_base": float(c.get("rope_theta") or (c.get("rope_parameters") or {}).get("rope_theta") or 10000.0),
        f"{arch}.vocab_size": c.get("vocab_size", 0),
    }
    if c.get("head_dim") or arch in ("qwen3", "qwen3moe", "gemma", "gemma2", "gemma3"):
        kv[f"{arch}.attention.key_length"] = hd
        kv[f"{arch}.attention.value_length"] = hd
    if arch == "llama":
        kv["llama.rope.dimension_count"] = hd
    vc = cfg.get("vision_config") if arch == "gemma3" else None
    if isinstance(vc, dict):     # convert/convert_gemma3.go:134-151
        kv["gemma3.vision.block_count"] = vc.get("num_hidden_layers", 27)
        kv["gemma3.vision.embedding_length"] = vc.get("hidden_size", 1152)
        kv["gemma3.vision.feed_forward_length"] = vc.get("intermediate_size", 4304)
        kv["gemma3.vision.image_size"] = vc.get("image_size", 896)
        kv["gemma3.vision.patch_size"] = vc.get("patch_size", 14)
        kv["gemma3.vision.num_channels"] = vc.get("num_channels", 3)
        kv["gemma3.vision.attention.head_count"] = vc.get("num_attention_heads", 16)
        kv["gemma3.vision.attention.layer_norm_epsilon"] = float(vc.get("layer_norm_eps", 1e-6))
        kv["gemma3.mm.tokens_per_image"] = cfg.get("mm_tokens_per_image", 256)
    if arch == "phi3":          # convert/convert_phi3.go:41-71
        kv["phi3.rope.dimension_count"] = c["hidden_size"] // n_head
        orig = c.get("original_max_position_embeddings") or (c.get("rope_parameters") or {}).get("original_max_position_embeddings") or c.get("max_position_embeddings", 4096)
        kv["phi3.rope.scaling.original_context_length"] = orig
        if c.get("sliding_window"):
            kv["phi3.attention.sliding_window"] = c["sliding_window"]
        rs3 = c.get("rope_scaling") or c.get("rope_parameters") or {}
        kind = rs3.get("type") or rs3.get("rope_type") or ""
        scale = c.get("max_position_embeddings", orig) / orig
        if kind in ("su", "longrope"):
            kv["phi3.rope.scaling.attn_factor"] = float(max(math.sqrt(1 + math.log(scale) / math.log(orig)), 1.0)) if scale > 1 else 1.0
        elif kind == "yarn":
            kv["phi3.rope.scaling.attn_factor"] = float(max(0.1 * math.log(scale) + 1.0, 1.0))
        elif kind and kind != "default":
            raise ConvertError(f"unknown rope scaling type {kind!r}")
    rs = c.get("rope_scaling") or c.get("rope_parameters") or {}      # newer configs keep theta and scaling in one `rope_parameters` table
    rtype = rs.get("rope_type") or rs.get("type")
    if rtype in ("linear", "yarn"):
        kv[f"{arch}.rope.scaling.type"] = rtype
        kv[f"{arch}.rope.scaling.factor"] = float(rs.get("factor", 1.0))
        if rs.get("original_max_position_embeddings"):
            kv[f"{arch}.rope.scaling.original_context_length"] = rs["original_max_position_embeddings"]
        if rtype == "yarn":
            kv[f"{arch}.rope.scaling.yarn_beta_fast"] = float(rs.get("beta_fast", 32.0))
            kv[f"{arch}.rope.scaling.yarn_beta_slow"] = float(rs.get("beta_slow", 1.0))
    n_exp = c.get("num_local_experts") or c.get("num_experts") or 0
    if n_exp:
        kv[f"{arch}.expert_count"] = n_exp
        kv[f"{arch}.expert_used_count"] = c.get("num_experts_per_tok", 2)
        if c.get("moe_intermediate_size"):
            kv[f"{arch}.expert_feed_forward_length"] = c["moe_intermediate_size"]
        if "norm_topk_prob" in c:
            kv[f"{arch}.norm_top_k_prob"] = bool(c["norm_topk_prob"])
    if c.get("sliding_window") and arch in ("gemma2", "gemma3", "llama", "gpt-oss"):
        kv[f"{arch}.attention.sliding_window"] = c["sliding_window"]
    if arch == "gemma2":
        kv["gemma2.attn_logit_softcapping"] = float(c.get("attn_logit_softcapping") or 50.0)
        kv["gemma2.final_logit_softcapping"] = float(c.get("final_logit_softcapping") or 30.0)
    if arch == "gemma3" and c.get("rope_local_base_freq"):
        kv["gemma3.rope.local.freq_base"] = float(c["rope_local_base_freq"])
    if arch in ("gemma2", "gemma3") and c.get("query_pre_attn_scalar"):
        kv[f"{arch}.attention.query_pre_attn_scalar"] = c["query_pre_attn_scalar"]
    return kv


def rope_freq_factors(cfg: dict[str, Any]) -> torch.Tensor | None:
    """llama3-style rope scaling is baked into a ``rope_freqs.weight`` tensor of per-frequency divisors."""
    rs = cfg.get("rope_scaling") or cfg.get("rope_parameters") or {}
    if (rs.get("rope_type") or rs.get("type")) != "llama3":
        return None
    hd = cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]
    base = float(cfg.get("rope_theta") or rs.get("rope_theta") or 10000.0)
    factor, lo, hi = float(rs.get("factor", 8.0)), float(rs.get("low_freq_factor", 1.0)), float(rs.get("high_freq_factor", 4.0))
    orig = float(rs.get("original_max_position_embeddings", 8192))
    out = []
    for i in range(0, hd, 2):
        freq = base ** (-i / hd)
        wavelen = 2 * torch.pi / freq
        if wavelen < orig / hi:
            out.append(1.0)
        elif wavelen > orig / lo:
            out.append(factor)
        else:
            smooth = (orig / wavelen - lo) / (hi - lo)
            out.append(1.0 / ((1 - smooth) / factor + smooth))
    return torch.tensor(out, dtype=torch.float32)


# ---------------------------------------------------------------------------------------------------
# tokenizer
# ---------------------------------------------------------------------------------------------------
_PRE_BY_MARK = [("(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\\r\\n\\p{L}\\p{N}]?\\p{L}+|\\p{N}{1,3}", "llama-bpe"),
                ("(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\\r\\n\\p{L}\\p{N}]?\\p{L}+|\\p{N}|", "qwen2")]


def _pretokenizer(tj: dict[str, Any]) -> str:
    pats: list[str] = []

    def walk(node):
        if isinstance(node, dict):
            if node.get("type") == "Split" and isinstance(node.get("pattern"), dict):
                pats.append(node["pattern"].get("Regex", ""))
            for v in node.values():
                walk(v)
        elif isinstance(node, list):
            for v in node:
                walk(v)

    walk(tj.get("pre_tokenizer"))
    joined = "".join(pats)
    for mark, name in _PRE_BY_MARK:
        if mark in joined:
            return name
    return "default"


_SPM_FORCED_CONTROL = ("<end_of_turn>", "<start_of_turn>", "<start_function_declaration>", "<end_function_declaration>",
                       "<start_function_call>", "<end_function_call>", "<start_function_response>", "<end_function_response>", "<escape>")


def _spm_vocabulary(path: str, vocab_size: int) -> dict[str, Any]:
    """Vocabulary of a SentencePiece ``tokenizer.model`` (convert/tokenizer_spm.go:18-100): pieces with their scores;
    unknown / control / unused / byte pieces keep their type, everything else is normal except the additional special
    tokens of ``special_tokens_map.json`` (and a fixed list of gemma markers), which become control tokens;
    ``added_tokens.json`` appends user-defined tokens with score -1000."""
    try:
        import sentencepiece as spm
    except ImportError:
        raise ConvertError("tokenizer.model needs the sentencepiece package") from None
    sp = spm.SentencePieceProcessor(model_file=os.path.join(path, "tokenizer.model"))
    extra: set[str] = set(_SPM_FORCED_CONTROL)
    stm = os.path.join(path, "special_tokens_map.json")
    if os.path.exists(stm):
        with open(stm, encoding="utf-8") as f:
            for t in json.load(f).get("additional_special_tokens") or []:
                extra.add(t if isinstance(t, str) else t.get("content", ""))
    tokens, scores, types = [], [], []
    for i in range(sp.get_piece_size()):
        piece = sp.id_to_piece(i)
        tokens.append(piece)
        scores.append(float(sp.get_score(i)))
        if sp.is_unknown(i):
            types.append(2)
        elif sp.is_control(i):
            types.append(3)
        elif sp.is_unused(i):
            types.append(5)
        elif sp.is_byte(i):
            types.append(6)
        else:
            types.append(3 if piece in extra else 1)
    at = os.path.join(path, "added_tokens.json")
    if os.path.exists(at):
        with open(at, encoding="utf-8") as f:
            added = sorted(((i, t) for t, i in json.load(f).items()))
        for i, t in added:
            if i < len(tokens):
                if tokens[i] != t:
                    raise ConvertError(f"token mismatch: {t} != {tokens[i]} at pos [{i}]")
                continue
            if i != len(tokens):
                raise ConvertError(f"invalid token id: [{i}] as pos [{len(tokens)}]")
            tokens.append(t)
            scores.append(-1000.0)
            types.append(4)
    for i in range(len(tokens), vocab_size):          # the embedding matrix may be padded beyond the vocabulary
        tokens.append(f"[PAD{i}]")
        scores.append(-1000.0)
        types.append(5)
    out = {"tokenizer.ggml.model": "llama", "tokenizer.ggml.tokens": tokens, "tokenizer.ggml.scores": scores,
           "tokenizer.ggml.token_type": types}
    for key, i in (("bos", sp.bos_id()), ("eos", sp.eos_id()), ("unknown", sp.unk_id()), ("padding", sp.pad_id())):
        if i >= 0:
            out[f"tokenizer.ggml.{key}_token_id"] = int(i)
    return out


def tokenizer_kv(path: str, vocab_size: int) -> dict[str, Any]:
    kv: dict[str, Any] = {}
    tj_path = os.path.join(path, "tokenizer.json")
    tc: dict[str, Any] = {}
    if os.path.exists(os.path.join(path, "tokenizer_config.json")):
        with open(os.path.join(path, "tokenizer_config.json"), encoding="utf-8") as f:
            tc = json.load(f)
    if os.path.exists(tj_path):
        with open(tj_path, encoding="utf-8") as f:
            tj = json.load(f)
        model = tj.get("model", {})
        vocab: dict[str, int] = dict(model.get("vocab", {}))
        special = set()
        for a in tj.get("added_tokens", []):
            vocab[a["content"]] = a["id"]
            if a.get("special"):
                special.add(a["id"])
        n = max(max(vocab.values()) + 1 if vocab else 0, vocab_size)
        tokens = [f"[PAD{i}]" for i in range(n)]
        types = [5] * n                      # unused
        for tok, i in vocab.items():
            tokens[i] = tok
            types[i] = 3 if i in special else 1
        if model.get("type") == "BPE" and not model.get("byte_fallback"):
            kv["tokenizer.ggml.model"] = "gpt2"
            kv["tokenizer.ggml.pre"] = _pretokenizer(tj)
            merges = model.get("merges", [])
            kv["tokenizer.ggml.merges"] = [m if isinstance(m, str) else " ".join(m) for m in merges]
        else:                                # SentencePiece-style vocabulary expressed in tokenizer.json (byte fallback, "▁" spaces)
            kv["tokenizer.ggml.model"] = "llama"
            kv["tokenizer.ggml.scores"] = [0.0 if types[i] == 3 else -float(i) for i in range(n)]
            for i, t in enumerate(tokens):
                if re.fullmatch(r"<0x[0-9A-F]{2}>", t):
                    types[i] = 6
            kv["tokenizer.ggml.add_space_prefix"] = not any(isinstance(nz, dict) and nz.get("type") == "Replace"
                                                            for nz in [tj.get("normalizer") or {}])
        kv["tokenizer.ggml.tokens"] = tokens
        kv["tokenizer.ggml.token_type"] = types
    elif os.path.exists(os.path.join(path, "tokenizer.model")):
        kv.update(_spm_vocabulary(path, vocab_size))
        vocab = {t: i for i, t in enumerate(kv["tokenizer.ggml.tokens"])}
    else:
        raise ConvertError("neither tokenizer.json nor tokenizer.model found")

    def tok_id(key: str) -> int | None:
        v = tc.get(key)
        if isinstance(v, dict):
            v = v.get("content")
        return vocab.get(v) if isinstance(v, str) else None

    for key, out in (("bos_token", "bos_token_id"), ("eos_token", "eos_token_id"), ("unk_token", "unknown_token_id"), ("pad_token", "padding_token_id")):
        i = tok_id(key)
        if i is not None:
            kv[f"tokenizer.ggml.{out}"] = i
    gen_path = os.path.join(path, "generation_config.json")
    if os.path.exists(gen_path):
        with open(gen_path, encoding="utf-8") as f:
            gc = json.load(f)
        eos = gc.get("eos_token_id")
        if isinstance(eos, list) and eos:
            kv["tokenizer.ggml.eos_token_ids"] = [int(e) for e in eos]
            kv.setdefault("tokenizer.ggml.eos_token_id", int(eos[0]))
        elif isinstance(eos, int):
            kv.setdefault("tokenizer.ggml.eos_token_id", eos)
        if isinstance(gc.get("bos_token_id"), int):
            kv.setdefault("tokenizer.ggml.bos_token_id", gc["bos_token_id"])
    if "add_bos_token" in tc:
        kv["tokenizer.ggml.add_bos_token"] = bool(tc["add_bos_token"])
    if "add_eos_token" in tc:
        kv["tokenizer.ggml.add_eos_token"] = bool(tc["add_eos_token"])
    if isinstance(tc.get("chat_template"), str):
        kv["tokenizer.chat_template"] = tc["chat_template"]
    return kv


# ---------------------------------------------------------------------------------------------------
# conversion
# ---------------------------------------------------------------------------------------------------
def _encode(t: torch.Tensor, name: str, outtype: str) -> tuple[GGMLType, torch.Tensor]:
    if t.dim() < 2 or name.endswith(("_norm.weight", ".bias")) or "ffn_gate_inp" in name or "attn_sinks" in name:
        return GGMLType.F32, quants.quantize(t.float(), GGMLType.F32)
    want = {"f32": GGMLType.F32, "f16": GGMLType.F16, "bf16": GGMLType.BF16}.get(outtype)
    if want is None:
        want = GGMLType.BF16 if t.dtype == torch.bfloat16 else GGMLType.F16 if t.dtype == torch.float16 else GGMLType.F32
    return want, quants.quantize(t.float(), want)


def mxfp4_blocks(blocks: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """Packed experts of a gpt-oss checkpoint -> GGML MXFP4 blocks (uint8 [..., in / 32, 17]).

    The checkpoint keeps consecutive elements in the two nibbles of a byte (element 2i low, 2i + 1 high); a GGML block
    keeps elements 0..15 in the low and 16..31 in the high nibbles, preceded by the e8m0 scale byte
    (convert/convert_gptoss.go:215-262).
    """
    if blocks.shape[-1] != 16 or blocks.shape[:-1] != scales.shape:
        raise ConvertError(f"MXFP4 blocks {tuple(blocks.shape)} do not match scales {tuple(scales.shape)}")
    blocks, scales = blocks.to(torch.uint8), scales.to(torch.uint8)
    a, b = blocks[..., :8], blocks[..., 8:]
    even = (a & 0x0F) | ((b & 0x0F) << 4)          # elements 2j and 16 + 2j
    odd = (a >> 4) | (b & 0xF0)                    # elements 2j + 1 and 17 + 2j
    nib = torch.stack([even, odd], -1).reshape(*blocks.shape[:-1], 16)
    return torch.cat([scales.unsqueeze(-1), nib], -1).contiguous()


def convert_tensors(src: ModelDir, cfg: dict[str, Any], arch: str, outtype: str = "auto",
                    progress: Callable[[str], None] | None = None) -> Iterator[WriteTensor]:
    c = cfg.get("text_config", cfg) if arch == "gemma3" else cfg
    n_head, n_kv = c["num_attention_heads"], c.get("num_key_value_heads", c["num_attention_heads"])
    experts: dict[str, dict[int, str]] = {}
    names: dict[str, str] = {}
    vision: dict[str, str] = {}
    keep_vision = arch == "gemma3" and isinstance(cfg.get("vision_config"), dict)
    for name in src.keys():
        if _SKIP.fullmatch(name):
            v_out = map_vision_name(name) if keep_vision else None
            if v_out is not None:
                vision[v_out] = name
            continue
        out = map_name(name, arch)
        if out is None:
            raise ConvertError(f"tensor {name} has no GGUF counterpart for architecture {arch}")
        if "#" in out:
            base, e = out.split("#")
            experts.setdefault(base, {})[int(e)] = name
        else:
            names[out] = name
    tied = "output.weight" not in names

    def emit(out: str, t: torch.Tensor) -> WriteTensor:
        if progress:
            progress(out)
        if arch == "llama" and re.fullmatch(r"blk\.\d+\.attn_[qk]\.(weight|bias)", out):
            t = permute_qk(t, n_head if ".attn_q." in out else n_kv)
        if arch in ("gemma", "gemma2", "gemma3") and out.endswith("_norm.weight"):
            t = t.float() + 1.0              # the checkpoint stores w - 1
        dt, raw = _encode(t, out, outtype)
        return WriteTensor(out, tuple(reversed(t.shape)), dt, raw.cpu().numpy())

    def emit_mxfp4(out: str, raw: torch.Tensor) -> WriteTensor:
        if progress:
            progress(out)
        e, rows, nb, _ = raw.shape
        return WriteTensor(out, (nb * 32, rows, e), GGMLType.MXFP4, raw.reshape(-1).cpu().numpy())

    for out in sorted(names, key=_order):
        if out == "output.weight" and tied:
            continue
        if out.endswith(".scales"):
            continue                                   # consumed together with the blocks
        if out.endswith(".blocks"):
            base = out[:-len(".blocks")]
            if base + ".scales" not in names:
                raise ConvertError(f"{names[out]} has no scales tensor")
            raw = mxfp4_blocks(src.tensor(names[out]), src.tensor(names[base + ".scales"]))
            if "gate_up" in base:                      # even rows gate, odd rows up
                yield emit_mxfp4(base.replace("gate_up", "gate") + ".weight", raw[:, 0::2].contiguous())
                yield emit_mxfp4(base.replace("gate_up", "up") + ".weight", raw[:, 1::2].contiguous())
            else:
                yield emit_mxfp4(base + ".weight", raw)
            continue
        t = src.tensor(names[out])
        if out.endswith("@T"):                         # stored [expert, in, out]
            yield emit(out[:-2], t.transpose(1, 2).contiguous())
        elif ".ffn_gate_up_exps." in out:              # even columns gate, odd columns up
            if out.endswith(".weight"):
                yield emit(out.replace("gate_up", "gate"), t[..., 0::2].transpose(1, 2).contiguous())
                yield emit(out.replace("gate_up", "up"), t[..., 1::2].transpose(1, 2).contiguous())
            else:
                yield emit(out.replace("gate_up", "gate"), t[..., 0::2].contiguous())
                yield emit(out.replace("gate_up", "up"), t[..., 1::2].contiguous())
        else:
            yield emit(out, t)
    for base in sorted(experts, key=_order):
        idx = experts[base]
        if sorted(idx) != list(range(len(idx))):
            raise ConvertError(f"{base}: expert indices are not contiguous")
        yield emit(base, torch.stack([src.tensor(idx[e]) for e in range(len(idx))]))
    for out in sorted(vision):       # the image tower rides along in the same file; matrices keep 16 bits, the rest fp32
        t = src.tensor(vision[out])
        if out == "v.patch_embedding.weight":
            t = t.reshape(t.shape[0], -1)                       # [width, channels * patch * patch]
        if out == "mm.mm_soft_emb_norm.weight":
            t = t.float() + 1.0                                 # stored as w - 1 like the text model's norms
        if progress:
            progress(out)
        small = t.dim() < 2 or out in ("v.position_embedding.weight", "v.patch_embedding.weight")
        dt, raw = _encode(t.float() if small else t, out, "f32" if small else ("f16" if outtype == "auto" else outtype))
        yield WriteTensor(out, tuple(reversed(t.shape)), dt, raw.cpu().numpy())
    if arch == "phi3":          # per-frequency divisors for contexts beyond / within the original window (convert/convert_phi3.go:73-101)
        rs3 = c.get("rope_scaling") or c.get("rope_parameters") or {}
        for key, out_name in (("long_factor", "rope_factors_long.weight"), ("short_factor", "rope_factors_short.weight")):
            if rs3.get(key):
                yield emit(out_name, torch.tensor(rs3[key], dtype=torch.float32))
    ff = rope_freq_factors(c)
    if ff is not None:
        yield emit("rope_freqs.weight", ff)


def _order(name: str) -> tuple:
    m = re.match(r"blk\.(\d+)\.(.*)", name)
    return (1, int(m.group(1)), m.group(2)) if m else (0, 0, name)


def convert_hf(path: str, out_path: str, outtype: str = "auto", progress: Callable[[str], None] | None = None) -> dict[str, Any]:
    """Convert the checkpoint directory ``path`` into the GGUF file ``out_path``; returns the metadata written."""
    with open(os.path.join(path, "config.json"), encoding="utf-8") as f:
        cfg = json.load(f)
    archs = cfg.get("architectures") or []
    if not archs or archs[0] not in ARCHS:
        raise ConvertError(f"unsupported architecture {archs[0] if archs else '(none)'}")
    arch = ARCHS[archs[0]]
    src = ModelDir(path)
    try:
        kv = _kv(cfg, arch, os.path.basename(os.path.normpath(path)))
        kv.update(tokenizer_kv(path, kv.get(f"{arch}.vocab_size", 0)))
        tensors = list(convert_tensors(src, cfg, arch, outtype, progress))
        types = {t.dtype for t in tensors if len(t.shape) >= 2}
        kv["general.file_type"] = 32 if GGMLType.BF16 in types else 1 if GGMLType.F16 in types else 0
        write_gguf(out_path, kv, tensors)
    finally:
        src.close()
    return kv


_LORA_NAME = re.compile(r"(?:base_model\.model\.)?(.+)\.lora_([AB])(?:\.default)?\.weight")


def convert_adapter(path: str, out_path: str, arch: str, n_head: int = 0, n_kv_head: int = 0) -> dict[str, Any]:
    """PEFT LoRA adapter directory (adapter_config.json + adapter_model.safetensors) -> adapter GGUF for a base model of
    architecture ``arch`` (convert/convert.go:182-238, convert_llama_adapter.go): tensors ``<base name>.lora_a`` [r, in]
    and ``<base name>.lora_b`` [out, r], ``adapter.lora.alpha`` from the configuration.  For llama-arch bases the rows of
    the B factor of Q and K projections get the same rotary re-ordering as the base matrices (``n_head`` / ``n_kv_head``
    of the base model are needed for that)."""
    with open(os.path.join(path, "adapter_config.json"), encoding="utf-8") as f:
        ac = json.load(f)
    if str(ac.get("peft_type", "LORA")).upper() != "LORA":
        raise ConvertError(f"unsupported adapter type {ac.get('peft_type')!r}")
    src = ModelDir(path)
    tensors: list[WriteTensor] = []
    try:
        for name in sorted(src.keys()):
            m = _LORA_NAME.fullmatch(name)
            if m is None:
                continue
            base = map_name(m.group(1) + ".weight", arch)
            if base is None or "#" in base or "@" in base:
                raise ConvertError(f"adapter tensor {name} has no GGUF counterpart for architecture {arch}")
            t = src.tensor(name).float()
            if m.group(2) == "B" and arch == "llama" and re.fullmatch(r"blk\.\d+\.attn_[qk]\.weight", base):
                heads = n_head if ".attn_q." in base else n_kv_head
                if heads <= 0:
                    raise ConvertError("the head counts of the base model are needed to convert Q/K adapters of a llama-arch model")
                t = permute_qk(t, heads)
            out = f"{base}.lora_{m.group(2).lower()}"
            tensors.append(WriteTensor(out, tuple(reversed(t.shape)), GGMLType.F32, quants.quantize(t, GGMLType.F32).numpy()))
        if not tensors:
            raise ConvertError("no LoRA tensors found in the adapter")
        kv = {"general.architecture": arch, "general.type": "adapter", "adapter.type": "lora",
              "adapter.lora.alpha": float(ac.get("lora_alpha", ac.get("alpha", 0.0)))}
        write_gguf(out_path, kv, tensors)
    finally:
        src.close()
    return kv


def is_hf_dir_listing(names: list[str]) -> bool:
    return "config.json" in names and any(n.endswith(".safetensors") for n in names)
