"""Random-init checkpoints of the benchmark architectures.

Nothing can be downloaded where the benchmarks run, so weights are drawn from N(0, 0.02) with a
fixed seed and encoded with this package's own quantisers.  The per-tensor type mixture of a
``Q4_K_M`` file follows the rule the upstream quantiser applies (Q6_K for ``output.weight`` and for
``attn_v`` / ``ffn_down`` on the "more bits" layers, Q4_K elsewhere, F32 for 1-D tensors and the MoE
router), which is what ``general.file_type = 15`` means in practice (fs/ggml/type.go:28,70-71).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Iterator

import torch

from ..gguf import quants
from ..gguf.types import FileType, GGMLType
from ..gguf.writer import WriteTensor, write_gguf


@dataclass
class ArchSpec:
    arch: str
    n_layers: int
    d_model: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    d_ff: int
    vocab: int
    rope_base: float = 10000.0
    eps: float = 1e-5
    ctx_train: int = 131072
    tied: bool = False
    n_experts: int = 0
    n_experts_used: int = 0
    d_ff_expert: int = 0
    sliding_window: int = 0
    extra_kv: dict = field(default_factory=dict)


SPECS: dict[str, ArchSpec] = {
    "tiny-llama": ArchSpec("llama", 2, 256, 4, 2, 64, 688, 32000, 10000.0, 1e-5, 2048),
    "llama-3.1-8b": ArchSpec("llama", 32, 4096, 32, 8, 128, 14336, 128256, 500000.0),
    "llama-3.1-70b": ArchSpec("llama", 80, 8192, 64, 8, 128, 28672, 128256, 500000.0),
    "qwen3-235b-a22b": ArchSpec("qwen3moe", 94, 4096, 64, 4, 128, 12288, 151936, 1e6, 1e-6, 40960,
                                n_experts=128, n_experts_used=8, d_ff_expert=1536),
    "gpt-oss-120b": ArchSpec("gpt-oss", 36, 2880, 64, 8, 64, 2880, 201088, 150000.0, 1e-5, 131072,
                             n_experts=128, n_experts_used=4, d_ff_expert=2880, sliding_window=128,
                             extra_kv={"rope.scaling.type": "yarn", "rope.scaling.factor": 32.0,
                                       "rope.scaling.original_context_length": 4096,
                                       "rope.scaling.yarn_beta_fast": 32.0, "rope.scaling.yarn_beta_slow": 1.0}),
    # small stand-ins of every family for tests
    "tiny-tp": ArchSpec("llama", 2, 1024, 16, 8, 64, 4096, 4096, 500000.0, 1e-5, 4096),      # divides 2, 4 and 8 ways
    "tiny-qwen3": ArchSpec("qwen3", 2, 256, 4, 2, 64, 768, 4096, 1e6, 1e-6, 4096),
    "tiny-qwen2": ArchSpec("qwen2", 2, 256, 4, 2, 64, 768, 4096, 1e6, 1e-6, 4096),
    "tiny-qwen3moe": ArchSpec("qwen3moe", 2, 256, 4, 2, 64, 768, 4096, 1e6, 1e-6, 4096, n_experts=8, n_experts_used=2, d_ff_expert=256),
    "tiny-gemma3": ArchSpec("gemma3", 6, 256, 4, 2, 64, 768, 4096, 1e6, 1e-6, 4096, tied=True, sliding_window=16),
    "tiny-gemma2": ArchSpec("gemma2", 2, 256, 4, 2, 64, 768, 4096, 10000.0, 1e-6, 4096, tied=True, sliding_window=16),
    "tiny-gpt-oss": ArchSpec("gpt-oss", 2, 256, 8, 2, 32, 256, 4096, 150000.0, 1e-5, 4096, n_experts=8, n_experts_used=2,
                             d_ff_expert=256, sliding_window=8,
                             extra_kv={"rope.scaling.type": "yarn", "rope.scaling.factor": 4.0,
                                       "rope.scaling.original_context_length": 64}),
    "tiny-mixtral": ArchSpec("llama", 2, 256, 4, 2, 64, 512, 4096, 10000.0, 1e-5, 4096, n_experts=4, n_experts_used=2, d_ff_expert=512),
}


def use_more_bits(i: int, n: int) -> bool:
    return i < n // 8 or i >= 7 * n // 8 or (i - n // 8) % 3 == 2


def tensor_type(name: str, shape: tuple[int, ...], file_type: int, layer: int, n_layers: int, spec: ArchSpec) -> GGMLType:
    """Encoding of one tensor inside a file of ``file_type``."""
    ft = FileType(file_type)
    if len(shape) == 1 or name.endswith(".bias") or "ffn_gate_inp" in name or name.endswith("_norm.weight") or "attn_sinks" in name:
        return GGMLType.F32
    if ft == FileType.F32:
        return GGMLType.F32
    if ft == FileType.F16:
        return GGMLType.F16
    if ft == FileType.BF16:
        return GGMLType.BF16
    base = {FileType.Q8_0: GGMLType.Q8_0, FileType.Q4_0: GGMLType.Q4_0, FileType.Q4_K_M: GGMLType.Q4_K,
            FileType.Q4_K_S: GGMLType.Q4_K, FileType.Q6_K: GGMLType.Q6_K, FileType.Q5_K_M: GGMLType.Q5_K,
            FileType.MXFP4_MOE: GGMLType.MXFP4}[ft]
    if ft == FileType.MXFP4_MOE:
        # gpt-oss layout: MXFP4 experts, bf16 attention / embeddings / output
        return GGMLType.MXFP4 if "_exps" in name else GGMLType.BF16
    k = shape[-1]
    t = base
    if ft in (FileType.Q4_K_M, FileType.Q4_K_S, FileType.Q5_K_M):
        if name == "output.weight" or (name == "token_embd.weight" and spec.tied):
            t = GGMLType.Q6_K
        elif ft != FileType.Q4_K_S and ("attn_v.weight" in name or "ffn_down" in name) and use_more_bits(layer, n_layers):
            t = GGMLType.Q6_K
        elif "attn_v.weight" in name and spec.n_layers == 80 and t == GGMLType.Q4_K:
            t = GGMLType.Q5_K     # the 70B rule: eight query heads share each V head, so it gets 5 bits
    if k % quants.block_size(t):
        t = GGMLType.Q8_0 if k % 32 == 0 else GGMLType.F16   # rows that do not fit a 256-block fall back
    return t


def tensor_table(spec: ArchSpec) -> list[tuple[str, tuple[int, ...], int]]:
    """(name, row-major shape, layer index or -1) for every tensor of the architecture."""
    s = spec
    q_dim, kv_dim = s.n_heads * s.head_dim, s.n_kv_heads * s.head_dim
    out: list[tuple[str, tuple[int, ...], int]] = [("token_embd.weight", (s.vocab, s.d_model), -1)]
    for i in range(s.n_layers):
        p = f"blk.{i}."
        out += [(p + "attn_norm.weight", (s.d_model,), i), (p + "attn_q.weight", (q_dim, s.d_model), i),
                (p + "attn_k.weight", (kv_dim, s.d_model), i), (p + "attn_v.weight", (kv_dim, s.d_model), i),
                (p + "attn_output.weight", (s.d_model, q_dim), i)]
        if s.arch in ("qwen2", "gpt-oss"):
            out += [(p + "attn_q.bias", (q_dim,), i), (p + "attn_k.bias", (kv_dim,), i), (p + "attn_v.bias", (kv_dim,), i)]
        if s.arch == "gpt-oss":
            out += [(p + "attn_output.bias", (s.d_model,), i), (p + "attn_sinks.weight", (s.n_heads,), i),
                    (p + "post_attention_norm.weight", (s.d_model,), i)]
        else:
            out += [(p + "ffn_norm.weight", (s.d_model,), i)]
        if s.arch in ("qwen3", "qwen3moe", "gemma3"):
            out += [(p + "attn_q_norm.weight", (s.head_dim,), i), (p + "attn_k_norm.weight", (s.head_dim,), i)]
        if s.arch in ("gemma2", "gemma3"):
            out += [(p + "post_attention_norm.weight", (s.d_model,), i), (p + "post_ffw_norm.weight", (s.d_model,), i)]
        if s.n_experts:
            fe = s.d_ff_expert
            out += [(p + "ffn_gate_inp.weight", (s.n_experts, s.d_model), i),
                    (p + "ffn_gate_exps.weight", (s.n_experts, fe, s.d_model), i),
                    (p + "ffn_up_exps.weight", (s.n_experts, fe, s.d_model), i),
                    (p + "ffn_down_exps.weight", (s.n_experts, s.d_model, fe), i)]
            if s.arch == "gpt-oss":
                out += [(p + "ffn_gate_inp.bias", (s.n_experts,), i), (p + "ffn_gate_exps.bias", (s.n_experts, fe), i),
                        (p + "ffn_up_exps.bias", (s.n_experts, fe), i), (p + "ffn_down_exps.bias", (s.n_experts, s.d_model), i)]
        else:
            out += [(p + "ffn_gate.weight", (s.d_ff, s.d_model), i), (p + "ffn_up.weight", (s.d_ff, s.d_model), i),
                    (p + "ffn_down.weight", (s.d_model, s.d_ff), i)]
    out.append(("output_norm.weight", (s.d_model,), -1))
    if not s.tied:
        out.append(("output.weight", (s.vocab, s.d_model), -1))
    return out


def metadata(spec: ArchSpec, file_type: int, name: str = "", with_tokenizer: bool = True) -> dict:
    s = spec
    kv: dict = {
        "general.architecture": s.arch, "general.name": name or s.arch, "general.file_type": int(file_type),
        "block_count": s.n_layers, "context_length": s.ctx_train, "embedding_length": s.d_model,
        "feed_forward_length": s.d_ff, "attention.head_count": s.n_heads, "attention.head_count_kv": s.n_kv_heads,
        "attention.key_length": s.head_dim, "attention.value_length": s.head_dim,
        "attention.layer_norm_rms_epsilon": float(s.eps), "rope.freq_base": float(s.rope_base),
        "rope.dimension_count": s.head_dim, "vocab_size": s.vocab,
    }
    if s.n_experts:
        kv.update({"expert_count": s.n_experts, "expert_used_count": s.n_experts_used, "expert_feed_forward_length": s.d_ff_expert})
    if s.sliding_window:
        kv["attention.sliding_window"] = s.sliding_window
    if s.arch == "gemma3":
        kv["rope.local.freq_base"] = 10000.0
    kv.update(s.extra_kv)
    if with_tokenizer:
        kv.update(synthetic_tokenizer_kv(s.vocab))
    return kv


def synthetic_tokenizer_kv(vocab: int) -> dict:
    """A vocabulary in which every id has a unique surface form ``<t{id}>`` that tokenises back to itself.

    Ids 0..2 are <unk>, <s>, </s>; ids 3..258 are the byte-fallback tokens ``<0xHH>`` so arbitrary text is
    representable; the rest are user-defined tokens (matched verbatim before the piece tokeniser runs).
    """
    toks, types, scores = [], [], []
    for i in range(vocab):
        if i == 0:
            toks.append("<unk>"); types.append(2)
        elif i == 1:
            toks.append("<s>"); types.append(3)
        elif i == 2:
            toks.append("</s>"); types.append(3)
        elif i < 259:
            toks.append(f"<0x{i - 3:02X}>"); types.append(6)
        else:
            toks.append(f"<t{i}>"); types.append(4)
        scores.append(0.0)
    return {
        "tokenizer.ggml.model": "llama", "tokenizer.ggml.tokens": toks, "tokenizer.ggml.token_type": types,
        "tokenizer.ggml.scores": scores, "tokenizer.ggml.bos_token_id": 1, "tokenizer.ggml.eos_token_id": 2,
        "tokenizer.ggml.unknown_token_id": 0, "tokenizer.ggml.add_bos_token": False, "tokenizer.ggml.add_eos_token": False,
        "tokenizer.ggml.add_space_prefix": False,
    }


def random_tensor(name: str, shape: tuple[int, ...], seed: int, device="cpu", std: float = 0.02) -> torch.Tensor:
    """Deterministic N(0, std) values for ``name`` (norm weights are 1 + noise, sinks/biases small)."""
    h = 0
    for ch in name:
        h = (h * 131 + ord(ch)) & 0x7FFFFFFF
    gen = torch.Generator(device=device)
    gen.manual_seed((seed * 1000003 + h) & 0x7FFFFFFFFFFF)
    n = math.prod(shape)
    x = torch.randn(n, generator=gen, device=device, dtype=torch.float32).mul_(std).view(*shape)
    if name.endswith("_norm.weight"):
        x = x + 1.0
    return x


def iter_tensors(spec: ArchSpec, file_type: int, seed: int = 0, device="cpu",
                 select: Callable[[str], bool] | None = None) -> Iterator[tuple[str, tuple[int, ...], GGMLType, torch.Tensor]]:
    """Yield (name, shape, type, encoded bytes) one tensor at a time."""
    for name, shape, layer in tensor_table(spec):
        if select is not None and not select(name):
            continue
        t = tensor_type(name, shape, file_type, max(layer, 0), spec.n_layers, spec)
        x = random_tensor(name, shape, seed, device)
        yield name, shape, t, quants.quantize(x, t)


def write_synthetic_gguf(path: str, spec_name: str, file_type: str | int = "F32", seed: int = 0, device="cpu",
                         template: str | None = None) -> None:
    spec = SPECS[spec_name]
    ft = file_type if isinstance(file_type, int) else int(getattr(FileType, file_type if file_type != "MXFP4" else "MXFP4_MOE"))
    kv = metadata(spec, ft, spec_name)
    if template:
        kv["tokenizer.chat_template"] = template
    tensors = []
    for name, shape, t, raw in iter_tensors(spec, ft, seed, device):
        tensors.append(WriteTensor(name, tuple(reversed(shape)), t, raw.cpu().numpy()))
    write_gguf(path, kv, tensors)


class SyntheticTensors:
    """Mapping-like source of :class:`QWeight` that draws and encodes each tensor when it is asked for.

    ``rows`` optionally restricts a tensor to a row range (tensor-parallel shards are generated
    directly, the full matrix is never materialised on one device).
    """

    def __init__(self, spec_name: str, file_type: str | int = "Q4_K_M", seed: int = 0, device="cpu"):
        from .weights import QWeight
        self._QWeight = QWeight
        self.spec = SPECS[spec_name]
        self.ft = file_type if isinstance(file_type, int) else int(getattr(FileType, file_type if file_type != "MXFP4" else "MXFP4_MOE"))
        self.seed, self.device = seed, device
        self.table = {n: (shape, layer) for n, shape, layer in tensor_table(self.spec)}

    def __contains__(self, name: str) -> bool:
        return name in self.table

    def keys(self):
        return self.table.keys()

    def type_of(self, name: str) -> GGMLType:
        shape, layer = self.table[name]
        return tensor_type(name, shape, self.ft, max(layer, 0), self.spec.n_layers, self.spec)

    def __getitem__(self, name: str):
        shape, layer = self.table[name]
        t = self.type_of(name)
        x = random_tensor(name, shape, self.seed, self.device)
        return self._QWeight(name, t, tuple(shape), quants.quantize(x, t))


def synthetic_header(spec_name: str, file_type: str | int = "Q4_K_M", with_tokenizer: bool = False):
    """A data-less :class:`GGUFFile` carrying the metadata of a synthetic checkpoint (for config parsing)."""
    from ..gguf.reader import GGUFFile, TensorInfo
    spec = SPECS[spec_name]
    ft = file_type if isinstance(file_type, int) else int(getattr(FileType, file_type if file_type != "MXFP4" else "MXFP4_MOE"))
    raw = metadata(spec, ft, spec_name, with_tokenizer=with_tokenizer)
    kv = {}
    for k, v in raw.items():
        kv[k if k.startswith(("general.", "tokenizer.")) else f"{spec.arch}.{k}"] = v
    tensors = {n: TensorInfo(n, tuple(reversed(shape)), tensor_type(n, shape, ft, max(layer, 0), spec.n_layers, spec), 0, 0)
               for n, shape, layer in tensor_table(spec)}
    return GGUFFile("", 3, "<", kv, {}, tensors, 0, 32)
