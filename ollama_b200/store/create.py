"""Model creation: ``FROM`` an existing model or GGUF blobs, optional re-quantisation, text layers, manifest.

Flow of the reference ``/api/create`` (server/create.go:51-356): resolve the base (model name or
uploaded files by digest), optionally quantise (the reference shells out to an external tool,
server/quantization.go:36-170; here tensors are re-encoded with this package's codecs), then write
template / system / params / messages / license layers (server/create.go:1313-1424), the config
blob and the manifest.
"""
from __future__ import annotations

import json
import os
import tempfile
from typing import Any, Callable, Iterator

import torch

from ..gguf import quants
from ..gguf.reader import open_gguf
from ..gguf.types import QUANTIZE_TARGETS, FileType, GGMLType, file_type_name, parse_file_type
from ..gguf.writer import WriteTensor, write_gguf
from . import manifest as M
from .model import ModelNotFound, get_model
from .names import parse_name


class CreateError(Exception):
    def __init__(self, msg: str, status: int = 400):
        super().__init__(msg)
        self.status = status


def _detect_template(layers) -> tuple[str, tuple[str, ...]]:
    """(Go template, stop strings) for the model layer's ``tokenizer.chat_template`` when it is a named layout, else ("", ())."""
    from ..gguf.reader import open_gguf
    from ..text import named
    for l in layers:
        if l.media_type != M.MT_MODEL:
            continue
        try:
            g = open_gguf(l.path())
        except Exception:
            return "", ()
        try:
            jinja = g.kv.get("tokenizer.chat_template")
        finally:
            g.close()
        layout = named.detect(jinja) if isinstance(jinja, str) else None
        if layout is not None:
            return named.gotemplate(layout), layout.stop
    return "", ()


def _param_size(n: int) -> str:
    from ..utils.format import human_number
    return human_number(n)


def gguf_config(path: str) -> dict[str, Any]:
    g = open_gguf(path, max_array=0, metadata_only=True)
    try:
        n_params = sum(t.n_elements for t in g.tensors.values())
        arch = g.architecture
        return {"model_format": "gguf", "model_family": arch, "model_families": [arch], "model_type": _param_size(n_params),
                "file_type": file_type_name(int(g.kv.get("general.file_type", 0))), "architecture": "amd64", "os": "linux"}
    finally:
        g.close()


def target_tensor_type(name: str, shape: tuple[int, ...], cur: GGMLType, ft: FileType, layer: int, n_layers: int, tied: bool) -> GGMLType:
    """Per-tensor encoding inside a file of type ``ft`` (same rule the synthetic generator uses)."""
    from ..models.synth import use_more_bits
    if len(shape) == 1 or "ffn_gate_inp" in name or "_norm." in name or name.startswith(("v.", "mm.", "a.")) or "rope_freqs" in name \
            or "attn_sinks" in name or name.endswith(".bias"):
        return cur if cur in (GGMLType.F32, GGMLType.F16, GGMLType.BF16) else GGMLType.F32
    if ft in (FileType.F32, FileType.F16, FileType.BF16):
        return {FileType.F32: GGMLType.F32, FileType.F16: GGMLType.F16, FileType.BF16: GGMLType.BF16}[ft]
    t = {FileType.Q8_0: GGMLType.Q8_0, FileType.Q4_K_S: GGMLType.Q4_K, FileType.Q4_K_M: GGMLType.Q4_K}[ft]
    if ft in (FileType.Q4_K_S, FileType.Q4_K_M):
        if name == "output.weight" or (name == "token_embd.weight" and tied):
            t = GGMLType.Q6_K
        elif ft == FileType.Q4_K_M and ("attn_v.weight" in name or "ffn_down" in name) and use_more_bits(layer, n_layers):
            t = GGMLType.Q6_K
    k = shape[-1]
    if k % quants.block_size(t):
        t = GGMLType.Q8_0 if k % 32 == 0 else GGMLType.F16
    return t


def quantize_gguf(src: str, dst: str, target: str, progress: Callable[[str], None] | None = None) -> None:
    ft = parse_file_type(target)
    if target.upper() not in QUANTIZE_TARGETS:
        raise CreateError(f"unsupported quantization type {target} - supported types are {', '.join(QUANTIZE_TARGETS)}")
    g = open_gguf(src)
    try:
        cur_ft = int(g.kv.get("general.file_type", 0))
        if cur_ft not in (int(FileType.F32), int(FileType.F16), int(FileType.BF16)):
            raise CreateError("quantization is only supported for F16 and F32 models")
        n_layers = g.uint("block_count", 0)
        tied = "output.weight" not in g.tensors
        kv = dict(g.kv)
        kv["general.file_type"] = int(ft)
        kv["general.quantization_version"] = 2
        out = []
        for ti in g.tensors.values():
            import re
            m = re.match(r"blk\.(\d+)\.", ti.name)
            layer = int(m.group(1)) if m else 0
            tt = target_tensor_type(ti.name, ti.torch_shape, ti.dtype, ft, layer, n_layers, tied)
            raw = torch.from_numpy(g.tensor_bytes(ti.name).copy())
            if tt != ti.dtype:
                if progress:
                    progress(f"quantizing {ti.name} to {tt.name}")
                x = quants.dequantize_tensor(raw, ti.dtype, ti.torch_shape)
                raw = quants.quantize(x, tt)
            out.append(WriteTensor(ti.name, ti.shape, tt, raw.numpy()))
        write_gguf(dst, kv, out)
    finally:
        g.close()


def _is_checkpoint_dir(names: list[str]) -> bool:
    return "config.json" in names and any(n.endswith(".safetensors") for n in names)


def create_model(req: dict[str, Any]) -> Iterator[dict[str, Any]]:
    """Generator of progress objects ({"status": ...}); raises :class:`CreateError` on bad requests."""
    name = parse_name(req.get("model") or req.get("name") or "")
    if not name.valid:
        raise CreateError("invalid model name")
    layers: list[M.Layer] = []
    config: dict[str, Any] = {"architecture": "amd64", "os": "linux"}
    base_opts: dict[str, Any] = {}
    base_template = base_system = ""
    base_messages: list[dict[str, Any]] = []
    base_license: list[str] = []

    if req.get("from"):
        yield {"status": "reading model metadata"}
        try:
            base = get_model(req["from"])
        except ModelNotFound:
            raise CreateError(f"model '{req['from']}' not found", 404) from None
        man = M.read_manifest(parse_name(req["from"]))
        for l in man.layers:
            if l.media_type in (M.MT_MODEL, M.MT_PROJECTOR, M.MT_ADAPTER, M.MT_DRAFT):
                layers.append(M.Layer(l.media_type, l.digest, l.size, l.from_ or (str(parse_name(req["from"])) if l.media_type == M.MT_MODEL else "")))
        config.update(base.config)
        base_opts, base_template, base_system = dict(base.options), base.template, base.system
        base_messages, base_license = list(base.messages), list(base.license)
    elif req.get("files") and _is_checkpoint_dir(list(req["files"])):
        # a Hugging Face checkpoint (config.json + *.safetensors + tokenizer files): convert to GGUF first
        from ..convert.hf import ConvertError, convert_hf
        yield {"status": "converting model"}
        with tempfile.TemporaryDirectory(dir=M.blobs_dir()) as tmp:
            for fname, digest in req["files"].items():
                p = M.blob_path(digest)
                if not os.path.exists(p):
                    raise CreateError(f"blob {digest} for file {fname} not found")
                if os.path.basename(fname) != fname or fname in ("", ".", ".."):
                    raise CreateError(f"invalid file name {fname!r}")
                os.symlink(p, os.path.join(tmp, fname))
            out = os.path.join(tmp, "model.gguf")
            try:
                convert_hf(tmp, out)
            except (ConvertError, KeyError, OSError) as e:
                raise CreateError(f"conversion failed: {e}") from None
            layer = M.new_layer(out, M.MT_MODEL)
        layers.append(layer)
        config.update(gguf_config(layer.path()))
    elif req.get("files"):
        for fname, digest in req["files"].items():
            p = M.blob_path(digest)
            if not os.path.exists(p):
                raise CreateError(f"blob {digest} for file {fname} not found")
            with open(p, "rb") as f:
                magic = f.read(4)
            if magic != b"GGUF":
                raise CreateError(f"{fname}: only GGUF files can be imported (safetensors import goes through `convert`)")
            yield {"status": f"parsing GGUF"}
            g = open_gguf(p, max_array=0, metadata_only=True)
            is_proj = g.architecture == "clip" or any(t.startswith(("v.", "mm.")) for t in g.tensors) and "token_embd.weight" not in g.tensors
            g.close()
            layers.append(M.layer_from_existing(digest, M.MT_PROJECTOR if is_proj else M.MT_MODEL))
            if not is_proj:
                config.update(gguf_config(p))
    else:
        raise CreateError("neither 'from' or 'files' was specified")

    adapters = req.get("adapters") or {}
    if "adapter_config.json" in adapters and any(n.endswith(".safetensors") for n in adapters):
        # a PEFT LoRA directory: converted to an adapter GGUF for the architecture of the base model
        from ..convert.hf import ConvertError, convert_adapter
        from ..gguf.reader import open_gguf as _open_meta
        base_layer = next((l for l in layers if l.media_type == M.MT_MODEL), None)
        if base_layer is None:
            raise CreateError("an adapter needs a base model")
        yield {"status": "converting adapter"}
        with _open_meta(base_layer.path(), max_array=64, metadata_only=True) as bg:
            arch = bg.kv.get("general.architecture", "")
            n_head, n_kv = int(bg.kv.get(f"{arch}.attention.head_count", 0) or 0), int(bg.kv.get(f"{arch}.attention.head_count_kv", 0) or 0)
        with tempfile.TemporaryDirectory(dir=M.blobs_dir()) as tmp:
            for fname, digest in adapters.items():
                p = M.blob_path(digest)
                if not os.path.exists(p):
                    raise CreateError(f"blob {digest} for file {fname} not found")
                if os.path.basename(fname) != fname or fname in ("", ".", ".."):
                    raise CreateError(f"invalid file name {fname!r}")
                os.symlink(p, os.path.join(tmp, fname))
            out = os.path.join(tmp, "adapter.gguf")
            try:
                convert_adapter(tmp, out, arch, n_head, n_kv or n_head)
            except (ConvertError, KeyError, OSError) as e:
                raise CreateError(f"adapter conversion failed: {e}") from None
            layers.append(M.new_layer(out, M.MT_ADAPTER))
    else:
        for fname, digest in adapters.items():
            layers.append(M.layer_from_existing(digest, M.MT_ADAPTER))
    drafts = req.get("draft_files") or req.get("drafts") or {}
    if drafts:      # a draft model for speculative decoding (api/types.go:674-675) replaces the one inherited from the base
        layers = [l for l in layers if l.media_type != M.MT_DRAFT]
        for fname, digest in drafts.items():
            layers.append(M.layer_from_existing(digest, M.MT_DRAFT))

    q = req.get("quantize") or req.get("quantization")
    if q:
        idx = next((i for i, l in enumerate(layers) if l.media_type == M.MT_MODEL), None)
        if idx is not None:
            src = layers[idx].path()
            yield {"status": f"quantizing {config.get('file_type', 'model')} model to {q.upper()}"}
            fd, tmp = tempfile.mkstemp(suffix=".gguf", dir=M.blobs_dir())
            os.close(fd)
            try:
                quantize_gguf(src, tmp, q)
                layers[idx] = M.new_layer(tmp, M.MT_MODEL)
                config.update(gguf_config(layers[idx].path()))
            finally:
                if os.path.exists(tmp):
                    os.unlink(tmp)

    template = req.get("template") or base_template
    system = req.get("system") if req.get("system") is not None else base_system
    detected_stop: tuple[str, ...] = ()
    if not template and not req.get("renderer"):
        # a bare checkpoint: when its Jinja chat template is one of the well-known layouts the model gets the equivalent Go
        # template and that layout's stop strings (server/create.go detectChatTemplate, template/template.go Named)
        template, detected_stop = _detect_template(layers)
    if template:
        from ..text.template import Template
        from ..text.gotemplate import TemplateError
        try:
            Template(template)
        except TemplateError as e:
            raise CreateError(f"template error: {e}") from None
        layers.append(M.new_layer(template.encode(), M.MT_TEMPLATE))
    if system:
        layers.append(M.new_layer(system.encode(), M.MT_SYSTEM))
    lic = req.get("license")
    lic = [lic] if isinstance(lic, str) else (lic or base_license)
    for l in lic:
        layers.append(M.new_layer(l.encode(), M.MT_LICENSE))
    params = dict(base_opts)
    if detected_stop and "stop" not in params:
        params["stop"] = list(detected_stop)
    params.update(req.get("parameters") or {})
    if params:
        layers.append(M.new_layer(json.dumps(params, sort_keys=True).encode(), M.MT_PARAMS))
    messages = req.get("messages") or base_messages
    if messages:
        layers.append(M.new_layer(json.dumps(messages).encode(), M.MT_MESSAGES))
    for k in ("renderer", "parser", "requires"):
        if req.get(k):
            config[k] = req[k]
    yield {"status": "writing manifest"}
    cfg_layer = M.new_layer(json.dumps(config, sort_keys=True).encode(), M.MT_CONFIG)
    M.write_manifest(name, cfg_layer, layers)
    yield {"status": "success"}
