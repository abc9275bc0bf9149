"""Hugging Face checkpoint -> GGUF: logits of the converted file on the fp32 graph equal the transformers model's."""
import json
import os

import pytest
import torch

from ollama_b200.convert.hf import convert_hf, map_name, permute_qk
from ollama_b200.convert.safetensors import SafetensorsError, SafetensorsFile, save_file


def test_safetensors_roundtrip_and_limits(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.arange(7, dtype=torch.int32), "c": torch.randn(2, 2).to(torch.bfloat16), "s": torch.tensor(3.0)}
    p = tmp_path / "x.safetensors"
    save_file(t, p, {"format": "pt"})
    with SafetensorsFile(p) as f:
        assert set(f.keys()) == set(t) and f.metadata == {"format": "pt"}
        for k, v in t.items():
            assert torch.equal(f.tensor(k), v) and f.shape(k) == tuple(v.shape)
    raw = bytearray(p.read_bytes())
    raw[:8] = (10 ** 12).to_bytes(8, "little")
    (tmp_path / "bad.safetensors").write_bytes(bytes(raw))
    with pytest.raises(SafetensorsError):
        SafetensorsFile(tmp_path / "bad.safetensors")


def test_name_mapping_and_permutation():
    assert map_name("model.layers.3.self_attn.q_proj.weight", "llama") == "blk.3.attn_q.weight"
    assert map_name("model.layers.0.post_attention_layernorm.weight", "llama") == "blk.0.ffn_norm.weight"
    assert map_name("model.layers.0.post_attention_layernorm.weight", "gemma2") == "blk.0.post_attention_norm.weight"
    assert map_name("model.layers.1.mlp.experts.5.down_proj.weight", "qwen3moe") == "blk.1.ffn_down_exps.weight#5"
    assert map_name("model.layers.1.block_sparse_moe.experts.2.w3.weight", "llama") == "blk.1.ffn_up_exps.weight#2"
    assert map_name("lm_head.weight", "qwen3") == "output.weight" and map_name("model.foo", "llama") is None
    w = torch.arange(16.0).view(8, 2)          # 2 heads x head_dim 4
    p = permute_qk(w, 2)
    assert p[:, 0].tolist() == [0.0, 4.0, 2.0, 6.0, 8.0, 12.0, 10.0, 14.0]     # (i, i + hd/2) pairs become neighbours


def _tiny_tokenizer(path):
    from tokenizers import Tokenizer, models, pre_tokenizers
    vocab = {chr(ord("a") + i): i for i in range(26)}
    vocab.update({"ab": 26, "<s>": 27, "</s>": 28})
    tok = Tokenizer(models.BPE(vocab=vocab, merges=[("a", "b")]))
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.add_special_tokens(["<s>", "</s>"])
    tok.save(os.path.join(path, "tokenizer.json"))
    with open(os.path.join(path, "tokenizer_config.json"), "w") as f:
        json.dump({"bos_token": "<s>", "eos_token": "</s>", "add_bos_token": True, "chat_template": "{{ messages }}"}, f)


@pytest.mark.parametrize("family", ["llama", "qwen3", "qwen3moe", "gpt-oss", "phi3", "phi3-long"])
def test_converted_checkpoint_matches_transformers(tmp_path, family):
    transformers = pytest.importorskip("transformers")
    torch.manual_seed(0)
    common = dict(vocab_size=64, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                  max_position_embeddings=128, rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False)
    if family == "llama":
        cfg = transformers.LlamaConfig(**common)
        model = transformers.LlamaForCausalLM(cfg)
    elif family == "qwen3":
        cfg = transformers.Qwen3Config(head_dim=32, **common)
        model = transformers.Qwen3ForCausalLM(cfg)
    elif family == "qwen3moe":
        cfg = transformers.Qwen3MoeConfig(head_dim=16, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, norm_topk_prob=True,
                                          decoder_sparse_step=1, mlp_only_layers=[], **common)
        model = transformers.Qwen3MoeForCausalLM(cfg)
    elif family.startswith("phi3"):     # fused Q|K|V and gate|up matrices; "long": per-frequency divisors and the attention factor
        extra = {}
        if family == "phi3-long":
            g = torch.Generator().manual_seed(3)
            extra = dict(max_position_embeddings=256, original_max_position_embeddings=64,
                         rope_scaling={"type": "longrope", "long_factor": (1 + 3 * torch.rand(8, generator=g)).tolist(),
                                       "short_factor": (1 + 0.2 * torch.rand(8, generator=g)).tolist()})
        cfg = transformers.Phi3Config(**{**common, **extra}, pad_token_id=0)
        model = transformers.Phi3ForCausalLM(cfg)
    else:       # gpt-oss: YaRN beyond the original context, sinks, alternating 8-token window, biased router, clamped SwiGLU
        cfg = transformers.GptOssConfig(vocab_size=64, hidden_size=64, intermediate_size=32, num_hidden_layers=2, num_attention_heads=4,
                                        num_key_value_heads=2, head_dim=16, num_local_experts=4, num_experts_per_tok=2, sliding_window=8,
                                        max_position_embeddings=2048, rope_theta=150000.0, tie_word_embeddings=False,
                                        rope_scaling={"rope_type": "yarn", "factor": 32.0, "beta_fast": 32.0, "beta_slow": 1.0,
                                                      "truncate": False, "original_max_position_embeddings": 64})
        model = transformers.GptOssForCausalLM(cfg)
        with torch.no_grad():
            for n, p in model.named_parameters():
                if "bias" in n or "sinks" in n:
                    p.normal_(0, 0.5)
    model = model.float().eval()
    src = tmp_path / "hf"
    model.save_pretrained(src, safe_serialization=True)
    _tiny_tokenizer(str(src))
    names = os.listdir(src)
    if not any(n.endswith(".safetensors") for n in names):
        pytest.skip("this transformers build did not write safetensors")
    out = str(tmp_path / "m.gguf")
    kv = convert_hf(str(src), out, outtype="f32")
    assert kv["general.architecture"] == family.removesuffix("-long") and kv["tokenizer.ggml.model"] == "gpt2" and kv["tokenizer.ggml.bos_token_id"] == 27
    assert kv["tokenizer.chat_template"] == "{{ messages }}" and len(kv["tokenizer.ggml.tokens"]) == 64

    from ollama_b200.engine.backend import TorchBackend, open_model
    be = TorchBackend(open_model(out), "cpu")
    be.alloc(1, 128)
    ids = torch.randint(0, 64, (90 if family in ("gpt-oss", "phi3-long") else 11,), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = model(ids[None]).logits[0, -1]
    got = be.prefill(0, ids.tolist(), 0)
    assert torch.allclose(got, ref, atol=2e-4, rtol=1e-3), (got - ref).abs().max()
    if family == "phi3":        # the views into the fused matrices hold for a block-quantised encoding too
        from ollama_b200.store.create import quantize_gguf
        q = str(tmp_path / "q.gguf")
        quantize_gguf(out, q, "q8_0")
        bq = TorchBackend(open_model(q), "cpu")
        bq.alloc(1, 128)
        assert (bq.prefill(0, ids.tolist(), 0) - ref).abs().max() < 0.02


def test_create_from_checkpoint_directory_through_the_api(tmp_path, monkeypatch):
    """POST /api/create with the files of a Hugging Face checkpoint: converted to GGUF, then served."""
    transformers = pytest.importorskip("transformers")
    import hashlib

    from starlette.testclient import TestClient
    monkeypatch.setenv("OLLAMA_MODELS", str(tmp_path / "store"))
    monkeypatch.setenv("B200_DEVICE", "cpu")
    monkeypatch.setenv("OLLAMA_CONTEXT_LENGTH", "128")
    torch.manual_seed(0)
    cfg = transformers.LlamaConfig(vocab_size=64, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, max_position_embeddings=128, tie_word_embeddings=False)
    src = tmp_path / "hf"
    transformers.LlamaForCausalLM(cfg).float().save_pretrained(src, safe_serialization=True)
    _tiny_tokenizer(str(src))
    from ollama_b200.server.routes import create_app
    with TestClient(create_app()) as c:
        files = {}
        for n in sorted(os.listdir(src)):
            data = open(src / n, "rb").read()
            digest = "sha256:" + hashlib.sha256(data).hexdigest()
            assert c.post(f"/api/blobs/{digest}", content=data).status_code in (200, 201)
            files[n] = digest
        r = c.post("/api/create", json={"model": "conv", "files": files, "template": "{{ .Prompt }}", "stream": False})
        assert r.status_code == 200 and r.json()["status"] == "success", r.text
        info = c.post("/api/show", json={"model": "conv"}).json()
        assert info["details"]["family"] == "llama" and info["model_info"]["llama.block_count"] == 2
        out = c.post("/api/generate", json={"model": "conv", "prompt": "abab", "stream": False, "options": {"num_predict": 4, "temperature": 0}}).json()
        assert out["done"] and out["eval_count"] == 4


def test_gpt_oss_checkpoint_with_packed_mxfp4_experts(tmp_path):
    """Experts shipped as MXFP4 blocks + scales are re-ordered into GGML blocks without re-quantising: the converted
    model gives the logits of transformers running the same (dequantised) expert weights."""
    transformers = pytest.importorskip("transformers")
    st = pytest.importorskip("safetensors.torch")
    from transformers.integrations.mxfp4 import _convert_moe_packed_tensors
    from ollama_b200.gguf import quants
    from ollama_b200.gguf.types import GGMLType
    torch.manual_seed(0)
    cfg = transformers.GptOssConfig(vocab_size=64, hidden_size=64, intermediate_size=32, num_hidden_layers=2, num_attention_heads=4,
                                    num_key_value_heads=2, head_dim=16, num_local_experts=4, num_experts_per_tok=2, sliding_window=8,
                                    max_position_embeddings=128, rope_theta=150000.0, tie_word_embeddings=False)
    model = transformers.GptOssForCausalLM(cfg).float().eval()
    src = tmp_path / "hf"
    model.save_pretrained(src, safe_serialization=True)
    _tiny_tokenizer(str(src))
    files = [n for n in os.listdir(src) if n.endswith(".safetensors")]
    if len(files) != 1:
        pytest.skip("expected one safetensors file")
    tensors = st.load_file(str(src / files[0]))
    packed = {}
    for name in [n for n in tensors if n.endswith(("experts.gate_up_proj", "experts.down_proj"))]:
        w = tensors.pop(name).float().transpose(1, 2).contiguous()          # [expert, out, in]
        e, rows, k = w.shape
        blk = quants.quantize(w, GGMLType.MXFP4).view(e, rows, k // 32, 17)
        deq = quants.dequantize(blk.reshape(-1), GGMLType.MXFP4).view(e, rows, k)
        nib = blk[..., 1:]
        lo, hi = nib[..., 0::2], nib[..., 1::2]                             # GGML bytes 2j and 2j + 1
        a = (lo & 0x0F) | ((hi & 0x0F) << 4)                                # checkpoint bytes 0..7: elements (2j, 2j + 1)
        b = (lo >> 4) | (hi & 0xF0)                                         # checkpoint bytes 8..15: elements (16 + 2j, 17 + 2j)
        blocks, scales = torch.cat([a, b], -1).contiguous(), blk[..., 0].contiguous()
        # the library's own unpacking of this layout gives the same values ([expert, in, out])
        assert torch.equal(_convert_moe_packed_tensors(blocks, scales, dtype=torch.float32), deq.transpose(1, 2))
        packed[name + "_blocks"], packed[name + "_scales"] = blocks, scales
        with torch.no_grad():
            dict(model.named_parameters())[name].copy_(deq.transpose(1, 2))
    tensors.update(packed)
    st.save_file(tensors, str(src / files[0]), metadata={"format": "pt"})
    out = str(tmp_path / "m.gguf")
    convert_hf(str(src), out, outtype="f32")
    from ollama_b200.engine.backend import TorchBackend, open_model
    g = open_model(out)
    assert g.tensors["blk.0.ffn_gate_exps.weight"].dtype == GGMLType.MXFP4 and g.tensors["blk.1.ffn_down_exps.weight"].dtype == GGMLType.MXFP4
    be = TorchBackend(g, "cpu")
    be.alloc(1, 128)
    ids = torch.randint(0, 64, (40,), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = model(ids[None]).logits[0, -1]
    got = be.prefill(0, ids.tolist(), 0)
    assert torch.allclose(got, ref, atol=2e-4, rtol=1e-3), (got - ref).abs().max()


def test_sentencepiece_model_file_vocabulary(tmp_path):
    """A checkpoint that ships only ``tokenizer.model``: pieces, scores and piece types come from the SentencePiece model,
    added tokens are appended, and the resulting tokenizer encodes like SentencePiece itself."""
    spm = pytest.importorskip("sentencepiece")
    from ollama_b200.convert.hf import tokenizer_kv
    from ollama_b200.text.tokenizer import SPMTokenizer, tokenizer_from_gguf
    corpus = tmp_path / "corpus.txt"
    words = "the quick brown fox jumps over the lazy dog while reading tokenizer models about byte fallback and pieces".split()
    corpus.write_text("\n".join(" ".join(words[(i * 7 + j) % len(words)] for j in range(9)) for i in range(400)))
    spm.SentencePieceTrainer.train(input=str(corpus), model_prefix=str(tmp_path / "tokenizer"), vocab_size=320, model_type="bpe",
                                   byte_fallback=True, character_coverage=1.0, bos_id=1, eos_id=2, unk_id=0, pad_id=-1,
                                   user_defined_symbols=["<start_of_turn>"], minloglevel=2)
    (tmp_path / "added_tokens.json").write_text(json.dumps({"<extra_a>": 320, "<extra_b>": 321}))
    (tmp_path / "tokenizer_config.json").write_text(json.dumps({"bos_token": "<s>", "eos_token": {"content": "</s>"}, "add_bos_token": True}))
    kv = tokenizer_kv(str(tmp_path), 324)
    sp = spm.SentencePieceProcessor(model_file=str(tmp_path / "tokenizer.model"))
    toks, types, scores = kv["tokenizer.ggml.tokens"], kv["tokenizer.ggml.token_type"], kv["tokenizer.ggml.scores"]
    assert kv["tokenizer.ggml.model"] == "llama" and len(toks) == 324 and toks[:3] == ["<unk>", "<s>", "</s>"] and types[:3] == [2, 3, 3]
    assert types[toks.index("<0x41>")] == 6 and types[toks.index("<start_of_turn>")] in (3, 4) and toks[320:322] == ["<extra_a>", "<extra_b>"]
    assert types[320:] == [4, 4, 5, 5] and scores[320] == -1000.0 and scores[10] == sp.get_score(10)
    assert kv["tokenizer.ggml.bos_token_id"] == 1 and kv["tokenizer.ggml.eos_token_id"] == 2 and kv["tokenizer.ggml.add_bos_token"] is True
    tk = tokenizer_from_gguf(kv)
    assert isinstance(tk, SPMTokenizer)
    for text in ("the quick brown fox", "reading about pieces and models", "unseen wörd ☃ 42"):
        assert tk.encode(text, add_special=False) == sp.encode(text), text
        assert tk.decode(tk.encode(text, add_special=False)).strip() == text
    (tmp_path / "added_tokens.json").write_text(json.dumps({"<gap>": 400}))
    with pytest.raises(Exception, match="invalid token id"):
        tokenizer_kv(str(tmp_path), 324)


def test_peft_lora_adapter_conversion_matches_merged_weights(tmp_path):
    """A PEFT LoRA directory converted to an adapter GGUF and merged at load equals transformers running the merged
    weights; the Q projection's B factor needs the llama rotary row permutation for that to hold."""
    transformers = pytest.importorskip("transformers")
    st = pytest.importorskip("safetensors.torch")
    from ollama_b200.convert.hf import convert_adapter
    from ollama_b200.engine.backend import TorchBackend, open_model
    torch.manual_seed(0)
    cfg = transformers.LlamaConfig(vocab_size=64, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, max_position_embeddings=128, rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False)
    model = transformers.LlamaForCausalLM(cfg).float().eval()
    src = tmp_path / "hf"
    model.save_pretrained(src, safe_serialization=True)
    _tiny_tokenizer(str(src))
    base = str(tmp_path / "base.gguf")
    convert_hf(str(src), base, outtype="f32")
    # adapter on q_proj, k_proj and down_proj of both layers
    r, alpha = 4, 8.0
    ad_dir = tmp_path / "peft"
    ad_dir.mkdir()
    tensors = {}
    params = dict(model.named_parameters())
    with torch.no_grad():
        for i in range(2):
            for mod in ("self_attn.q_proj", "self_attn.k_proj", "mlp.down_proj"):
                w = params[f"model.layers.{i}.{mod}.weight"]
                a, b = torch.randn(r, w.shape[1]) * 0.1, torch.randn(w.shape[0], r) * 0.1
                tensors[f"base_model.model.model.layers.{i}.{mod}.lora_A.weight"] = a
                tensors[f"base_model.model.model.layers.{i}.{mod}.lora_B.weight"] = b
                w.add_((b @ a) * (alpha / r))                    # the reference result: merged weights
    st.save_file(tensors, str(ad_dir / "adapter_model.safetensors"), metadata={"format": "pt"})
    (ad_dir / "adapter_config.json").write_text(json.dumps({"peft_type": "LORA", "r": r, "lora_alpha": alpha, "target_modules": ["q_proj", "k_proj", "down_proj"]}))
    ad = str(tmp_path / "adapter.gguf")
    kv = convert_adapter(str(ad_dir), ad, "llama", n_head=4, n_kv_head=2)
    assert kv["adapter.lora.alpha"] == alpha and kv["general.type"] == "adapter"
    g = open_model(base)
    be = TorchBackend(g, "cpu", adapters=[ad])
    be.alloc(1, 128)
    ids = torch.randint(0, 64, (13,), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = model(ids[None]).logits[0, -1]
    got = be.prefill(0, ids.tolist(), 0)
    assert torch.allclose(got, ref, atol=2e-4, rtol=1e-3), (got - ref).abs().max()
    plain = TorchBackend(g, "cpu")
    plain.alloc(1, 128)
    assert (plain.prefill(0, ids.tolist(), 0) - ref).abs().max().item() > 1e-2
    with pytest.raises(Exception, match="head counts"):
        convert_adapter(str(ad_dir), str(tmp_path / "x.gguf"), "llama")


def test_create_with_a_peft_adapter_directory(tmp_path, monkeypatch):
    """``create`` with the files of a PEFT adapter: an adapter layer (GGUF) is added to the model and named by `show`."""
    st = pytest.importorskip("safetensors.torch")
    from ollama_b200.gguf.reader import open_gguf
    from ollama_b200.models.synth import write_synthetic_gguf
    from ollama_b200.store import manifest as M
    from ollama_b200.store.create import CreateError, create_model
    from ollama_b200.store.model import get_model
    monkeypatch.setenv("OLLAMA_MODELS", str(tmp_path / "store"))
    base = tmp_path / "m.gguf"
    write_synthetic_gguf(str(base), "tiny-llama", "Q8_0")
    model_layer = M.new_layer(str(base), M.MT_MODEL)
    a, b = torch.randn(4, 256) * 0.1, torch.randn(256, 4) * 0.1
    f = tmp_path / "adapter_model.safetensors"
    st.save_file({"base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight": a,
                  "base_model.model.model.layers.0.self_attn.q_proj.lora_B.weight": b}, str(f), metadata={"format": "pt"})
    c = tmp_path / "adapter_config.json"
    c.write_text(json.dumps({"peft_type": "LORA", "r": 4, "lora_alpha": 16}))
    files = {"adapter_model.safetensors": M.new_layer(str(f), "application/octet-stream").digest,
             "adapter_config.json": M.new_layer(str(c), "application/octet-stream").digest}
    ev = list(create_model({"model": "tuned", "files": {"m.gguf": model_layer.digest}, "adapters": files}))
    assert ev[-1]["status"] == "success" and any(e["status"] == "converting adapter" for e in ev)
    m = get_model("tuned")
    assert len(m.adapter_paths) == 1 and "ADAPTER " in m.modelfile()
    with open_gguf(m.adapter_paths[0]) as g:
        assert g.kv["adapter.lora.alpha"] == 16.0 and set(g.tensors) == {"blk.0.attn_q.weight.lora_a", "blk.0.attn_q.weight.lora_b"}
    with pytest.raises(CreateError):
        list(create_model({"model": "bad", "adapters": files}))


def test_safetensors_reader_survives_corrupted_headers(tmp_path):
    """Byte flips and truncations of a valid file: the reader opens it or raises SafetensorsError, nothing else."""
    import random
    st = pytest.importorskip("safetensors.torch")
    from ollama_b200.convert.safetensors import SafetensorsError, SafetensorsFile
    p = str(tmp_path / "a.safetensors")
    st.save_file({"a": torch.zeros(4, 8), "b": torch.ones(3, dtype=torch.float16), "c": torch.zeros((), dtype=torch.bfloat16)}, p)
    data = open(p, "rb").read()
    rnd = random.Random(3)
    q = str(tmp_path / "m.safetensors")
    opened = 0
    for _ in range(800):
        b = bytearray(data)
        for _ in range(rnd.randint(1, 4)):
            b[rnd.randrange(0, min(len(b), 300))] = rnd.randrange(256)
        if rnd.random() < 0.2:
            b = b[:rnd.randrange(1, len(b))]
        with open(q, "wb") as f:
            f.write(b)
        try:
            sf = SafetensorsFile(q)
            for k in sf.keys():
                sf.tensor(k)
            sf.close()
            opened += 1
        except SafetensorsError:
            pass
    assert 0 < opened < 800


def _tiny_gemma3_vision(path):
    """A random multimodal gemma3 checkpoint (2-layer text model, 2-layer SigLIP tower on 56 x 56 images, 4 image tokens)."""
    transformers = pytest.importorskip("transformers")
    torch.manual_seed(0)
    tc = dict(vocab_size=64, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              head_dim=16, max_position_embeddings=128, rms_norm_eps=1e-6, sliding_window=8, query_pre_attn_scalar=16)
    vc = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, image_size=56, patch_size=14, num_channels=3)
    cfg = transformers.Gemma3Config(text_config=tc, vision_config=vc, mm_tokens_per_image=4, image_token_index=60, boi_token_index=61,
                                    eoi_token_index=62)
    model = transformers.Gemma3ForConditionalGeneration(cfg).float().eval()
    with torch.no_grad():
        for n, p in model.named_parameters():
            if "norm" in n or "bias" in n:
                p.normal_(0, 0.3)
            if "mm_input_projection" in n:          # zero-initialised in the library: every image would project to nothing
                p.normal_(0, 0.2)
    model.save_pretrained(path, safe_serialization=True)
    _tiny_tokenizer(str(path))
    return model


def _png(seed: int, w: int = 100, h: int = 80) -> bytes:
    import io

    import numpy as np
    from PIL import Image
    buf = io.BytesIO()
    Image.fromarray((np.random.RandomState(seed).rand(h, w, 3) * 255).astype("uint8")).save(buf, format="PNG")
    return buf.getvalue()


def test_gemma3_image_input_matches_transformers(tmp_path):
    """A multimodal gemma3 checkpoint keeps its vision tower through the conversion; the tower + projector give the image
    features of the transformers model, and a prompt with the image in it (embedding rows in place of the soft tokens, the
    image positions attending to each other in both directions) gives its logits."""
    src = tmp_path / "hf"
    model = _tiny_gemma3_vision(src)
    out = str(tmp_path / "m.gguf")
    kv = convert_hf(str(src), out, outtype="f32")
    assert kv["gemma3.vision.block_count"] == 2 and kv["gemma3.vision.image_size"] == 56 and kv["gemma3.mm.tokens_per_image"] == 4
    from ollama_b200.engine.backend import TorchBackend, open_model
    from ollama_b200.models.vision import load_tower, preprocess
    g = open_model(out)
    assert g.has("v.patch_embedding.weight") and g.has("mm.mm_input_projection.weight") and g.has("v.blk.1.mlp.fc2.bias")
    tower = load_tower(g)
    data = _png(0)
    px = preprocess(data, 56)
    assert px.shape == (3, 56, 56) and -1.0 <= float(px.min()) and float(px.max()) <= 1.0
    emb = tower.encode(data)
    with torch.no_grad():
        feats = model.get_image_features(pixel_values=px[None])
    feats = feats if torch.is_tensor(feats) else getattr(feats, "pooler_output", feats[0])
    assert emb.shape == (4, 64) and torch.allclose(emb, feats.reshape(4, 64), atol=1e-5) and float(emb.abs().mean()) > 0.05
    ids = [5, 7, 61, 60, 60, 60, 60, 62, 9, 11, 13]
    with torch.no_grad():
        ref = model(input_ids=torch.tensor([ids]), pixel_values=px[None], token_type_ids=torch.tensor([[int(t == 60) for t in ids]])).logits[0, -1]
    be = TorchBackend(g, "cpu")
    be.alloc(1, 64)
    rows = [i for i, t in enumerate(ids) if t == 60]
    toks = [-(1 + i) if t == 60 else t for i, t in enumerate(ids)]
    got = be.prefill(0, toks, 0, embeds=(rows, emb), spans=[(rows[0], rows[-1] + 1)])
    assert torch.allclose(got, ref, atol=2e-5), (got - ref).abs().max()
    causal_only = be.prefill(0, toks, 0, embeds=(rows, emb))
    assert (causal_only - ref).abs().max() > 1e-4            # the two-way attention inside the image is part of the model


def test_chat_with_images_through_the_api(tmp_path, monkeypatch):
    """POST /api/chat with ``images``: the vision model answers, the prompt count includes the image's positions, another
    image changes the first token's distribution, and a text-only model still refuses images with 400."""
    import base64
    import hashlib

    from starlette.testclient import TestClient
    monkeypatch.setenv("OLLAMA_MODELS", str(tmp_path / "store"))
    monkeypatch.setenv("B200_DEVICE", "cpu")
    monkeypatch.setenv("OLLAMA_CONTEXT_LENGTH", "128")
    src = tmp_path / "hf"
    _tiny_gemma3_vision(src)
    from ollama_b200.server.routes import create_app
    with TestClient(create_app()) as c:
        files = {}
        for n in sorted(os.listdir(src)):
            data = open(src / n, "rb").read()
            digest = "sha256:" + hashlib.sha256(data).hexdigest()
            assert c.post(f"/api/blobs/{digest}", content=data).status_code in (200, 201)
            files[n] = digest
        r = c.post("/api/create", json={"model": "g3v", "files": files, "template": "{{ .Prompt }}", "stream": False})
        assert r.status_code == 200 and r.json()["status"] == "success", r.text
        info = c.post("/api/show", json={"model": "g3v"}).json()
        assert "vision" in info["capabilities"] and info["model_info"]["gemma3.vision.block_count"] == 2
        ask = lambda images, content="abab": c.post("/api/chat", json={                                  # noqa: E731
            "model": "g3v", "messages": [{"role": "user", "content": content, "images": images}], "stream": False, "logprobs": True,
            "top_logprobs": 3, "options": {"num_predict": 2, "temperature": 0}})
        plain = c.post("/api/chat", json={"model": "g3v", "messages": [{"role": "user", "content": "abab"}], "stream": False,
                                          "options": {"num_predict": 2, "temperature": 0}}).json()
        one = ask([base64.b64encode(_png(1)).decode()])
        assert one.status_code == 200, one.text
        one = one.json()
        assert one["done"] and one["eval_count"] == 2
        assert one["prompt_eval_count"] >= plain["prompt_eval_count"] + 4         # four image positions (this toy vocabulary has no line break)
        other = ask([base64.b64encode(_png(2)).decode()]).json()
        lp = lambda r: [round(t["logprob"], 4) for t in r["logprobs"][0]["top_logprobs"]]                 # noqa: E731
        assert lp(one) != lp(other)
        again = ask([base64.b64encode(_png(1)).decode()]).json()
        assert lp(again) == lp(one)
        placed = ask([base64.b64encode(_png(1)).decode()], "ab [img] ab").json()
        assert placed["done"] and lp(placed) != lp(one)
        bad = ask(["bm90IGFuIGltYWdl"])
        assert bad.status_code == 400 and "image" in bad.json()["error"]
        url = "data:image/png;base64," + base64.b64encode(_png(1)).decode()
        oa = c.post("/v1/chat/completions", json={"model": "g3v", "max_tokens": 2, "temperature": 0, "messages": [
            {"role": "user", "content": [{"type": "text", "text": "abab"}, {"type": "image_url", "image_url": {"url": url}}]}]})
        assert oa.status_code == 200 and oa.json()["usage"]["prompt_tokens"] == one["prompt_eval_count"], oa.text
        an = c.post("/v1/messages", json={"model": "g3v", "max_tokens": 2, "messages": [{"role": "user", "content": [
            {"type": "image", "source": {"type": "base64", "media_type": "image/png", "data": base64.b64encode(_png(1)).decode()}},
            {"type": "text", "text": "abab"}]}]})
        assert an.status_code == 200 and an.json()["usage"]["input_tokens"] == one["prompt_eval_count"], an.text
        gen = c.post("/api/generate", json={"model": "g3v", "prompt": "abab", "images": [base64.b64encode(_png(1)).decode()], "stream": False,
                                            "options": {"num_predict": 2, "temperature": 0}})
        assert gen.status_code == 200 and gen.json()["prompt_eval_count"] == one["prompt_eval_count"], gen.text
