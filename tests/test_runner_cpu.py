"""CPU plumbing: tiny llama (2 layers, d 256, 4/2 heads, FFN 688, vocab 32000) through the runner."""
import pytest
import torch

from ollama_b200.engine.runner import CompletionRequest, Runner, RunnerOptions
from ollama_b200.engine.sampler import SamplingParams


def _prompt():
    g = torch.Generator().manual_seed(1)
    return torch.randint(259, 32000, (16,), generator=g).tolist()


def _greedy(path, **kw):
    r = Runner(path, RunnerOptions(num_ctx=512, device="cpu", **kw))
    try:
        out = list(r.completion(CompletionRequest(prompt=_prompt(), sampling=SamplingParams(temperature=0), num_predict=32)))
    finally:
        r.close()
    return out


def test_generate_greedy_f32_and_q8(tiny_llama_path, tiny_llama_q8_path):
    a = _greedy(tiny_llama_path)
    b = _greedy(tiny_llama_q8_path)
    ta = [t for c in a for t in c.tokens]
    tb = [t for c in b for t in c.tokens]
    assert len(ta) == 32 and a[-1].done and a[-1].done_reason == "length"
    assert a[-1].prompt_eval_count == 16 and a[-1].eval_count == 32
    assert ta[:8] == tb[:8]                      # Q8_0 keeps the greedy path for the first tokens
    assert "".join(c.content for c in a).startswith(f"<t{ta[0]}>")


def test_prefix_cache_and_parallel_slots(tiny_llama_path):
    r = Runner(tiny_llama_path, RunnerOptions(num_ctx=128, num_parallel=2, device="cpu"))
    try:
        p = _prompt()
        req = lambda: CompletionRequest(prompt=p, sampling=SamplingParams(temperature=0), num_predict=4)
        first = list(r.completion(req()))
        again = list(r.completion(req()))
        assert [c.tokens for c in first] == [c.tokens for c in again]
        assert again[-1].cached_tokens == len(p) - 1 or again[-1].cached_tokens >= len(p) - 1
        # two concurrent requests on two slots
        s1, s2 = r.submit(req()), r.submit(req())
        o1, o2 = [], []
        for s, o in ((s1, o1), (s2, o2)):
            while True:
                ch = s.out.get(timeout=60)
                o.append(ch)
                if ch.done:
                    break
        assert [c.tokens for c in o1] == [c.tokens for c in o2] == [c.tokens for c in first]
    finally:
        r.close()


def test_prompts_of_waiting_sequences_share_one_prefill_pass(tiny_llama_path):
    """Three requests arrive together with prompts of 40, 9 and 23 tokens and a budget of 16 rows per pass: a pass is filled in
    arrival order (what the first prompt leaves over goes to the next), and each request decodes what it decodes alone."""
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(259, 32000, (n,), generator=g).tolist() for n in (40, 9, 23)]
    req = lambda p: CompletionRequest(prompt=p, sampling=SamplingParams(temperature=0), num_predict=5, cache_prompt=False)
    solo = Runner(tiny_llama_path, RunnerOptions(num_ctx=128, device="cpu"))
    try:
        want = [[t for c in solo.completion(req(p)) for t in c.tokens] for p in prompts]
    finally:
        solo.close()
    r = Runner(tiny_llama_path, RunnerOptions(num_ctx=128, num_parallel=3, num_batch=16, device="cpu"))
    try:
        calls = []
        inner = r.backend.prefill_many
        r.backend.prefill_many = lambda segs, need: (calls.append([(len(t), p0) for _, t, p0 in segs]), inner(segs, need))[1]
        with r.cv:                                  # all three are queued before the loop admits any
            seqs = [r.submit(req(p)) for p in prompts]
        got = []
        for s in seqs:
            toks = []
            while True:
                ch = s.out.get(timeout=60)
                toks += ch.tokens
                if ch.done:
                    assert ch.prompt_eval_count == len(s.prompt) and not ch.error
                    break
            got.append(toks)
        assert got == want
        assert all(sum(n for n, _ in c) <= 16 for c in calls)
        assert calls[0] == [(16, 0)] and calls[1] == [(16, 16)]          # the first prompt fills the pass while it can
        assert calls[2] == [(8, 32), (8, 0)]                             # its last rows, and the second prompt rides along
        assert calls[3] == [(1, 8), (15, 0)]                             # the second ends, the third starts in the same pass
        assert r.stats["prefill_batches"] == len(calls) >= 4
    finally:
        r.close()


def test_context_limit_and_shift(tiny_llama_path):
    r = Runner(tiny_llama_path, RunnerOptions(num_ctx=32, device="cpu"))
    try:
        p = _prompt()
        out = list(r.completion(CompletionRequest(prompt=p, sampling=SamplingParams(temperature=0), num_predict=64, shift=False)))
        assert out[-1].done_reason == "length" and out[-1].eval_count <= 32 - 16 + 1
        out = list(r.completion(CompletionRequest(prompt=p, sampling=SamplingParams(temperature=0), num_predict=40, shift=True)))
        assert out[-1].eval_count == 40
    finally:
        r.close()


def test_prefix_held_by_a_busy_slot_is_copied_not_evaluated_again(tiny_llama_path):
    """While one request is still generating, a second one with the same 48-token preamble arrives: it gets another slot, the
    preamble's cache rows are copied from the busy slot, only the new tokens are evaluated, and the answer is what the
    request produces on its own."""
    g = torch.Generator().manual_seed(9)
    shared = torch.randint(259, 32000, (48,), generator=g).tolist()
    tail = torch.randint(259, 32000, (6,), generator=g).tolist()
    req = lambda p, n: CompletionRequest(prompt=p, sampling=SamplingParams(temperature=0), num_predict=n, ignore_eos=True)
    solo = Runner(tiny_llama_path, RunnerOptions(num_ctx=256, device="cpu"))
    try:
        want = [t for c in solo.completion(req(shared + tail, 6)) for t in c.tokens]
    finally:
        solo.close()
    r = Runner(tiny_llama_path, RunnerOptions(num_ctx=256, num_parallel=2, device="cpu"))
    try:
        a = r.submit(req(shared + [300, 301], 150))
        assert not a.out.get(timeout=60).done                      # its prompt is in the cache and it is generating
        b = r.submit(req(shared + tail, 6))
        got, last = [], None
        while last is None or not last.done:
            last = b.out.get(timeout=60)
            got += last.tokens
        assert got == want
        assert last.cached_tokens == 48 and last.prompt_eval_count == 54
        assert r.stats["prefix_copies"] == 1 and r.stats["prefix_copied_tokens"] == 48
        a.cancelled = True
    finally:
        r.close()


def test_context_shift_turns_cached_keys_to_their_new_positions(tiny_llama_path):
    """Dropping rows [keep, keep + discard) of a slot: the first layer's keys and values (functions of token and position only)
    equal those of a fresh pass over the shortened sequence; deeper layers keep their content, turned back by the shift."""
    from ollama_b200.engine.backend import TorchBackend, open_model
    from ollama_b200.ops import reference as R
    be = TorchBackend(open_model(tiny_llama_path), "cpu")
    be.alloc(2, 64)
    toks = torch.randint(259, 32000, (40,), generator=torch.Generator().manual_seed(2)).tolist()
    keep, discard = 4, 10
    be.prefill(0, toks, 0)
    before = [k[0, :40].clone() for k in be.cache.k]
    be.shift(0, keep, discard, 40)
    new = toks[:keep] + toks[keep + discard:]
    be.prefill(1, new, 0)
    assert torch.allclose(be.cache.k[0][0, :30], be.cache.k[0][1, :30], atol=1e-4)
    assert torch.allclose(be.cache.v[0][0, :30], be.cache.v[0][1, :30], atol=1e-6)
    fwd = torch.full((26,), discard)
    for i in range(be.cfg.n_layers):
        again = R.rope(be.cache.k[i][0, keep:30], fwd, be.model.layer_rope(i), be.cfg.rope_style, 1.0)
        assert torch.allclose(again, before[i][keep + discard:40], atol=1e-4)
        assert torch.equal(be.cache.k[i][0, :keep], before[i][:keep])
    # the next token's logits: attention sees 30 consecutive positions
    a = be.decode([0], [toks[-1]], [30])[0]
    assert torch.isfinite(a).all()


def test_stop_strings_and_seeded_sampling(tiny_llama_path):
    r = Runner(tiny_llama_path, RunnerOptions(num_ctx=128, device="cpu"))
    try:
        p = _prompt()
        base = list(r.completion(CompletionRequest(prompt=p, sampling=SamplingParams(temperature=0), num_predict=8)))
        toks = [t for c in base for t in c.tokens]
        stop = f"<t{toks[3]}>"
        out = list(r.completion(CompletionRequest(prompt=p, sampling=SamplingParams(temperature=0), num_predict=8, stop=[stop])))
        text = "".join(c.content for c in out)
        assert out[-1].done_reason == "stop" and stop not in text and text == "".join(f"<t{t}>" for t in toks[:3])
        sp = SamplingParams(temperature=1.0, seed=42)
        a = [t for c in r.completion(CompletionRequest(prompt=p, sampling=sp, num_predict=8)) for t in c.tokens]
        b = [t for c in r.completion(CompletionRequest(prompt=p, sampling=sp, num_predict=8)) for t in c.tokens]
        assert a == b
    finally:
        r.close()


def _tokens(r, n, prompt=None, **kw):
    out = list(r.completion(CompletionRequest(prompt=prompt or _prompt(), sampling=SamplingParams(temperature=0), num_predict=n, ignore_eos=True, **kw)))
    return [t for c in out for t in c.tokens], out[-1]


def test_speculative_decoding_keeps_the_greedy_tokens(tiny_llama_path, tiny_llama_q8_path):
    """A draft model (Modelfile DRAFT) only changes how fast tokens appear: the target's greedy sequence stays the same,
    whether the draft agrees always (the same weights), mostly (their Q8_0 copy) or the context has to shift."""
    plain = Runner(tiny_llama_path, RunnerOptions(num_ctx=512, device="cpu"))
    want, fin = _tokens(plain, 41)
    plain.close()
    assert len(want) == 41 and fin.done_reason == "length"
    for draft, k in ((tiny_llama_path, 4), (tiny_llama_q8_path, 3), (tiny_llama_q8_path, 7)):
        r = Runner(tiny_llama_path, RunnerOptions(num_ctx=512, device="cpu", draft_path=draft, draft_num_predict=k))
        try:
            assert r.draft is not None
            got, fin = _tokens(r, 41)
            assert got == want and fin.eval_count == 41 and fin.done_reason == "length", (draft, k)
            st = r.stats
            assert st["draft_tokens"] > 0 and 0 < st["draft_accepted_tokens"] <= st["draft_tokens"]
            assert st["decode_steps"] < 40                       # several tokens per step
            if draft == tiny_llama_path:
                assert st["draft_accepted_tokens"] == st["draft_tokens"]
            # a second request on the same slot (prefix reuse on the target, draft cache rebuilt) and a stop string
            again, _ = _tokens(r, 9)
            assert again == want[:9]
            stop_at = f"<t{want[5]}>"
            out = list(r.completion(CompletionRequest(prompt=_prompt(), sampling=SamplingParams(temperature=0), num_predict=30, stop=[stop_at])))
            assert out[-1].done_reason == "stop" and stop_at not in "".join(c.content for c in out)
        finally:
            r.close()
    # sampling with a temperature, or two sequences at once, take the ordinary step
    r = Runner(tiny_llama_path, RunnerOptions(num_ctx=512, device="cpu", draft_path=tiny_llama_q8_path))
    try:
        list(r.completion(CompletionRequest(prompt=_prompt(), sampling=SamplingParams(temperature=0.8, seed=1), num_predict=6)))
        assert r.stats["draft_tokens"] == 0
    finally:
        r.close()
    # a full context: speculation stops short of the end, the shift rebuilds both caches, the tokens equal the plain run
    outs = []
    for draft in ("", tiny_llama_q8_path):
        r = Runner(tiny_llama_path, RunnerOptions(num_ctx=32, device="cpu", draft_path=draft))
        try:
            outs.append(_tokens(r, 40)[0])
            if draft:
                assert r.stats["context_shifts"] >= 1 and r.stats["draft_accepted_tokens"] > 0
        finally:
            r.close()
    assert outs[0] == outs[1] and len(outs[0]) == 40


def _write_adapter(path, base_gguf, names, rank=4, alpha=8.0, seed=0):
    """A LoRA adapter GGUF for ``names`` of the base model: random A [r, in] and B [out, r]."""
    from ollama_b200.gguf.types import GGMLType
    from ollama_b200.gguf.writer import WriteTensor, write_gguf
    g = torch.Generator().manual_seed(seed)
    tensors, deltas = [], {}
    for n in names:
        out_dim, in_dim = base_gguf.tensors[n].torch_shape
        a = torch.randn(rank, in_dim, generator=g) * 0.05
        b = torch.randn(out_dim, rank, generator=g) * 0.05
        deltas[n] = (b @ a) * (alpha / rank)
        tensors.append(WriteTensor(n + ".lora_a", (in_dim, rank), GGMLType.F32, a.numpy().tobytes()))
        tensors.append(WriteTensor(n + ".lora_b", (rank, out_dim), GGMLType.F32, b.numpy().tobytes()))
    write_gguf(path, {"general.architecture": "llama", "general.type": "adapter", "adapter.type": "lora", "adapter.lora.alpha": alpha}, tensors)
    return deltas


def test_lora_adapter_is_merged_at_load(tmp_path, tiny_llama_q8_path):
    """Modelfile ADAPTER: the low-rank update lands in the matrices it names (kept as F16), the rest keeps its encoding,
    and the runner's tokens are those of a model whose weights were updated by hand."""
    from ollama_b200.engine.backend import TorchBackend, open_model
    from ollama_b200.gguf.types import GGMLType
    from ollama_b200.models.lora import LoraError, LoraTensors
    g = open_model(tiny_llama_q8_path)
    names = ["blk.0.attn_q.weight", "blk.1.attn_v.weight", "blk.1.ffn_down.weight"]
    ad = str(tmp_path / "adapter.gguf")
    deltas = _write_adapter(ad, g, names)
    src = LoraTensors(g, [ad])
    plain = TorchBackend(g, "cpu")
    for n in names:
        w = src[n]
        assert w.dtype == GGMLType.F16 and src.type_of(n) == GGMLType.F16
        assert torch.allclose(w.dequant(), plain.weights[n].dequant() + deltas[n], atol=2e-3)
    assert src["blk.0.attn_k.weight"].dtype == GGMLType.Q8_0 and src.type_of("blk.0.attn_norm.weight") == GGMLType.F32
    src.close()
    be = TorchBackend(g, "cpu", adapters=[ad])
    plain.alloc(1, 64)
    be.alloc(1, 64)
    prompt = _prompt()
    la, lb = plain.prefill(0, prompt, 0), be.prefill(0, prompt, 0)
    assert (la - lb).abs().max().item() > 1e-3                       # the adapter changes the model ...
    for n in names:                                                  # ... exactly like editing the weights by hand
        plain.weights[n] = type(plain.weights[n]).from_float(n, plain.weights[n].dequant() + deltas[n], GGMLType.F16)
    from ollama_b200.models.reference import ReferenceModel
    plain.model = ReferenceModel(plain.cfg, plain.weights, "cpu")
    plain.alloc(1, 64)
    assert torch.allclose(plain.prefill(0, prompt, 0), lb, atol=1e-4)
    r = Runner(tiny_llama_q8_path, RunnerOptions(num_ctx=128, device="cpu", adapter_paths=(ad,)))
    try:
        toks, _ = _tokens(r, 6)
        assert toks[0] == int(lb.argmax())
    finally:
        r.close()
    # an adapter for another model is refused
    bad = str(tmp_path / "bad.gguf")
    from ollama_b200.gguf.writer import WriteTensor, write_gguf
    write_gguf(bad, {"general.architecture": "llama", "general.type": "adapter", "adapter.type": "lora", "adapter.lora.alpha": 1.0},
               [WriteTensor("blk.9.attn_q.weight.lora_a", (8, 2), GGMLType.F32, bytes(64)), WriteTensor("blk.9.attn_q.weight.lora_b", (2, 8), GGMLType.F32, bytes(64))])
    with pytest.raises(LoraError):
        LoraTensors(g, [bad])
    g.close()


def test_grammar_waits_for_the_end_of_the_reasoning_block(tiny_llama_path):
    """Structured output of a reasoning model: tokens are free until ``grammar_after`` has been generated, then the
    grammar constrains the answer and ends the request when it is complete."""
    r = Runner(tiny_llama_path, RunnerOptions(num_ctx=256, device="cpu"))
    try:
        free, _ = _tokens(r, 8)
        marker = r.tokenizer.decode(free[3:4])
        assert marker.startswith("<t")
        req = CompletionRequest(prompt=_prompt(), sampling=SamplingParams(temperature=0), num_predict=32, cache_prompt=False,
                                grammar='root ::= "<t300>" "<t301>"', grammar_after=marker)
        out = list(r.completion(req))
        toks = [t for c in out for t in c.tokens]
        text = "".join(c.content for c in out)
        assert toks[:4] == free[:4] and out[-1].done_reason == "stop"
        assert text == r.tokenizer.decode(free[:4]) + "<t300><t301>"          # spelled with whatever tokens the model prefers
        # without the gate the grammar applies from the first token
        req = CompletionRequest(prompt=_prompt(), sampling=SamplingParams(temperature=0), num_predict=32, cache_prompt=False,
                                grammar='root ::= "<t300>" "<t301>"')
        assert "".join(c.content for c in r.completion(req)) == "<t300><t301>"
    finally:
        r.close()


def test_concurrent_random_requests_neither_fail_nor_stall(tiny_llama_path):
    """Three client threads submit requests with random sampling settings, stop strings, grammars, cancellations, context
    shifts and embeddings against three slots: every request ends, none with an error, and the runner stays healthy."""
    import random
    import threading
    r = Runner(tiny_llama_path, RunnerOptions(num_ctx=96, num_parallel=3, device="cpu", num_batch=16))
    errs, done = [], [0]

    def worker(seed):
        rr = random.Random(seed)
        for _ in range(5):
            prompt = [rr.randint(259, 31999) for _ in range(rr.randint(1, 90))]
            sp = SamplingParams(temperature=rr.choice([0, 0.8]), seed=rr.randint(0, 99), top_k=rr.choice([1, 40]), repeat_penalty=rr.choice([1.0, 1.2]),
                                logprobs=rr.random() < 0.2, top_logprobs=2)
            req = CompletionRequest(prompt=prompt, sampling=sp, num_predict=rr.choice([1, 5, 30, 120]), stop=rr.choice([[], ["<t5"], ["a"]]),
                                    grammar=rr.choice([None, None, 'root ::= "<t300>" ("<t301>")*']), shift=rr.random() < 0.7,
                                    cache_prompt=rr.random() < 0.7, embedding=rr.random() < 0.1, ignore_eos=rr.random() < 0.5)
            seq = r.submit(req)
            cancel_at, k = rr.choice([None, None, 1, 3]), 0
            while True:
                try:
                    ch = seq.out.get(timeout=60)
                except Exception:
                    errs.append(("stalled", seed))
                    return
                k += 1
                if ch.error:
                    errs.append(ch.error)
                if ch.done or ch.error:
                    break
                if cancel_at and k >= cancel_at:
                    seq.cancelled, cancel_at = True, None
            done[0] += 1

    ths = [threading.Thread(target=worker, args=(s,)) for s in range(3)]
    try:
        for t in ths:
            t.start()
        for t in ths:
            t.join(timeout=240)
        assert not errs and done[0] == 15 and not any(t.is_alive() for t in ths) and r.ping()
    finally:
        r.close()


def test_vision_language_checkpoint_runs_as_its_text_model(tmp_path):
    """llama/compat/llama-ollama-compat.cpp:1776-1868: a qwen3vl blob (keys under ``qwen3vl.``, vision tensors embedded) is loaded
    as qwen3; text-only prompts give the tokens of the plain qwen3 file with the same weights, and the model still reports vision."""
    import numpy as np

    from ollama_b200.gguf.reader import open_gguf
    from ollama_b200.gguf.writer import WriteTensor, write_gguf
    from ollama_b200.models.synth import write_synthetic_gguf
    plain, vl = str(tmp_path / "q3.gguf"), str(tmp_path / "q3vl.gguf")
    write_synthetic_gguf(plain, "tiny-qwen3", "F32")
    g = open_gguf(plain)
    kv = {}
    for k, v in g.kv.items():
        kv["qwen3vl." + k[len("qwen3."):] if k.startswith("qwen3.") else k] = v
    kv["general.architecture"] = "qwen3vl"
    kv["qwen3vl.vision.block_count"] = 2
    kv["qwen3vl.rope.dimension_sections"] = [24, 20, 20, 0]
    tensors = [WriteTensor(n, tuple(t.shape), t.dtype, np.array(g.tensor_bytes(n))) for n, t in g.tensors.items()]
    f32 = g.tensors["output_norm.weight"].dtype
    tensors.append(WriteTensor("v.patch_embd.weight", (4, 4), f32, np.zeros(16, dtype=np.float32).view(np.uint8)))
    tensors.append(WriteTensor("mm.0.weight", (4, 4), f32, np.zeros(16, dtype=np.float32).view(np.uint8)))
    write_gguf(vl, kv, tensors)
    out = []
    for path in (plain, vl):
        r = Runner(path, RunnerOptions(num_ctx=64, device="cpu"))
        try:
            out.append(_tokens(r, 6, prompt=list(range(300, 316)))[0])
            if path == vl:
                assert r.backend.cfg.arch == "qwen3"
        finally:
            r.close()
    assert out[0] == out[1] and len(out[0]) == 6


def test_mistral3_blob_runs_on_the_llama_decoder(tmp_path):
    """llama/compat/llama-ollama-compat.cpp:1643-1665: a mistral3 blob (keys under ``mistral3.``, YaRN betas under their older
    names, no pre-tokenizer id, vision tensors embedded) is loaded as the llama decoder it is; the tokens equal those of the plain
    llama file with the same weights, the pre-tokenizer defaults to tekken and the YaRN keys are found under their current names."""
    import numpy as np

    from ollama_b200.engine.backend import open_model
    from ollama_b200.gguf.reader import open_gguf
    from ollama_b200.gguf.writer import WriteTensor, write_gguf
    from ollama_b200.models.synth import write_synthetic_gguf
    from ollama_b200.text.tokenizer import PRETOKENIZERS
    plain, m3 = str(tmp_path / "l.gguf"), str(tmp_path / "m3.gguf")
    write_synthetic_gguf(plain, "tiny-llama", "F32")
    g = open_gguf(plain)
    kv = {}
    for k, v in g.kv.items():
        kv["mistral3." + k[len("llama."):] if k.startswith("llama.") else k] = v
    kv["general.architecture"] = "mistral3"
    kv["mistral3.rope.scaling.beta_fast"] = 32.0
    kv["mistral3.rope.scaling.beta_slow"] = 1.0
    kv.pop("tokenizer.ggml.pre", None)
    tensors = [WriteTensor(n, tuple(t.shape), t.dtype, np.array(g.tensor_bytes(n))) for n, t in g.tensors.items()]
    f32 = g.tensors["output_norm.weight"].dtype
    tensors.append(WriteTensor("v.patch_conv.weight", (4, 4), f32, np.zeros(16, dtype=np.float32).view(np.uint8)))
    write_gguf(m3, kv, tensors)
    gm = open_model(m3)
    assert gm.architecture == "llama" and gm.kv["tokenizer.ggml.pre"] == "tekken" and gm.kv["llama.rope.scaling.yarn_beta_fast"] == 32.0
    assert not gm.has("v.patch_conv.weight")
    import regex
    pieces = [m.group(0) for m in regex.compile(PRETOKENIZERS["tekken"][0]).finditer("Hello WORLD don't 1234\n\n x")]
    assert pieces == ["Hello", " WORLD", " don", "'t", " ", "1", "2", "3", "4", "\n\n", " x"]
    out = []
    for path in (plain, m3):
        r = Runner(path, RunnerOptions(num_ctx=64, device="cpu"))
        try:
            out.append(_tokens(r, 6, prompt=list(range(300, 316)))[0])
        finally:
            r.close()
    assert out[0] == out[1]
