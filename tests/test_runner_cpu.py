"""CPU plumbing: tiny llama (2 layers, d 256, 4/2 heads, FFN 688, vocab 32000) through the runner."""
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
