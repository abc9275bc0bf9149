"""Layer pipeline (consecutive blocks on consecutive GPUs): the split on CPU, the stages against the single-device engine on a GPU."""
import pytest
import torch

from ollama_b200.engine.pipeline import split_layers


def test_split_layers_covers_every_layer_once():
    assert split_layers(32, 4) == [(0, 8), (8, 16), (16, 24), (24, 32)]
    assert split_layers(6, 4) == [(0, 2), (2, 4), (4, 5), (5, 6)]          # the remainder goes to the earlier stages
    assert split_layers(80, 3) == [(0, 27), (27, 54), (54, 80)]
    for n, s, w in ((62, 8, None), (10, 3, (1.0, 5.0, 1.0)), (7, 7, None), (9, 2, (0.0, 1.0))):
        r = split_layers(n, s, w)
        assert r[0][0] == 0 and r[-1][1] == n and all(a[1] == b[0] for a, b in zip(r, r[1:])) and all(hi > lo for lo, hi in r)
    assert split_layers(10, 3, (1.0, 5.0, 1.0)) == [(0, 2), (2, 9), (9, 10)]   # more free memory, more layers
    with pytest.raises(ValueError):
        split_layers(3, 4)
    with pytest.raises(ValueError):
        split_layers(8, 2, (1.0,))


def _check_pipeline(tmp_path, devices, spec, ft):
    from ollama_b200.engine.b200 import B200Backend
    from ollama_b200.engine.backend import open_model
    from ollama_b200.engine.pipeline import PipelineBackend
    from ollama_b200.models.synth import write_synthetic_gguf
    p = str(tmp_path / "m.gguf")
    write_synthetic_gguf(p, spec, ft)
    g = open_model(p)
    one, pp = B200Backend(g, "cuda:0"), PipelineBackend(g, devices)
    assert [s.l_lo for s in pp.stages] == [r[0] for r in pp.ranges] and pp.stages[0].head is None and pp.stages[-1].head is not None
    one.alloc(2, 128)
    pp.alloc(2, 128)
    assert pp.kv_bytes() == one.kv_bytes()
    prompt = torch.randint(259, 4096, (70,), generator=torch.Generator().manual_seed(4)).tolist()
    one.prefill(1, prompt[:40], 0, need_logits=False)
    pp.prefill(1, prompt[:40], 0, need_logits=False)          # two chunks: the second one attends to the first one's cache rows
    la, lb = one.prefill(1, prompt[40:], 40).cpu(), pp.prefill(1, prompt[40:], 40).cpu()
    assert torch.allclose(la, lb, atol=1e-4 * la.abs().max().item() + 1e-5)
    tok = int(la.argmax())
    for step in range(5):        # eager, then graph capture, then replays
        pos = len(prompt) + step
        da, db = one.decode([1], [tok], [pos])[0].cpu(), pp.decode([1], [tok], [pos])[0].cpu()
        assert torch.allclose(da, db, atol=1e-4 * da.abs().max().item() + 1e-5), step
        tok = int(da.argmax())
    pos = len(prompt) + 5
    assert pp.decode_argmax([1, 0], [tok, 7], [pos, 0]) == one.decode_argmax([1, 0], [tok, 7], [pos, 0])
    la = one.decode_loop([1, 0], [tok, 7], [pos + 1, 1], 6).cpu()
    lb = pp.decode_loop([1, 0], [tok, 7], [pos + 1, 1], 6).cpu()        # ids fed back on the device, stage to stage
    assert torch.equal(la, lb)
    h1, h2 = one.hidden(0, prompt[:9]).cpu(), pp.hidden(0, prompt[:9]).cpu()
    assert torch.allclose(h1, h2, atol=1e-4 * h1.abs().max().item() + 1e-5)
    pp.close()


@pytest.mark.gpu
@pytest.mark.parametrize("spec,ft,stages", [("tiny-gemma3", "Q8_0", 3), ("tiny-qwen3", "Q4_K_M", 2), ("tiny-gpt-oss", "MXFP4", 2)])
def test_pipeline_stages_on_one_device_match_the_whole_model(tmp_path, spec, ft, stages):
    """All stages on GPU 0: the layer ranges, the hand-over of the residual stream and the per-stage graphs."""
    _check_pipeline(tmp_path, [0] * stages, spec, ft)


@pytest.mark.gpu
def test_pipeline_over_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _check_pipeline(tmp_path, [0, 1], "tiny-gemma3", "Q8_0")


@pytest.mark.gpu
def test_runner_falls_back_to_the_pipeline(tmp_path, monkeypatch):
    """A sandwich-norm model is not taken by the tensor-parallel engine: B200_PP (or a refused B200_TP) selects the pipeline."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from ollama_b200.engine.runner import CompletionRequest, Runner, RunnerOptions
    from ollama_b200.engine.sampler import SamplingParams
    from ollama_b200.models.synth import write_synthetic_gguf
    p = str(tmp_path / "m.gguf")
    write_synthetic_gguf(p, "tiny-gemma3", "Q8_0")
    outs = []
    for tp in (1, 2):
        r = Runner(p, RunnerOptions(num_ctx=256, device="cuda", tp=tp))
        try:
            assert r.backend.name == ("b200-pp" if tp == 2 else "b200") and r._tp_group is None
            seq = r.submit(CompletionRequest(prompt=list(range(300, 330)), sampling=SamplingParams(temperature=0), num_predict=8, ignore_eos=True))
            toks = []
            while True:
                ch = seq.out.get(timeout=120)
                assert not ch.error, ch.error
                toks += ch.tokens
                if ch.done:
                    break
            outs.append(toks)
        finally:
            r.close()
    assert len(outs[0]) == 8 and outs[0] == outs[1]


@pytest.mark.gpu
def test_runner_on_the_gpu_the_scheduler_chose(tmp_path):
    """A single-GPU model placed on a GPU other than the first one: weights, caches and kernel launches all land there,
    and a tensor-parallel group uses the listed devices in the listed order."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from ollama_b200.engine.runner import CompletionRequest, Runner, RunnerOptions
    from ollama_b200.engine.sampler import SamplingParams
    from ollama_b200.models.synth import write_synthetic_gguf
    p = str(tmp_path / "m.gguf")
    write_synthetic_gguf(p, "tiny-tp", "Q8_0")
    prompt = list(range(300, 340))
    outs = []
    for opts in (dict(device="cuda:0"), dict(device="cuda:1", gpu_ids=(1,)), dict(device="cuda", tp=2, gpu_ids=(1, 0))):
        before = [torch.cuda.memory_allocated(i) for i in range(2)]
        r = Runner(p, RunnerOptions(num_ctx=256, **opts))
        try:
            if opts.get("tp"):
                assert r._tp_group is not None and str(r.backend.device) == "cuda:1"
            else:
                assert str(r.backend.device) == opts["device"]
                other = 1 - int(opts["device"][-1])
                assert torch.cuda.memory_allocated(other) <= before[other]          # nothing was placed on the other GPU
            seq = r.submit(CompletionRequest(prompt=prompt, sampling=SamplingParams(temperature=0.7, seed=3, top_k=20), num_predict=10, ignore_eos=True))
            toks = []
            while True:
                ch = seq.out.get(timeout=120)
                assert not ch.error, ch.error
                toks += ch.tokens
                if ch.done:
                    break
            outs.append(toks)
        finally:
            r.close()
    assert len(outs[0]) == 10 and outs[0] == outs[1]
    assert len(outs[2]) == 10
