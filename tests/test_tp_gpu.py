"""Tensor-parallel engine on 2 (and 4) GPUs of one box: child processes under torch.distributed.run."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(world: int, port: int, *extra: str) -> dict:
    env = dict(os.environ, PYTHONPATH=ROOT, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), "-m", "ollama_b200.parallel.selftest", *extra]
    p = subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=600)
    lines = [ln for ln in p.stdout.splitlines() if ln.startswith("{")]
    assert p.returncode == 0 and lines, p.stdout[-2000:] + p.stderr[-4000:]
    return json.loads(lines[-1])


@pytest.mark.parametrize("world,model,quant", [(2, "tiny-tp", "Q4_K_M"), (2, "tiny-qwen3moe", "Q8_0"), (2, "tiny-gpt-oss", "MXFP4"),
                                               (4, "tiny-tp", "Q8_0"), (8, "tiny-tp", "Q8_0")])
def test_tp_matches_single_gpu(world, model, quant):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    res = _run(world, 29540 + world, "--model", model, "--quant", quant)
    assert res["ok"] and res["comm_status"] == 0


def test_runner_leads_a_spawned_group(tmp_path):
    """The public runner with tp=2: followers are spawned per GPU, connected by pipes, and the tokens equal the single-GPU run."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from ollama_b200.engine.runner import CompletionRequest, Runner, RunnerOptions
    from ollama_b200.engine.sampler import SamplingParams
    from ollama_b200.models.synth import write_synthetic_gguf
    p = str(tmp_path / "m.gguf")
    write_synthetic_gguf(p, "tiny-tp", "Q8_0")
    prompt = torch.randint(259, 4000, (40,), generator=torch.Generator().manual_seed(2)).tolist()
    outs = []
    for tp in (1, 2):
        r = Runner(p, RunnerOptions(num_ctx=256, num_parallel=2, device="cuda", tp=tp))
        try:
            assert (r._tp_group is not None) == (tp == 2)
            seq = r.submit(CompletionRequest(prompt=prompt, sampling=SamplingParams(temperature=0), num_predict=12, ignore_eos=True))
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
    assert len(outs[0]) == 12 and outs[0] == outs[1]
