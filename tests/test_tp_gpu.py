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
