"""Self-check of the tensor-parallel engine against the single-GPU engine on a small random model.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 --master-port 29541 \
        -m ollama_b200.parallel.selftest [--model tiny-tp] [--quant Q4_K_M] [--prompt 300] [--steps 6]

Every rank builds the full model on its own GPU (reference) and its shard of the tensor-parallel model, runs
a prefill and a few greedy decode steps through both (eager, then CUDA-graph replay) and compares logits.
Rank 0 prints one JSON line; the exit code is non-zero on a mismatch or when a bounded wait ran out.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist


def run_selfcheck(rank: int, world: int, dev: str, model: str = "tiny-tp", quant: str = "Q4_K_M", prompt: int = 300, steps: int = 6,
                  slots: int = 2) -> dict:
    """Compare the tensor-parallel engine with the single-GPU engine inside an initialised process group; every rank calls it.

    Returns the result record (``ok`` is the group's verdict: no rank saw a mismatch or a wait that ran out)."""
    from ..engine.b200 import B200Backend
    from ..models.config import config_from_gguf
    from ..models.synth import SyntheticTensors, synthetic_header
    from ..ops import cuda as K
    from .tp_engine import TPBackend

    cfg = config_from_gguf(synthetic_header(model, quant))
    src = SyntheticTensors(model, quant, seed=0, device=dev)
    ref = B200Backend(None, device=dev, cfg=cfg, tensors=src)
    tp = TPBackend(cfg, src, device=dev, rank=rank, world=world)
    ctx = max(512, prompt + 64)
    ref.alloc(slots, ctx)
    tp.alloc(slots, ctx)
    res = {"world": world, "model": model, "quant": quant}
    ok = True
    gen = torch.Generator().manual_seed(7)
    for graphs in (False, True):
        ref.use_graphs = tp.use_graphs = graphs
        prompts = torch.randint(0, cfg.vocab_size, (slots, prompt), generator=gen)
        toks, errs = [], []
        for s in range(slots):
            lr, lt = ref.prefill(s, prompts[s].tolist(), 0), tp.prefill(s, prompts[s].tolist(), 0)
            errs.append(((lr - lt).abs().max() / lr.abs().max()).item())
            toks.append(int(lr.argmax()))
        sl = list(range(slots))
        for step in range(steps):
            pos = [prompt + step] * slots
            lr, lt = ref.decode(sl, toks, pos), tp.decode(sl, toks, pos)
            errs.append(((lr - lt).abs().max() / lr.abs().max()).item())
            toks = lr.argmax(-1).tolist()
        a = ref.decode_argmax(sl, toks, [prompt + steps] * slots)
        b = tp.decode_argmax(sl, toks, [prompt + steps] * slots)
        res[f"max_rel_err_graphs_{int(graphs)}"] = max(errs)
        res[f"argmax_equal_graphs_{int(graphs)}"] = a == b
        ok = ok and max(errs) < 0.05
    res["comm_status"] = tp.comm_status()
    res["gemm_status"] = K.gemm_status()
    ok = ok and res["comm_status"] == 0 and res["gemm_status"] == 0
    flag = torch.tensor([0 if ok else 1], device=dev)
    dist.all_reduce(flag)
    res["ok"] = flag.item() == 0
    tp.close()
    ref.close()
    return res


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="tiny-tp")
    ap.add_argument("--quant", default="Q4_K_M")
    ap.add_argument("--prompt", type=int, default=300)
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--slots", type=int, default=2)
    args = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    dist.init_process_group("nccl", device_id=torch.device(dev))
    res = run_selfcheck(rank, world, dev, args.model, args.quant, args.prompt, args.steps, args.slots)
    if rank == 0:
        print(json.dumps(res), flush=True)
    dist.destroy_process_group()
    return 0 if res["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
