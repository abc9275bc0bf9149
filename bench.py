"""Headline benchmark: decode tok/s + prompt-eval tok/s (+ p50 TTFT) on a random-init GGUF-architecture model.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--model NAME] [--slots S]

N = 1 runs Llama-3.1-8B-architecture Q4_K_M (512-token random prompt, 128 generated tokens, greedy,
num_ctx 8192); N >= 2 runs Llama-3.1-70B-architecture Q4_K_M tensor-parallel over N GPUs (2048-token
prompt, 256 generated tokens).  One *step* is one request epoch on every slot: prefill of a fresh
random prompt followed by the whole generation.  Timing is on the device with CUDA events, max over
ranks; weights (GBs) are far larger than L2, so no flush is needed between iterations.

The line printed by rank 0 follows the driver contract; ``value`` is the decode rate of the whole job,
``prompt_eval_tok_s`` / ``ttft_ms_p50`` ride along, and ``e2e`` is the same workload through the public
runner API (pinned host->device copies of the inputs and a device->host read of every sampled token
inside the timed region).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

WORKLOADS = {
    "llama-3.1-8b": dict(prompt=512, gen=128, ctx=8192, ft="Q4_K_M"),
    "llama-3.1-70b": dict(prompt=2048, gen=256, ctx=8192, ft="Q4_K_M"),
    "gpt-oss-120b": dict(prompt=1024, gen=256, ctx=8192, ft="MXFP4", slots=16),
    "qwen3-235b-a22b": dict(prompt=8192, gen=512, ctx=32768, ft="Q4_K_M", slots=32),
    "tiny-qwen3": dict(prompt=64, gen=32, ctx=512, ft="Q4_K_M"),
    "tiny-qwen3moe": dict(prompt=64, gen=32, ctx=512, ft="Q8_0"),
}
PREFILL_CHUNK = 2048


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.rows: list[list[str]] = []
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        rows = [r for r in self.rows if len(r) >= 9]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        def num(x):
            try:
                return float(x)
            except ValueError:
                return None
        power = [num(r[3]) or 0.0 for r in rows]
        hi = max(power)
        load = [r for r, p in zip(rows, power) if p >= 0.6 * hi] or rows
        sm = [num(r[1]) for r in load if num(r[1]) is not None]
        reasons = set()
        for r in load:
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
                if r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": num(rows[0][2]), "reasons": sorted(reasons),
                "power_w_max": hi, "samples": len(rows)}


def reference_arm(args) -> None:
    why = ("the reference is a Go program that drives an externally fetched llama.cpp build; this image has no Go toolchain and "
           "no network, and a pip install of the reference tree fails (no setup.py / pyproject.toml)")
    print(json.dumps({"impl": "reference", "unavailable": why}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--model", default="auto")
    ap.add_argument("--slots", type=int, default=0, help="parallel sequences (0 = the workload's default)")
    ap.add_argument("--prompt", type=int, default=0)
    ap.add_argument("--gen", type=int, default=0)
    ap.add_argument("--ctx", type=int, default=0)
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--no-pdl", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--parallelism", default="tp", choices=["tp", "pp"],
                    help="N > 1: tp = tensor/expert parallel ranks (default), pp = layer pipeline driven by rank 0 (the reference's multi-GPU mode)")
    ap.add_argument("--kv-type", default="f16", choices=["f16", "q8_0"], help="K/V cache encoding (OLLAMA_KV_CACHE_TYPE)")
    ap.add_argument("--layers", type=int, default=0, help="truncate the model to this many layers (profiling only; not a benchmark number)")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    pp_gpus = 0
    if args.parallelism == "pp" and max(world, args.gpus) > 1:
        # a layer pipeline is driven by one process: the other launched ranks leave at once, without touching a GPU
        # (a rank parked in a collective would occupy the very GPU that the driving process needs)
        if rank != 0:
            return
        pp_gpus, world = max(world, args.gpus), 1
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    n_gpus = pp_gpus or max(world, 1)
    if args.gpus != n_gpus and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE={world}", file=sys.stderr)

    model = args.model if args.model != "auto" else ("llama-3.1-8b" if n_gpus == 1 else "llama-3.1-70b")
    wl = dict(WORKLOADS[model])
    for k in ("prompt", "gen", "ctx"):
        if getattr(args, k):
            wl[k] = getattr(args, k)
    slots = args.slots if args.slots > 0 else wl.get("slots", 1)

    from ollama_b200.engine.runner import CompletionRequest, Runner, RunnerOptions
    from ollama_b200.engine.sampler import SamplingParams
    from ollama_b200.models.config import config_from_gguf
    from ollama_b200.models.synth import SyntheticTensors, synthetic_header

    dev = f"cuda:{local}"
    if args.layers:      # profiling aid: a truncated stack keeps ncu captures short; the result is flagged below
        import dataclasses
        from ollama_b200.models import synth
        synth.SPECS[model] = dataclasses.replace(synth.SPECS[model], n_layers=args.layers)
    hdr = synthetic_header(model, wl["ft"])
    cfg = config_from_gguf(hdr)
    t_load = time.time()
    pp = pp_gpus > 1
    if pp:
        from ollama_b200.engine.pipeline import PipelineBackend
        be = PipelineBackend(None, list(range(n_gpus)), cfg=cfg, tensors=lambda d: SyntheticTensors(model, wl["ft"], seed=0, device=str(d)),
                             kv_type=args.kv_type)
    elif n_gpus == 1:
        from ollama_b200.engine.b200 import B200Backend
        be = B200Backend(None, device=dev, cfg=cfg, tensors=SyntheticTensors(model, wl["ft"], seed=0, device=dev), kv_type=args.kv_type)
    else:
        from ollama_b200.parallel.tp_engine import TPBackend
        be = TPBackend(cfg, SyntheticTensors(model, wl["ft"], seed=0, device=dev), device=dev, rank=rank, world=world, kv_type=args.kv_type)
    for part in (be.stages if pp else [be]):
        part.use_graphs = not args.no_graphs
        part.pdl = not args.no_pdl
    be.alloc(slots, wl["ctx"])
    torch.cuda.synchronize()
    t_load = time.time() - t_load

    P, G = wl["prompt"], wl["gen"]
    gen = torch.Generator().manual_seed(1234)
    slot_ids = list(range(slots))

    def sync_stages():
        """Pipeline: the events live on the first device, so the work of the later stages is waited for before each record."""
        if pp:
            for d in be.devices:
                torch.cuda.synchronize(d)

    def epoch(timed: bool):
        """One request epoch, device-only: returns (prefill_ms, decode_ms)."""
        prompts = torch.randint(0, cfg.vocab_size, (slots, P), generator=gen)   # fresh ids every epoch: no prefix reuse
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        firsts = []
        for s in slot_ids:
            toks = prompts[s].tolist()
            for c0 in range(0, P, PREFILL_CHUNK):
                logits = be.prefill(s, toks[c0:c0 + PREFILL_CHUNK], c0, need_logits=c0 + PREFILL_CHUNK >= P)
            firsts.append(logits.argmax())
        first = torch.stack(firsts).to(torch.int32)
        sync_stages()
        e1.record()
        toks = be.decode_loop(slot_ids, [0] * slots, [P] * slots, G - 1, first_tokens=first)
        sync_stages()
        e2.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1), e1.elapsed_time(e2), toks

    for _ in range(max(args.warmup, 3)):
        epoch(False)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local).start() if rank == 0 else None
    launches0 = be.kernel_launches
    pre_ms, dec_ms = [], []
    for _ in range(args.steps):
        a, b, _ = epoch(True)
        pre_ms.append(a)
        dec_ms.append(b)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    launches = be.kernel_launches - launches0
    if world > 1:   # max over ranks
        t = torch.tensor([sum(pre_ms), sum(dec_ms)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        tot_pre, tot_dec = t.tolist()
    else:
        tot_pre, tot_dec = sum(pre_ms), sum(dec_ms)
    decode_tok_s = slots * (G - 1) * args.steps / (tot_dec / 1e3)
    prefill_tok_s = slots * P * args.steps / (tot_pre / 1e3)
    ttft_p50 = statistics.median(pre_ms) / slots

    # ---- end to end through the public runner API --------------------------------------------------
    e2e = None
    runner_be = be
    if not args.no_e2e and n_gpus > 1 and not pp:
        # the serving stack runs in rank 0 only; the other ranks repeat its backend calls until it closes the group
        from ollama_b200.parallel.control import TPControl, TPLeader, follow
        ctl = TPControl(rank, world)
        if rank == 0:
            runner_be = TPLeader(be, ctl)
        else:
            follow(be, ctl)
    if not args.no_e2e and rank == 0:
        r = Runner(None, RunnerOptions(num_ctx=wl["ctx"], num_parallel=slots, device=dev, num_batch=min(max(P, 512), PREFILL_CHUNK)), backend=runner_be)
        r.n_ctx = wl["ctx"]
        sp = SamplingParams(temperature=0)
        def one_epoch():
            prompts = torch.randint(0, cfg.vocab_size, (slots, P), generator=gen).tolist()
            seqs = [r.submit(CompletionRequest(prompt=p, sampling=sp, num_predict=G, ignore_eos=True, cache_prompt=False)) for p in prompts]
            t0 = time.perf_counter()
            ttfts, finals = [], []
            for s in seqs:
                got_first = False
                while True:
                    ch = s.out.get()
                    if ch.error:
                        raise RuntimeError(ch.error)
                    if not got_first and ch.tokens:
                        ttfts.append(time.perf_counter() - t0)
                        got_first = True
                    if ch.done:
                        finals.append(ch)
                        break
            return ttfts, finals
        for _ in range(2):
            one_epoch()
        h0, d0 = be.h2d_bytes, be.d2h_bytes
        ev_n = ev_t = pe_n = pe_t = 0.0
        tt = []
        for _ in range(args.steps):
            ttfts, finals = one_epoch()
            tt += ttfts
            # all slots decode in the same batched steps: the epoch's decode time is the longest slot's
            ev_n += sum(f.eval_count - 1 for f in finals)
            ev_t += max(f.eval_duration for f in finals)
            pe_n += sum(f.prompt_eval_count for f in finals)
            pe_t += sum(f.prompt_eval_duration for f in finals)
        e2e = {"value": round(ev_n / ev_t, 2), "unit": "tok/s", "prompt_eval_tok_s": round(pe_n / pe_t, 1),
               "ttft_ms_p50": round(statistics.median(tt) * 1e3, 2),
               "h2d_bytes_per_step": (be.h2d_bytes - h0) // args.steps, "d2h_bytes_per_step": (be.d2h_bytes - d0) // args.steps,
               "api": "ollama_b200.engine.runner.Runner.submit/completion"}
        r.close()
    clocks = sampler.stop() if sampler else None

    if rank == 0:
        out = {
            "metric": "decode_tok_s", "value": round(decode_tok_s, 2), "unit": "tok/s", "n_gpus": n_gpus, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round((tot_pre + tot_dec) / args.steps, 3), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "prompt_eval_tok_s": round(prefill_tok_s, 1), "ttft_ms_p50": round(ttft_p50, 3),
            "config": {"model": model, "quant": wl["ft"], "global_batch": slots, "seq_len": P + G, "prompt_tokens": P,
                       "generated_tokens": G, "num_ctx": wl["ctx"], "slots": slots, "kv_cache": be.kv_type,
                       "parallelism": "single" if n_gpus == 1 else f"{args.parallelism}{n_gpus}",
                       "l2": "inputs larger than L2 (weights of several GB are re-read every token)",
                       "weights": "random-init N(0,0.02), seed 0", "graphs": not args.no_graphs, "pdl": not args.no_pdl,
                       **({"layers_override": args.layers, "invalid_as_benchmark": True} if args.layers else {})},
            "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches), "load_s": round(t_load, 1), "impl": "ours",
        }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
