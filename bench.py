"""Headline benchmark: decode tok/s + prompt-eval tok/s (+ p50 TTFT) on a random-init GGUF-architecture model.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--model NAME] [--slots S]

N = 1 runs Llama-3.1-8B-architecture Q4_K_M (512-token random prompt, 128 generated tokens, greedy,
num_ctx 8192); N >= 2 runs Llama-3.1-70B-architecture Q4_K_M tensor-parallel over N GPUs (2048-token
prompt, 256 generated tokens).  One *step* is one request epoch on every slot: prefill of a fresh
random prompt followed by the whole generation.  Timing is on the device with CUDA events, max over
ranks; weights (GBs) are far larger than L2, so no flush is needed between iterations.

Because the two headline workloads are different models, the line also carries the other halves of those
workloads under ``extras`` (never part of ``value``): at N = 1 the 8B model at 4 slots and the 70B model
on the single GPU (``same_model_n1``: the start of a same-model 1 -> 8 curve); at N >= 2 the 70B model at
concurrency 8.  At N >= 2 the tensor-parallel engine is first compared with the single-GPU engine on a
small model (``tp_selfcheck``), the generated tokens of all ranks are compared, and a run whose
exchanges reported a timed-out wait is refused.

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


def build_backend(model: str, ft: str, n_gpus: int, world: int, rank: int, dev: str, kv_type: str, pp: bool, args):
    from ollama_b200.models.config import config_from_gguf
    from ollama_b200.models.synth import SyntheticTensors, synthetic_header
    cfg = config_from_gguf(synthetic_header(model, ft))
    if pp:
        from ollama_b200.engine.pipeline import PipelineBackend
        be = PipelineBackend(None, list(range(n_gpus)), cfg=cfg, tensors=lambda d: SyntheticTensors(model, ft, seed=0, device=str(d)), kv_type=kv_type)
    elif n_gpus == 1:
        from ollama_b200.engine.b200 import B200Backend
        be = B200Backend(None, device=dev, cfg=cfg, tensors=SyntheticTensors(model, ft, seed=0, device=dev), kv_type=kv_type)
    else:
        from ollama_b200.parallel.tp_engine import TPBackend
        be = TPBackend(cfg, SyntheticTensors(model, ft, seed=0, device=dev), device=dev, rank=rank, world=world, kv_type=kv_type)
    for part in (be.stages if pp else [be]):
        part.use_graphs = not args.no_graphs
        part.pdl = not args.no_pdl
    return be, cfg


def device_epochs(be, cfg, P: int, G: int, slots: int, steps: int, warmup: int, world: int, pp: bool, dev: str, gen) -> dict:
    """``steps`` request epochs timed on the device (CUDA events, max over ranks) after ``warmup`` untimed ones."""
    import torch
    import torch.distributed as dist
    slot_ids = list(range(slots))

    def sync_stages():
        """Pipeline: the events live on the first device, so the work of the later stages is waited for before each record."""
        if pp:
            for d in be.devices:
                torch.cuda.synchronize(d)

    def epoch():
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

    for _ in range(warmup):
        epoch()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    launches0 = be.kernel_launches
    pre_ms, dec_ms, toks = [], [], None
    for _ in range(steps):
        a, b, toks = epoch()
        pre_ms.append(a)
        dec_ms.append(b)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        t = torch.tensor([sum(pre_ms), sum(dec_ms)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        tot_pre, tot_dec = t.tolist()
    else:
        tot_pre, tot_dec = sum(pre_ms), sum(dec_ms)
    return {"decode_tok_s": slots * (G - 1) * steps / (tot_dec / 1e3), "prompt_eval_tok_s": slots * P * steps / (tot_pre / 1e3),
            "ttft_ms_p50": statistics.median(pre_ms) / slots, "tot_ms": tot_pre + tot_dec, "launches": be.kernel_launches - launches0,
            "tokens": toks}


def check_ranks(be, toks, world: int, dev: str) -> str:
    """Tensor-parallel run: no exchange may have timed out and every rank must have generated the same tokens."""
    import torch
    import torch.distributed as dist
    bad = torch.tensor([int(be.comm_status() != 0)], device=dev)
    dist.all_reduce(bad, op=dist.ReduceOp.MAX)
    if bad.item():
        return "an exchange timed out"
    got = [torch.empty_like(toks) for _ in range(world)]
    dist.all_gather(got, toks.contiguous())
    return "ok" if all(torch.equal(g, got[0]) for g in got) else "ranks generated different tokens"


def short(r: dict) -> dict:
    return {"decode_tok_s": round(r["decode_tok_s"], 2), "prompt_eval_tok_s": round(r["prompt_eval_tok_s"], 1), "ttft_ms_p50": round(r["ttft_ms_p50"], 3)}


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
    ap.add_argument("--no-extras", action="store_true", help="skip the other halves of the headline workloads (4 slots, concurrency 8, 70B on one GPU)")
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

    auto = args.model == "auto"
    model = args.model if not auto else ("llama-3.1-8b" if n_gpus == 1 else "llama-3.1-70b")
    wl = dict(WORKLOADS[model])
    for k in ("prompt", "gen", "ctx"):
        if getattr(args, k):
            wl[k] = getattr(args, k)
    slots = args.slots if args.slots > 0 else wl.get("slots", 1)
    extras_wanted = auto and not args.no_extras and not args.layers and args.slots == 0

    from ollama_b200.engine.runner import CompletionRequest, Runner, RunnerOptions
    from ollama_b200.engine.sampler import SamplingParams

    dev = f"cuda:{local}"
    pp = pp_gpus > 1
    tp_selfcheck = None
    if world > 1 and not pp:
        from ollama_b200.parallel.selftest import run_selfcheck
        # 8-bit blocks of 32 divide the small model's 128 columns per rank at 4 and 8 ranks; 256-element K-quant blocks only at 2
        sc = run_selfcheck(rank, world, dev, quant="Q4_K_M" if world == 2 else "Q8_0", steps=3)
        tp_selfcheck = "ok" if sc["ok"] else f"failed: {json.dumps(sc)}"
        if not sc["ok"]:
            if rank == 0:
                print(json.dumps({"impl": "ours", "invalid": "tensor-parallel self-check failed", "tp_selfcheck": sc}))
            dist.destroy_process_group()
            sys.exit(1)
    if args.layers:      # profiling aid: a truncated stack keeps ncu captures short; the result is flagged below
        import dataclasses
        from ollama_b200.models import synth
        synth.SPECS[model] = dataclasses.replace(synth.SPECS[model], n_layers=args.layers)
    t_load = time.time()
    be, cfg = build_backend(model, wl["ft"], n_gpus, world, rank, dev, args.kv_type, pp, args)
    be.alloc(slots, wl["ctx"])
    torch.cuda.synchronize()
    t_load = time.time() - t_load

    P, G = wl["prompt"], wl["gen"]
    gen = torch.Generator().manual_seed(1234)
    warmup = max(args.warmup, 3)
    sampler = ClockSampler(local).start() if rank == 0 else None
    main_r = device_epochs(be, cfg, P, G, slots, args.steps, warmup, world, pp, dev, gen)
    clocks = sampler.stop() if sampler else None
    decode_tok_s, prefill_tok_s, ttft_p50 = main_r["decode_tok_s"], main_r["prompt_eval_tok_s"], main_r["ttft_ms_p50"]
    launches = main_r["launches"]
    rank_check = check_ranks(be, main_r["tokens"], world, dev) if world > 1 and not pp else None
    if rank_check not in (None, "ok"):
        if rank == 0:
            print(json.dumps({"impl": "ours", "invalid": rank_check, "n_gpus": n_gpus}))
        dist.destroy_process_group()
        sys.exit(1)

    # ---- the other halves of the headline workloads (never part of `value`) --------------------------
    extras = {}
    if extras_wanted and not pp:
        esteps = max(2, min(args.steps, 3))
        s2 = 4 if n_gpus == 1 else 8
        be.alloc(s2, wl["ctx"])
        r2 = device_epochs(be, cfg, P, G, s2, esteps, 3, world, pp, dev, gen)
        extras["slots4" if n_gpus == 1 else "concurrency8"] = {"model": model, "slots": s2, **short(r2)}
        if world > 1:
            extras["concurrency8"]["ranks_agree"] = check_ranks(be, r2["tokens"], world, dev)
        be.alloc(slots, wl["ctx"])

    # ---- end to end through the public runner API --------------------------------------------------
    e2e = None
    runner_be = be
    ctl = None
    if not args.no_e2e and n_gpus > 1 and not pp:
        # the serving stack runs in rank 0 only; the other ranks repeat its backend calls until it hands the group back
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

    if extras_wanted and n_gpus == 1:
        be.close()
        del be, runner_be
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        m70 = "llama-3.1-70b"
        w70 = WORKLOADS[m70]
        try:
            be70, cfg70 = build_backend(m70, w70["ft"], 1, 1, 0, dev, args.kv_type, False, args)
            be70.alloc(1, w70["ctx"])
            extras["same_model_n1"] = {"model": m70, "slots": 1, "prompt_tokens": w70["prompt"], "generated_tokens": w70["gen"],
                                       **short(device_epochs(be70, cfg70, w70["prompt"], w70["gen"], 1, 2, 3, 1, False, dev, gen))}
            be70.close()
        except RuntimeError as e:      # e.g. the GPU is shared and 42 GB are not free
            extras["same_model_n1"] = {"model": m70, "unavailable": str(e)[:200]}

    if rank == 0:
        out = {
            "metric": "decode_tok_s", "value": round(decode_tok_s, 2), "unit": "tok/s", "n_gpus": n_gpus, "steps": args.steps,
            "warmup": warmup, "ms_per_step": round(main_r["tot_ms"] / args.steps, 3), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None,
            "dtype": ("int8 activations x MXFP4 experts and 8 / 16-bit dense weights (decode), bf16 (prefill)" if wl["ft"] == "MXFP4"
                      else "int8 activations x Q4_K/Q6_K weights (decode), bf16 (prefill)"), "data": "synthetic",
            "prompt_eval_tok_s": round(prefill_tok_s, 1), "ttft_ms_p50": round(ttft_p50, 3),
            "config": {"model": model, "quant": wl["ft"], "global_batch": slots, "seq_len": P + G, "prompt_tokens": P,
                       "generated_tokens": G, "num_ctx": wl["ctx"], "slots": slots, "kv_cache": args.kv_type,
                       "parallelism": "single" if n_gpus == 1 else f"{args.parallelism}{n_gpus}",
                       "l2": "inputs larger than L2 (weights of several GB are re-read every token)",
                       "weights": "random-init N(0,0.02), seed 0", "graphs": not args.no_graphs, "pdl": not args.no_pdl,
                       "scaling_note": "N = 1 is Llama-8B and N >= 2 Llama-70B (the two headline workloads); the same-model curve starts "
                                       "at extras.same_model_n1",
                       **({"layers_override": args.layers, "invalid_as_benchmark": True} if args.layers else {})},
            "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches), "load_s": round(t_load, 1), "impl": "ours",
            "extras": extras,
        }
        if tp_selfcheck is not None:
            out["tp_selfcheck"] = tp_selfcheck
            out["ranks_agree"] = rank_check
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
