"""Host-side logic of the tensor-parallel engine: weight sharding and the leader/follower control channel (gloo, CPU)."""
import json
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ollama_b200.models.config import config_from_gguf
from ollama_b200.models.synth import SyntheticTensors, synthetic_header


def test_shards_recombine_to_the_full_matrices():
    from ollama_b200.parallel.tp_engine import ShardedTensors, shard_plan
    cfg = config_from_gguf(synthetic_header("tiny-tp", "Q4_K_M"))
    src = SyntheticTensors("tiny-tp", "Q4_K_M")
    world = 4
    shards = [ShardedTensors(src, cfg, r, world) for r in range(world)]
    # column-parallel: rows concatenate
    for leaf in ("attn_q", "attn_k", "attn_v", "ffn_gate", "ffn_up"):
        name = f"blk.1.{leaf}.weight"
        full = src[name].dequant()
        assert torch.equal(torch.cat([s[name].dequant() for s in shards]), full)
    # row-parallel: partial products add up
    for leaf, k in (("attn_output", cfg.q_dim), ("ffn_down", cfg.d_ff)):
        name = f"blk.0.{leaf}.weight"
        full = src[name].dequant()
        x = torch.randn(3, k, generator=torch.Generator().manual_seed(1))
        acc = sum(x[:, r * k // world:(r + 1) * k // world] @ shards[r][name].dequant().t() for r in range(world))
        assert torch.allclose(acc, x @ full.t(), atol=1e-5)
    # vocabulary rows
    out = torch.cat([s["output.weight"].dequant() for s in shards])
    assert torch.equal(out, src["output.weight"].dequant())
    # replicated tensors pass through
    assert torch.equal(shards[2]["blk.0.attn_norm.weight"].dequant(), src["blk.0.attn_norm.weight"].dequant())
    with pytest.raises(ValueError):
        shard_plan(cfg, 3)
    with pytest.raises(ValueError):      # 16 heads x 64 / 16 ranks = 64 columns: not a multiple of the 256-element K-quant block
        shard_plan(config_from_gguf(synthetic_header("tiny-tp", "Q4_K_M")), 16)


class _FakeBackend:
    name = "fake"

    def __init__(self, log):
        self.log, self.use_graphs, self.pdl = log, True, True

    def _rec(self, *a):
        self.log.append(list(a))

    def alloc(self, n_slots, n_ctx):
        self._rec("alloc", n_slots, n_ctx)

    def prefill(self, slot, tokens, pos0, need_logits=True):
        self._rec("prefill", slot, list(tokens), pos0, bool(need_logits))
        return torch.zeros(4)

    def hidden(self, slot, tokens):
        self._rec("hidden", slot, list(tokens))
        return torch.zeros(1, 4)

    def decode(self, slots, tokens, positions):
        self._rec("decode", list(slots), list(tokens), list(positions))
        return torch.zeros(len(slots), 4)

    def decode_argmax(self, slots, tokens, positions):
        self._rec("decode_argmax", list(slots), list(tokens), list(positions))
        return [0] * len(slots)

    def decode_loop(self, slots, tokens, positions, n_steps, first_tokens=None):
        self._rec("decode_loop", list(slots), list(tokens), list(positions), n_steps)
        return torch.zeros(n_steps, len(slots))

    def close(self):
        self._rec("close")


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from ollama_b200.parallel.control import TPControl, TPLeader, follow
    log = []
    be = _FakeBackend(log)
    ctl = TPControl(rank, world)
    if rank == 0:
        lead = TPLeader(be, ctl)
        lead.set_flags(False, True)
        lead.alloc(4, 256)
        lead.prefill(2, list(range(100)), 0, True)        # longer than one record: travels as a second message
        lead.prefill(1, [5, 6, 7], 100, False)
        lead.decode([0, 3], [11, 12], [7, 9])
        lead.decode_argmax([1], [42], [103])
        lead.decode_loop([0, 1], [0, 0], [5, 6], 3, first_tokens=torch.tensor([8, 9]))
        lead.hidden(0, [1, 2, 3])
        lead.close()
    else:
        follow(be, ctl)
    with open(os.path.join(out_dir, f"log{rank}.json"), "w") as f:
        json.dump({"log": log, "flags": [be.use_graphs, be.pdl]}, f)
    dist.destroy_process_group()


def test_followers_repeat_the_leaders_calls(tmp_path):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    world = 3
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    logs = [json.load(open(tmp_path / f"log{r}.json")) for r in range(world)]
    assert logs[0]["log"][0] == ["alloc", 4, 256] and logs[0]["log"][-1] == ["close"]
    assert ["decode_loop", [0, 1], [8, 9], [5, 6], 3] in logs[0]["log"]
    for r in (1, 2):
        assert logs[r]["log"] == logs[0]["log"]
        assert logs[r]["flags"] == [False, True]


def _pipe_follower(conn, rank, world, out_path):
    from ollama_b200.parallel.control import TPControl, follow
    from ollama_b200.parallel.transport import PipeTransport
    log = []
    tr = PipeTransport(rank, world, [conn])
    assert tr.all_gather(f"h{rank}") == ["h0", "h1", "h2"]
    tr.barrier()
    follow(_FakeBackend(log), TPControl(rank, world, tr))
    with open(out_path, "w") as f:
        json.dump(log, f)


def test_pipe_transport_carries_rendezvous_and_call_records(tmp_path):
    """The server-side carrier: pipes from a leader to spawned followers (no torch.distributed in the leader)."""
    from ollama_b200.parallel.control import TPControl, TPLeader
    from ollama_b200.parallel.transport import PipeTransport
    ctx = mp.get_context("spawn")
    world, conns, procs = 3, [], []
    for r in range(1, world):
        parent, child = ctx.Pipe()
        p = ctx.Process(target=_pipe_follower, args=(child, r, world, str(tmp_path / f"f{r}.json")))
        p.start()
        child.close()
        conns.append(parent)
        procs.append(p)
    tr = PipeTransport(0, world, conns)
    assert tr.all_gather("h0") == ["h0", "h1", "h2"]
    tr.barrier()
    log = []
    lead = TPLeader(_FakeBackend(log), TPControl(0, world, tr))
    lead.alloc(2, 128)
    lead.prefill(0, list(range(70)), 0, True)
    lead.decode_argmax([0, 1], [3, 4], [70, 9])
    lead.close()
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for r in (1, 2):
        assert json.load(open(tmp_path / f"f{r}.json")) == log


def test_runner_ping_follows_the_follower_processes():
    """A follower process that is gone makes the runner unhealthy, so that the scheduler's reload check replaces it."""
    from ollama_b200.engine.runner import Runner
    from ollama_b200.parallel.launcher import TPGroup

    class _Proc:
        def __init__(self, alive):
            self._alive = alive

        def is_alive(self):
            return self._alive

    grp = TPGroup.__new__(TPGroup)
    grp.procs = [_Proc(True), _Proc(True)]
    assert grp.alive()
    r = Runner.__new__(Runner)
    r.closed, r.error, r._tp_group = False, None, grp
    r.thread = _Proc(True)
    assert r.ping()
    grp.procs[1]._alive = False
    assert not grp.alive() and not r.ping()
    r._tp_group = None
    assert r.ping()


def test_pipe_transport_bounds_every_wait_and_tags_its_messages():
    """A follower that fails, hangs or dies never leaves the leader blocked, and its error is not mistaken for data."""
    import multiprocessing as mp
    import pytest
    from ollama_b200.parallel.transport import PipeTransport, TransportError
    ctx = mp.get_context("spawn")

    def leader(n=1, timeout=0.3):
        pairs = [ctx.Pipe() for _ in range(n)]
        return PipeTransport(0, n + 1, [p for p, _ in pairs], timeout=timeout), [c for _, c in pairs]

    # an error that arrives in the middle of an all-gather is raised, not returned as that rank's share
    tr, (child,) = leader()
    child.send(("error", "rank 1: out of memory"))
    with pytest.raises(TransportError, match="out of memory"):
        tr.all_gather("handle-0")
    # a follower that never answers
    tr, _ = leader()
    with pytest.raises(TransportError, match="did not answer"):
        tr.all_gather("handle-0")
    with pytest.raises(TransportError, match="in time"):
        tr.wait_ready()
    # "ready" may overtake the leader's next all-gather: it is remembered, the gather still completes
    tr, (child,) = leader()
    child.send(("ready", 1))
    child.send(("gather", "handle-1"))
    assert tr.all_gather("handle-0") == ["handle-0", "handle-1"] and child.recv() == ("gather", ["handle-0", "handle-1"])
    tr.wait_ready()          # already seen
    # a follower learns that the leader is gone from the closed pipe
    parent, child = ctx.Pipe()
    f = PipeTransport(1, 2, [child])
    parent.close()
    with pytest.raises(TransportError, match="leader gone"):
        f.bcast_ints(None, 6)


def test_every_split_of_an_expert_model_passes_the_engine_support_check():
    """gpt-oss-120b under 2, 4 and 8 ranks: the per-rank configuration (heads, KV heads, experts and the unused dense-FFN width
    divided by the rank count) is one the sm_100a engine takes; a dense model whose FFN width per rank is not a multiple of 32
    is still refused."""
    import dataclasses

    from ollama_b200.engine.b200 import supports
    from ollama_b200.models.config import config_from_gguf
    from ollama_b200.models.synth import synthetic_header
    from ollama_b200.parallel.tp_engine import shard_plan
    cfg = config_from_gguf(synthetic_header("gpt-oss-120b", "MXFP4"))
    for world in (2, 4, 8):
        p = shard_plan(cfg, world)
        local = dataclasses.replace(cfg, n_heads=p["heads"], n_kv_heads=p["kv_heads"], d_ff=p["d_ff"], n_experts=p["experts"])
        assert p["d_ff"] % 32 != 0 or world == 2
        assert supports(local), world
    dense = config_from_gguf(synthetic_header("llama-3.1-8b", "Q4_K_M"))
    assert supports(dense) and not supports(dataclasses.replace(dense, d_ff=14336 // 8 + 8))
