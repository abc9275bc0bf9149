"""Scheduler behaviour with fake runners and fabricated devices (the reference tests its scheduler the same way:
injected newServerFn / getGpuFn and mock runners, server/sched_test.go:210-276, 1221-2049)."""
import math
import threading
import time

import pytest

from ollama_b200.discover.devices import DeviceInfo
from ollama_b200.server.sched import ERR_MAX_QUEUE, Scheduler, SchedulerError, auto_num_batch, default_context, is_out_of_memory, predict_memory

GiB = 1 << 30


class FakeModel:
    def __init__(self, name, size=1 * GiB, adapters=()):
        self.name = self.short_name = name
        self.model_path = f"/blobs/{name}"
        self.size = size
        self.adapter_paths = list(adapters)
        self.projector_paths = []
        self.digest = name

    def kv(self):
        return {"general.architecture": "llama", "llama.block_count": 2, "llama.attention.head_count": 4,
                "llama.attention.head_count_kv": 2, "llama.embedding_length": 256}

    def capabilities(self):
        return ["completion"]


class FakeRunner:
    def __init__(self, model, opts, num_parallel, gpus, fail=None):
        if fail:
            raise fail
        self.model, self.opts, self.num_parallel, self.gpus = model, opts, num_parallel, gpus
        self.closed = False
        self.alive = True
        self.n_ctx = opts["num_ctx"]

    def ping(self):
        return self.alive and not self.closed

    def close(self):
        self.closed = True

    def memory(self):
        return {"total": self.model.size, "vram": self.model.size if self.gpus else 0}


def gpus(n=1, free=80 * GiB):
    return [DeviceInfo(id=f"GPU-{i}", index=i, name="B200", compute_major=10, total_memory=180 * GiB, free_memory=free) for i in range(n)]


def make(n_gpus=1, free=80 * GiB, **kw):
    created = []

    def factory(model, opts, num_parallel, use):
        r = FakeRunner(model, opts, num_parallel, use)
        created.append(r)
        return r

    s = Scheduler(new_runner_fn=kw.get("factory", factory), get_gpus_fn=kw.get("get_gpus", lambda: gpus(n_gpus, free)),
                  wait_for_recovery=kw.get("wait_for_recovery", 0.0))
    return s, created


OPTS = {"num_ctx": 2048, "num_batch": 512, "num_gpu": -1, "main_gpu": None, "use_mmap": None, "num_thread": 0, "draft_num_predict": 4}


def test_reuse_and_reload_predicate():
    s, created = make()
    m = FakeModel("a")
    r1 = s.get_runner(m, dict(OPTS), 60)
    r2 = s.get_runner(m, dict(OPTS), 60)
    assert r1 is r2 and len(created) == 1 and r1.ref_count == 2
    s.release(r1); s.release(r2)
    # automatic values do not force a reload, explicit changes do
    r3 = s.get_runner(m, {**OPTS, "num_ctx": 0, "num_gpu": -1}, 60)
    assert r3 is r1
    s.release(r3)
    r4 = s.get_runner(m, {**OPTS, "num_ctx": 4096}, 60)
    assert r4 is not r1 and created[0].closed and r4.options["num_ctx"] == 4096
    s.release(r4)
    r5 = s.get_runner(FakeModel("a", adapters=["/lora"]), {**OPTS, "num_ctx": 4096}, 60)
    assert r5 is not r4
    s.release(r5)
    created[-1].alive = False                      # failed ping -> replaced
    r6 = s.get_runner(FakeModel("a", adapters=["/lora"]), {**OPTS, "num_ctx": 4096}, 60)
    assert r6 is not r5
    s.unload_all()
    assert all(r.closed for r in created)


def test_keep_alive_timer_zero_and_forever():
    s, created = make()
    a = s.get_runner(FakeModel("a"), dict(OPTS), 0.15)
    s.release(a)
    assert not created[0].closed
    time.sleep(0.5)
    assert created[0].closed and s.ps() == []
    b = s.get_runner(FakeModel("b"), dict(OPTS), 0)       # zero keep-alive: unloaded as soon as it is idle
    assert not created[1].closed
    s.release(b)
    assert created[1].closed
    c = s.get_runner(FakeModel("c"), dict(OPTS), math.inf)
    s.release(c)
    assert math.isinf(c.expires_at) and not created[2].closed
    s.expire_runner(FakeModel("c"))
    assert created[2].closed


def test_expire_waits_for_inflight_request():
    s, created = make()
    m = FakeModel("a")
    r = s.get_runner(m, dict(OPTS), 60)
    s.expire_runner(m)
    assert not created[0].closed                           # still referenced
    s.release(r)
    assert created[0].closed


def test_max_loaded_models_evicts_idle_shortest_session(monkeypatch):
    monkeypatch.setenv("OLLAMA_MAX_LOADED_MODELS", "2")
    s, created = make()
    a = s.get_runner(FakeModel("a"), dict(OPTS), 600); s.release(a)
    b = s.get_runner(FakeModel("b"), dict(OPTS), 30); s.release(b)
    c = s.get_runner(FakeModel("c"), dict(OPTS), 60); s.release(c)
    names = sorted(r.model.name for r in s.ps())
    assert names == ["a", "c"] and created[1].closed       # "b" had the shortest session
    s.unload_all()


def test_memory_eviction_and_multi_gpu_placement():
    s, created = make(n_gpus=2, free=20 * GiB)
    small = s.get_runner(FakeModel("small", 4 * GiB), dict(OPTS), 60)
    assert len(created[0].gpus) == 1                       # fits 80 % of one GPU
    s.release(small)
    big = s.get_runner(FakeModel("big", int(39.5 * GiB)), dict(OPTS), 60)
    assert len(created[1].gpus) == 2                       # does not fit one GPU: spread over the node
    assert created[0].closed                               # and the idle small model was evicted to make room
    s.release(big)
    s.unload_all()


def test_placement_picks_the_smallest_group_that_fits():
    """1, 2, 4, ... GPUs, most free memory first; the chosen devices (not simply 0..n-1) are what the runner is given."""
    from ollama_b200.server.sched import Scheduler
    gpus = [DeviceInfo(id=str(i), index=i, total_memory=80 * GiB, free_memory=f * GiB) for i, f in enumerate((10, 70, 20, 60, 65, 5, 50, 40))]
    pick = lambda need: [g.index for g in Scheduler._place(gpus, int(need * GiB))]      # noqa: E731
    assert pick(30) == [1]                                  # the GPU with the most free memory
    assert pick(90) == [1, 4]                               # 2 x 0.8 x 65
    assert pick(150) == [1, 4, 3, 6]                        # 4 x 0.8 x 50
    assert sorted(pick(400)) == list(range(8))              # nothing fits: the whole node
    assert pick(1) == [1] and Scheduler._place([], 1) == []


def test_auto_context_shrinks_when_memory_is_short():
    assert default_context(gpus(1)) == 262144 and default_context([]) == 4096
    m = FakeModel("a", 1 * GiB)
    assert predict_memory(m, 4096, 1) == 1 * GiB + 2 * 2 * 2 * 64 * 4096 * 2
    s, created = make(n_gpus=1, free=int(1.6 * GiB))      # 256k tokens of KV do not fit, 32k do
    r = s.get_runner(m, {**OPTS, "num_ctx": 0}, 60)
    assert created[0].opts["num_ctx"] in (32768, 4096) and created[0].opts["num_ctx"] < 262144
    s.release(r)
    s.unload_all()


def test_queue_limit_and_single_loader(monkeypatch):
    monkeypatch.setenv("OLLAMA_MAX_QUEUE", "1")
    gate = threading.Event()
    started = threading.Event()

    def slow_factory(model, opts, num_parallel, use):
        started.set()
        gate.wait(5)
        return FakeRunner(model, opts, num_parallel, use)

    s, _ = make(factory=slow_factory)
    out = {}
    t = threading.Thread(target=lambda: out.setdefault("a", s.get_runner(FakeModel("a"), dict(OPTS), 60)))
    t.start()
    assert started.wait(5)
    with pytest.raises(SchedulerError) as e:              # queue of one is taken by the loading request
        s.get_runner(FakeModel("b"), dict(OPTS), 60)
    assert e.value.status == 503 and str(e.value) == ERR_MAX_QUEUE
    gate.set()
    t.join(5)
    assert out["a"].ref_count == 1
    s.unload_all()


def test_load_failure_and_oom_retry():
    calls = []

    def factory(model, opts, num_parallel, use):
        calls.append(opts["num_ctx"])
        if len(calls) == 1:
            raise MemoryError("CUDA out of memory")
        return FakeRunner(model, opts, num_parallel, use)

    s, _ = make(factory=factory)
    r = s.get_runner(FakeModel("a"), {**OPTS, "num_ctx": 0}, 60)     # automatic context: retried smaller after the OOM
    assert len(calls) == 2 and calls[1] < calls[0]
    s.release(r)

    def broken(model, opts, num_parallel, use):
        raise RuntimeError("bad file")

    s2, _ = make(factory=broken)
    with pytest.raises(SchedulerError) as e:
        s2.get_runner(FakeModel("a"), dict(OPTS), 60)
    assert e.value.status == 500 and "bad file" in str(e.value)


def test_prompt_batch_nobody_chose_follows_context_and_memory():
    """server/sched_test.go (automatic generation batch): 512 up to 4k of total context, 1024 up to 32k, 2048 above, stepping
    down when the model leaves too little of the device; two automatic sizes never force a reload, an explicit one does."""
    assert auto_num_batch(4096, 10 * GiB, 80 * GiB) == 512 and auto_num_batch(8192, 10 * GiB, 80 * GiB) == 1024
    assert auto_num_batch(65536, 10 * GiB, 80 * GiB) == 2048
    assert auto_num_batch(65536, 50 * GiB, 80 * GiB) == 1024            # over 60 % of the device: no room for the largest batch
    assert auto_num_batch(65536, 62 * GiB, 80 * GiB) == 512             # over 75 %
    assert auto_num_batch(65536, 63 * GiB + 512 * (1 << 20), 80 * GiB) == 512 and auto_num_batch(65536, 0, 0) == 2048
    s, created = make()
    m = FakeModel("a")
    r = s.get_runner(m, {**OPTS, "num_ctx": 16384}, 60, batch_auto=True)
    assert created[0].opts["num_batch"] == 1024 and r.batch_auto
    s.release(r)
    assert s.get_runner(m, {**OPTS, "num_ctx": 16384, "num_batch": 512}, 60, batch_auto=True) is r      # the default 512 is not a wish
    s.release(r)
    r2 = s.get_runner(m, {**OPTS, "num_ctx": 16384, "num_batch": 256}, 60)                               # an explicit size is
    assert r2 is not r and created[1].opts["num_batch"] == 256 and created[0].closed
    s.release(r2)


def test_eviction_waits_for_the_memory_to_come_back():
    """server/sched_test.go (VRAM recovery): after an unload the next load polls the devices until about three quarters of the
    runner's memory shows up as free, and goes on after a bounded wait when it never does."""
    state = {"free": 22 * GiB, "polls": 0, "closed_at": None}

    def get_gpus():
        state["polls"] += 1
        if state["closed_at"] is not None and state["polls"] - state["closed_at"] >= 3:
            return gpus(1, 70 * GiB)                                    # the driver catches up a few polls after the process is gone
        return gpus(1, state["free"])

    s, created = make(get_gpus=get_gpus, wait_for_recovery=5.0)
    a = s.get_runner(FakeModel("a", 20 * GiB), dict(OPTS), 60)
    s.release(a)
    orig_close = created[0].close

    def close():
        orig_close()
        state["closed_at"] = state["polls"]

    created[0].close = close
    t0 = time.monotonic()
    b = s.get_runner(FakeModel("b", 25 * GiB), dict(OPTS), 60)           # 25 GiB do not fit into the 22 that are free: a has to go
    assert created[0].closed and 0.2 < time.monotonic() - t0 < 4.9 and b.runner is created[1]      # before the 5 s limit
    s.release(b)
    # memory that never comes back: the wait gives up at its limit
    s2, c2 = make(free=30 * GiB, wait_for_recovery=0.3)
    x = s2.get_runner(FakeModel("x", 20 * GiB), dict(OPTS), 60)
    s2.release(x)
    t0 = time.monotonic()
    y = s2.get_runner(FakeModel("y", 40 * GiB), dict(OPTS), 60)          # the load goes ahead on the estimate after the bounded wait
    assert c2[0].closed and 0.25 < time.monotonic() - t0 < 10.0 and y.runner is c2[1]


def test_running_out_of_memory_at_run_time_expires_every_runner():
    """server/sched_test.go (runtime OOM): idle runners go at once, busy ones when their request ends; other errors change nothing."""
    s, created = make(n_gpus=2)
    a = s.get_runner(FakeModel("a"), dict(OPTS), 600)
    b = s.get_runner(FakeModel("b"), dict(OPTS), 600)
    s.release(a)
    assert not s.expire_for_runtime_oom(RuntimeError("tokenizer mismatch")) and len(s.loaded) == 2
    assert is_out_of_memory("CUDA out of memory. Tried to allocate 2 GiB") and is_out_of_memory(MemoryError()) and not is_out_of_memory("timeout")
    assert s.expire_for_runtime_oom(RuntimeError("CUDA out of memory. Tried to allocate 2 GiB"))
    assert created[0].closed and not created[1].closed and list(s.loaded) == ["/blobs/b"]
    s.release(b)
    assert created[1].closed and not s.loaded


def test_a_slow_runner_does_not_hold_the_table_lock():
    """A liveness probe or a shutdown that takes long runs with the lock released: requests for other models go through meanwhile."""
    s, created = make(n_gpus=2)
    a = s.get_runner(FakeModel("a"), dict(OPTS), 60)
    s.release(a)
    gate, entered = threading.Event(), threading.Event()

    def slow_ping():
        entered.set()
        gate.wait(5)
        return True

    created[0].ping = slow_ping
    got = []
    t = threading.Thread(target=lambda: got.append(s.get_runner(FakeModel("a"), dict(OPTS), 60)))
    t.start()
    assert entered.wait(2)
    t0 = time.monotonic()
    b = s.get_runner(FakeModel("b"), dict(OPTS), 60)                     # loads while a's probe is still out
    assert s.ps() and time.monotonic() - t0 < 4.0 and b.runner is created[1]      # well inside the 5 s the probe would block for
    gate.set()
    t.join(5)
    assert got and got[0] is a and a.ref_count == 1
    s.release(a); s.release(b)
    # the same for close(): a zero keep-alive unload that blocks does not stop ps() or other requests
    gate.clear(); entered.clear()

    def slow_close():
        entered.set()
        gate.wait(5)

    created[1].close = slow_close
    b2 = s.get_runner(FakeModel("b"), dict(OPTS), 0)
    t = threading.Thread(target=lambda: s.release(b2))
    t.start()
    assert entered.wait(2)
    t0 = time.monotonic()
    assert [r.model_key for r in s.ps()] == ["/blobs/a"] and time.monotonic() - t0 < 4.0
    gate.set()
    t.join(5)


def test_predicted_memory_counts_the_prefill_copy_when_it_would_be_made():
    m = FakeModel("a", 4 * GiB)
    base = predict_memory(m, 2048, 1)
    kv = dict(m.kv(), **{"llama.feed_forward_length": 1024, "llama.vocab_size": 32000})
    m.kv = lambda: kv
    copy = 2 * (2 * (256 * (2 * 4 * 64 + 2 * 2 * 64) + 3 * 256 * 1024) + 32000 * 256)
    assert predict_memory(m, 2048, 1, free=80 * GiB) == base + copy
    assert predict_memory(m, 2048, 1, free=2 * copy) == base             # would take more than 40 % of the free memory: not made
    kv["llama.expert_count"] = 8
    assert predict_memory(m, 2048, 1, free=80 * GiB) == base + copy - 2 * 2 * 3 * 256 * 1024   # expert matrices are not part of the dense copy


def test_replicas_spread_requests_over_whole_copies(monkeypatch):
    """B200_REPLICAS: one runner per GPU behind one interface; a request goes to the copy with the fewest requests in flight,
    a follow-up that shares its prompt prefix goes back to the copy that holds it, the set reports summed memory and closes whole."""
    from ollama_b200.engine.replicas import ReplicaSet
    from ollama_b200.server.sched import Scheduler as S

    class R:
        def __init__(self, i):
            self.i, self.closed, self.n_ctx, self.seen = i, False, 64, []
            self.stats = {"requests": 0}

        def completion(self, req):
            self.seen.append(req.prompt)
            self.stats["requests"] += 1
            yield self.i
            yield "done"

        def ping(self):
            return not self.closed

        def memory(self):
            return {"total": 10, "vram": 10}

        def close(self):
            self.closed = True

        def tokenize(self, text, **kw):
            return [self.i]

    class Req:
        def __init__(self, prompt):
            self.prompt = prompt

    rs = ReplicaSet(R, 3)
    a = rs.completion(Req([1, 2, 3]))
    assert next(a) == 0                                     # first request: first copy, still in flight
    b = rs.completion(Req([7, 8]))
    assert next(b) == 1                                     # the idle copies come first
    assert list(rs.completion(Req([9]))) == [2, "done"]
    list(a), list(b)
    assert list(rs.completion(Req([7, 8, 9, 10])))[0] == 1  # shares a prefix with what copy 1 served last
    assert list(rs.completion(Req([1, 2, 3, 4])))[0] == 0
    assert rs.inflight == [0, 0, 0] and rs.memory() == {"total": 30, "vram": 30} and rs.stats["requests"] == 5 and rs.stats["replicas"] == 3
    assert rs.n_ctx == 64 and rs.tokenize("x") == [0] and rs.ping()
    rs.replicas[1].closed = True
    assert not rs.ping()
    rs.close()
    assert all(r.closed for r in rs.replicas)
    # a copy that fails to start takes the ones before it down with it
    made = []

    def flaky(i):
        if i == 2:
            raise MemoryError("no room")
        made.append(R(i))
        return made[-1]

    with pytest.raises(MemoryError):
        ReplicaSet(flaky, 3)
    assert len(made) == 2 and all(r.closed for r in made)
    # placement: as many one-copy groups as asked for and as the node has, most free memory first
    g = gpus(4)
    assert len(S._place_copies(g, 10 * GiB, 2)) == 2 and len(S._place_copies(g, 10 * GiB, 8)) == 4
    assert len(S._place_copies(g, 100 * GiB, 2)) == 4       # one copy already needs two GPUs
    monkeypatch.setenv("B200_REPLICAS", "2")
    s, created = make(n_gpus=4)
    ref = s.get_runner(FakeModel("a", 10 * GiB), dict(OPTS), 60)
    assert len(created[0].gpus) == 2                        # the factory is handed the GPUs of both copies
    s.release(ref)
