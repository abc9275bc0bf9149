"""Model scheduler: load / reuse / evict runners, keep-alive timers, bounded request queue.

Semantics follow the reference scheduler (server/sched.go):
  * one runner per model; requests for a loaded model whose load-time options still match reuse it
    (:169-211, reload predicate :1381-1431 -- adapters/projectors, num_ctx / num_batch / num_gpu /
    main_gpu / use_mmap / num_thread with "automatic" values ignored, failed ping);
  * one model loads at a time (:66-74, :517-606); the queue holds OLLAMA_MAX_QUEUE requests, beyond
    that callers get "server busy" / HTTP 503 (:88, :204-208);
  * at most OLLAMA_MAX_LOADED_MODELS runners (default 3 x GPUs, :83-86, :280-291); to make room the
    idle runner with the shortest session is unloaded first (:1557-1693);
  * a finished request restarts the keep-alive timer; zero keep-alive unloads immediately, a negative
    one never expires (:374-413); expiry waits until the reference count drops to zero (:414-468);
  * predicted memory = weights + KV cache of num_ctx x num_parallel tokens (:535-536); a model that
    does not fit the free memory of one GPU is spread over the GPUs of the node (:972-1031);
  * num_ctx floor 4 (:170-172), default context tier by total VRAM (server/routes.go:2043-2058);
  * a prompt batch nobody chose is sized by the context and by the memory left after the model (:797-915);
  * after an eviction the load waits until the GPUs report the memory back, for a bounded time (:1441-1499);
  * a request that died of device memory exhaustion expires every runner, so that the next request starts from an
    empty device (:1632-1661).
The table lock guards bookkeeping only: a runner is pinged, closed and waited for with the lock released, so one slow
runner cannot stall requests for the others.
Dependencies (runner factory, device query, clock) are constructor arguments so tests can run the
whole matrix with fabricated devices and fake runners, as the reference's tests do (sched_test.go).
"""
from __future__ import annotations

import logging
import math
import os
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Callable

from .. import envconfig
from ..api.types import runner_options
from ..discover.devices import GPU_OVERHEAD_DEFAULT, DeviceInfo

log = logging.getLogger("ollama_b200.sched")


class SchedulerError(Exception):
    def __init__(self, msg: str, status: int = 500):
        super().__init__(msg)
        self.status = status


ERR_MAX_QUEUE = "server busy, please try again.  maximum pending requests exceeded"


@dataclass
class RunnerRef:
    model_key: str
    model: Any
    runner: Any
    options: dict[str, Any]
    num_parallel: int = 1
    ref_count: int = 0
    session_duration: float = 300.0
    expires_at: float = math.inf
    total_size: int = 0
    vram_size: int = 0
    gpus: list[str] = field(default_factory=list)
    loaded_at: float = 0.0
    timer: threading.Timer | None = None
    context_length: int = 0
    batch_auto: bool = False                  # num_batch was chosen by the scheduler, not by the Modelfile or the request
    loading: bool = False

    def needs_reload(self, model: Any, opts: dict[str, Any], batch_auto: bool = False) -> bool:
        return self.options_differ(model, opts, batch_auto) or not self.alive()

    def alive(self) -> bool:
        """Liveness probe of the runner; called without the scheduler's lock."""
        try:
            return bool(self.runner.ping())
        except Exception:
            return False

    def options_differ(self, model: Any, opts: dict[str, Any], batch_auto: bool = False) -> bool:
        if list(getattr(model, "adapter_paths", [])) != list(getattr(self.model, "adapter_paths", [])):
            return True
        if list(getattr(model, "projector_paths", [])) != list(getattr(self.model, "projector_paths", [])):
            return True
        if list(getattr(model, "draft_paths", [])) != list(getattr(self.model, "draft_paths", [])):
            return True
        want, have = runner_options(opts), self.options
        for k in ("num_batch", "num_thread", "main_gpu", "use_mmap", "draft_num_predict"):
            if k == "num_batch" and batch_auto and self.batch_auto:
                continue                          # both sizes are the scheduler's own choice
            if want.get(k) is not None and want.get(k) != have.get(k):
                return True
        if want.get("num_ctx") and want["num_ctx"] != have.get("num_ctx"):
            return True
        if want.get("num_gpu", -1) not in (-1, None) and want["num_gpu"] != have.get("num_gpu"):
            return True
        return False


def default_context(gpus: list[DeviceInfo]) -> int:
    """4k / 32k / 256k tokens by total VRAM (< 24, 24-48, >= 48 GiB)."""
    total = sum(g.total_memory for g in gpus)
    if total >= 47 << 30:
        return 262144
    if total >= 23 << 30:
        return 32768
    return 4096


def _first_int(v, default=0):
    if v is None:
        return default
    try:
        return int(v[0]) if hasattr(v, "__len__") and not isinstance(v, str) else int(v)
    except (TypeError, ValueError, IndexError):
        return default


def predict_memory(model: Any, num_ctx: int, num_parallel: int, free: int | None = None) -> int:
    """Weights (+ draft model) + KV cache of the configured type for num_ctx x num_parallel tokens (llm/llama_server.go:2681-2700).
    Every layer is counted at the full context: the engine gives sliding-window layers a cache of that length too.  With
    ``free`` (bytes free on the GPU the model would go to) the 16-bit copy of the dense matrices that the engine keeps for
    prefill is counted as well, under the engine's own rule: it is made when it takes less than 40 % of the free memory."""
    size = int(getattr(model, "size", 0) or 0)
    kv = getattr(model, "kv", lambda: {})() or {}
    arch = kv.get("general.architecture", "")
    layers = _first_int(kv.get(f"{arch}.block_count"))
    heads = _first_int(kv.get(f"{arch}.attention.head_count"), 1) or 1
    kvh = _first_int(kv.get(f"{arch}.attention.head_count_kv"), heads) or heads
    d = _first_int(kv.get(f"{arch}.embedding_length"))
    hd = _first_int(kv.get(f"{arch}.attention.key_length"), d // heads if heads else 0)
    per_elem = 2.0                                   # f16 cache
    if (envconfig.kv_cache_type() or "f16").lower() in ("q8_0", "q4_0") and hd % 32 == 0:
        per_elem = 1.0 + 2.0 / 32                    # int8 + one f16 scale per 32 dims (q4_0 requests are served as q8_0)
    extra = sum(os.path.getsize(p) for p in list(getattr(model, "draft_paths", None) or []) if os.path.exists(p))
    total = size + extra + int(2 * layers * kvh * hd * num_ctx * num_parallel * per_elem)
    if free:
        ff = _first_int(kv.get(f"{arch}.feed_forward_length"))
        vocab = _first_int(kv.get(f"{arch}.vocab_size")) or len(kv.get("tokenizer.ggml.tokens") or ())
        experts = _first_int(kv.get(f"{arch}.expert_count"))
        copy = 2 * (layers * (d * (2 * heads * hd + 2 * kvh * hd) + (0 if experts else 3 * d * ff)) + vocab * d)
        if copy < 0.4 * free:
            total += copy
    return total


# prompt batch the scheduler picks when nobody set num_batch: (batch, for a total context above, share of the memory the
# model may take, activation memory the batch itself needs); the first row that fits wins (server/sched.go:797-915)
BATCH_TIERS = ((2048, 32768, 0.60, 2 << 30), (1024, 4096, 0.75, 768 << 20), (512, 0, 0.80, 0))


def auto_num_batch(total_ctx: int, predicted: int, available: int) -> int:
    for batch, above, share, surcharge in BATCH_TIERS:
        if total_ctx <= above and batch > 512:
            continue
        if batch == 512 or not (predicted and available):
            return batch
        if predicted <= share * available and predicted + surcharge <= 0.8 * available:
            return batch
    return 512


def is_out_of_memory(err: BaseException | str) -> bool:
    text = str(err).lower()
    return isinstance(err, MemoryError) or "out of memory" in text or "cudaerrormemoryallocation" in text or "failed to allocate" in text


class Scheduler:
    def __init__(self, new_runner_fn: Callable[..., Any] | None = None, get_gpus_fn: Callable[[], list[DeviceInfo]] | None = None,
                 now: Callable[[], float] = time.monotonic, wait_for_recovery: float = 5.0):
        self.new_runner_fn = new_runner_fn or _default_runner
        self.get_gpus_fn = get_gpus_fn or (lambda: [])
        self.now = now
        self.wait_for_recovery = wait_for_recovery     # longest wait for the GPUs to report an evicted runner's memory as free
        self.loaded: dict[str, RunnerRef] = {}
        self.lock = threading.Condition()
        self.load_lock = threading.Lock()
        self.pending = 0
        self._gpus: list[DeviceInfo] | None = None

    # -- configuration ----------------------------------------------------------------------------------
    def gpus(self, refresh: bool = False) -> list[DeviceInfo]:
        if self._gpus is None or refresh:
            self._gpus = list(self.get_gpus_fn())
        return self._gpus

    def max_runners(self) -> int:
        n = envconfig.max_runners()
        return n if n > 0 else 3 * max(1, len(self.gpus()))

    def free_memory(self) -> int:
        """Free VRAM of the node after subtracting what our own runners hold and the per-device reserve."""
        gpus = self.gpus(refresh=True)
        reserve = (GPU_OVERHEAD_DEFAULT + envconfig.gpu_overhead()) * len(gpus)
        total = sum(g.total_memory for g in gpus)
        reported = sum(g.free_memory for g in gpus)
        with self.lock:
            ours = sum(r.vram_size for r in self.loaded.values())
        return max(0, min(reported, total - ours) - reserve)

    # -- public API --------------------------------------------------------------------------------------
    def get_runner(self, model: Any, opts: dict[str, Any], keep_alive: float | None = None, batch_auto: bool = False) -> RunnerRef:
        key = getattr(model, "model_path", None) or getattr(model, "name", "")
        opts = dict(opts)
        if opts.get("num_ctx", 0) and opts["num_ctx"] < 4:
            opts["num_ctx"] = 4
        session = envconfig.keep_alive() if keep_alive is None else keep_alive
        ref = self._reuse(key, model, opts, session, batch_auto)
        if ref is not None:
            return ref
        with self.lock:
            if self.pending >= envconfig.max_queue():
                raise SchedulerError(ERR_MAX_QUEUE, 503)
            self.pending += 1
        try:
            with self.load_lock:          # one model loads at a time
                ref = self._reuse(key, model, opts, session, batch_auto)
                if ref is not None:
                    return ref
                with self.lock:
                    stale = self.loaded.get(key)
                if stale is not None:
                    self._evict(stale)
                ref = self._load(key, model, opts, session, batch_auto)
                with self.lock:
                    self.loaded[key] = ref
                    self._acquire(ref, session)
                    self.lock.notify_all()
                return ref
        finally:
            with self.lock:
                self.pending -= 1

    def _reuse(self, key: str, model: Any, opts: dict[str, Any], session: float, batch_auto: bool) -> RunnerRef | None:
        """The loaded runner of this model if it can serve the request.  It is pinned while it is probed, so that it cannot be
        evicted in between, and the probe itself runs without the lock."""
        with self.lock:
            ref = self.loaded.get(key)
            if ref is None or ref.options_differ(model, opts, batch_auto):
                return None
            self._acquire(ref, session)
        if ref.alive():
            return ref
        self.release(ref)
        return None

    def release(self, ref: RunnerRef) -> None:
        gone = None
        with self.lock:
            ref.ref_count = max(0, ref.ref_count - 1)
            if ref.ref_count == 0 and self.loaded.get(ref.model_key) is ref:
                if ref.session_duration <= 0:
                    gone = self._detach(ref)
                else:
                    self._arm_timer(ref)
            self.lock.notify_all()
        self._close(gone)

    def expire_runner(self, model: Any) -> None:
        """Unload as soon as the runner is idle (``keep_alive: 0`` with an empty prompt, ``ollama stop``)."""
        key = getattr(model, "model_path", None) or getattr(model, "name", "")
        gone = None
        with self.lock:
            ref = self.loaded.get(key)
            if ref is None:
                return
            ref.session_duration = 0
            ref.expires_at = self.now()
            if ref.ref_count == 0:
                gone = self._detach(ref)
        self._close(gone)

    def expire_for_runtime_oom(self, err: BaseException | str) -> bool:
        """A request died because the device ran out of memory while the model was running: let every runner expire as soon
        as it is idle (idle ones now), so that the next request loads onto an empty device.  True if ``err`` was such a failure."""
        if not is_out_of_memory(err):
            return False
        gone = []
        with self.lock:
            if self.loaded:
                log.warning("device memory ran out at run time; expiring %d loaded model(s): %s", len(self.loaded), err)
            for ref in list(self.loaded.values()):
                ref.session_duration = 0
                ref.expires_at = self.now()
                if ref.ref_count == 0:
                    gone.append(self._detach(ref))
        for ref in gone:
            self._close(ref)
        return True

    def unload_all(self) -> None:
        with self.lock:
            gone = [self._detach(ref) for ref in list(self.loaded.values())]
        for ref in gone:
            self._close(ref)

    def ps(self) -> list[RunnerRef]:
        with self.lock:
            return sorted(self.loaded.values(), key=lambda r: r.expires_at)

    # -- internals ---------------------------------------------------------------------------------------
    def _acquire(self, ref: RunnerRef, session: float) -> None:
        ref.ref_count += 1
        ref.session_duration = session
        if ref.timer is not None:
            ref.timer.cancel()
            ref.timer = None
        ref.expires_at = math.inf if math.isinf(session) else self.now() + session

    def _arm_timer(self, ref: RunnerRef) -> None:
        if ref.timer is not None:
            ref.timer.cancel()
            ref.timer = None
        if math.isinf(ref.session_duration):
            ref.expires_at = math.inf
            return
        ref.expires_at = self.now() + ref.session_duration

        def fire():
            gone = None
            with self.lock:
                if self.loaded.get(ref.model_key) is ref and ref.ref_count == 0 and self.now() >= ref.expires_at - 1e-3:
                    gone = self._detach(ref)
                    self.lock.notify_all()
            self._close(gone)

        ref.timer = threading.Timer(ref.session_duration, fire)
        ref.timer.daemon = True
        ref.timer.start()

    def _detach(self, ref: RunnerRef) -> RunnerRef:
        """Take a runner out of the table (lock held).  The caller closes it after releasing the lock."""
        if ref.timer is not None:
            ref.timer.cancel()
            ref.timer = None
        if self.loaded.get(ref.model_key) is ref:
            del self.loaded[ref.model_key]
        return ref

    def _close(self, ref: RunnerRef | None, recover: bool = False) -> None:
        """Shut a detached runner down (lock not held); with ``recover`` also wait for its memory to show up as free."""
        if ref is None:
            return
        before = sum(g.free_memory for g in self.gpus(refresh=True)) if recover and ref.gpus and ref.vram_size else None
        try:
            ref.runner.close()
        except Exception as e:  # a runner that fails to shut down is dropped anyway
            log.warning("runner close failed: %s", e)
        if before is not None:
            self._await_recovery(before, ref.vram_size)
        with self.lock:
            self.lock.notify_all()

    def _await_recovery(self, free_before: int, expect: int) -> bool:
        """Free memory as the driver reports it lags behind a process exit: poll until about three quarters of what the runner
        held is back, or give up after ``wait_for_recovery`` seconds and let the estimate stand (server/sched.go:1441-1499)."""
        deadline = time.monotonic() + self.wait_for_recovery
        while True:
            free_now = sum(g.free_memory for g in self.gpus(refresh=True))
            if free_now - free_before > 0.75 * expect:
                return True
            if time.monotonic() >= deadline:
                log.debug("GPU memory did not come back within %.1f s (before %d, now %d)", self.wait_for_recovery, free_before, free_now)
                return False
            time.sleep(min(0.25, max(0.0, deadline - time.monotonic())))

    def _evict(self, ref: RunnerRef, recover: bool = True) -> None:
        """Wait (bounded) until nobody uses the runner, then unload it; called without the lock."""
        deadline = time.monotonic() + 600
        with self.lock:
            while ref.ref_count > 0 and time.monotonic() < deadline:
                self.lock.wait(timeout=0.05)
            if self.loaded.get(ref.model_key) is not ref:
                return                             # somebody else already unloaded it
            self._detach(ref)
        self._close(ref, recover=recover)

    def _find_runner_to_unload(self) -> RunnerRef | None:
        with self.lock:
            refs = sorted(self.loaded.values(), key=lambda r: (r.session_duration, r.model_key))
        for r in refs:
            if r.ref_count == 0:
                return r
        return refs[0] if refs else None

    def _load(self, key: str, model: Any, opts: dict[str, Any], session: float, batch_auto: bool = False) -> RunnerRef:
        gpus = self.gpus(refresh=True)
        num_parallel = max(1, envconfig.num_parallel())
        caps = getattr(model, "capabilities", lambda: [])()
        if "embedding" in caps:
            num_parallel = 1                       # pooling models run one sequence at a time (sched.go:497-510)
        auto_ctx = not opts.get("num_ctx")
        if auto_ctx:
            opts["num_ctx"] = default_context(gpus) if gpus else 4096
        # make room: model count first, then memory
        while True:
            with self.lock:
                if len(self.loaded) < self.max_runners():
                    break
            victim = self._find_runner_to_unload()
            if victim is None:
                break
            self._evict(victim)
        ladder = [opts["num_ctx"]] + ([c for c in (32768, 4096) if c < opts["num_ctx"]] if auto_ctx else [])
        last_err: Exception | None = None
        for attempt, ctx in enumerate(ladder):
            opts["num_ctx"] = ctx
            one_gpu = max((g.free_memory for g in gpus), default=0)
            need = predict_memory(model, ctx, num_parallel, free=one_gpu or None)
            copies = max(1, min(envconfig.replicas(), len(gpus))) if gpus else 1
            if gpus:
                while need * copies > self.free_memory():
                    victim = self._find_runner_to_unload()
                    if victim is None:
                        break
                    self._evict(victim)
                if need > self.free_memory() and attempt + 1 < len(ladder):
                    continue                      # automatic context shrinks 256k -> 32k -> 4k before giving up (sched.go:649-669)
            use = self._place(gpus, need) if copies == 1 else self._place_copies(gpus, need, copies)
            if batch_auto and "embedding" not in caps:
                opts["num_batch"] = auto_num_batch(ctx * num_parallel, need, sum(g.free_memory for g in use))
            try:
                t0 = time.time()
                runner = self.new_runner_fn(model, dict(opts), num_parallel, use)
                mem = runner.memory() if hasattr(runner, "memory") else {}
                ref = RunnerRef(key, model, runner, runner_options(opts), num_parallel, 0, session, total_size=int(mem.get("total", need)),
                                vram_size=int(mem.get("vram", need if gpus else 0)), gpus=[g.id for g in use], loaded_at=time.time(),
                                context_length=int(getattr(runner, "n_ctx", ctx)), batch_auto=batch_auto)
                log.info("loaded %s in %.2fs (ctx %d x %d slots, batch %s, %d GPUs)", key, time.time() - t0, ctx, num_parallel,
                         opts.get("num_batch"), len(use))
                return ref
            except MemoryError as e:
                last_err = e
                with self.lock:                   # out of memory: unload everything else and retry once (sched.go:641-673)
                    idle = [self._detach(r) for r in list(self.loaded.values()) if r.ref_count == 0]
                for r in idle:
                    self._close(r, recover=True)
                continue
            except Exception as e:
                raise SchedulerError(f"failed to load model: {e}", 500) from e
        raise SchedulerError(f"model requires more system memory than is available: {last_err}", 500)

    @classmethod
    def _place_copies(cls, gpus: list[DeviceInfo], need: int, copies: int) -> list[DeviceInfo]:
        """GPUs for ``copies`` whole copies of a model: the group one copy needs, that many times over, on distinct devices
        (most free memory first); fewer copies when the node does not have the devices."""
        one = cls._place(gpus, need)
        k = len(one)
        by_free = sorted(gpus, key=lambda g: -g.free_memory)
        n = max(1, min(copies, len(by_free) // k))
        return by_free[:n * k]

    @staticmethod
    def _place(gpus: list[DeviceInfo], need: int) -> list[DeviceInfo]:
        """The smallest group of 1, 2, 4, ... GPUs (most free memory first) whose members can each hold their share within
        80 % of their free memory; every GPU when no such group exists."""
        if not gpus:
            return []
        if envconfig.sched_spread():
            return list(gpus)
        by_free = sorted(gpus, key=lambda g: -g.free_memory)
        k = 1
        while k <= len(by_free):                     # 1, 2, 4, 8 ... GPUs: group sizes a tensor-parallel split divides by
            group = by_free[:k]
            if need <= 0.8 * k * min(g.free_memory for g in group):
                return group
            k *= 2
        return list(gpus)


def _default_runner(model: Any, opts: dict[str, Any], num_parallel: int, gpus: list[DeviceInfo]):
    from ..engine.runner import Runner, RunnerOptions
    want = envconfig.replicas()
    if want > 1 and len(gpus) >= 2:
        # data-parallel copies: the placement's GPUs are dealt out in equal groups, one runner per group
        n = min(want, len(gpus))
        per = len(gpus) // n
        from ..engine.replicas import ReplicaSet
        return ReplicaSet(lambda i: _default_runner_on(model, opts, num_parallel, gpus[i * per:(i + 1) * per]), n)
    return _default_runner_on(model, opts, num_parallel, gpus)


def _default_runner_on(model: Any, opts: dict[str, Any], num_parallel: int, gpus: list[DeviceInfo]):
    from ..engine.runner import Runner, RunnerOptions
    device = envconfig.device()
    if len(gpus) == 1 and device in ("auto", "cuda"):
        device = f"cuda:{gpus[0].index}"            # the GPU the placement chose, not whichever is current
    ro = RunnerOptions(num_ctx=int(opts.get("num_ctx") or 4096), num_batch=int(opts.get("num_batch") or 512), num_parallel=num_parallel,
                       kv_cache_type=envconfig.kv_cache_type() or "f16", device=device, tp=max(1, len(gpus)),
                       gpu_ids=tuple(g.index for g in gpus),
                       adapter_paths=tuple(getattr(model, "adapter_paths", None) or ()),
                       draft_path=(getattr(model, "draft_paths", None) or [""])[0],
                       draft_num_predict=int(opts.get("draft_num_predict") if opts.get("draft_num_predict") is not None else 4))
    try:
        return Runner(model.model_path, ro)
    except RuntimeError as e:
        if "out of memory" in str(e).lower():
            raise MemoryError(str(e)) from e
        raise
