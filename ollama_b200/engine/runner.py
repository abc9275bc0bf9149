"""The model runner: one loaded model, N slots, continuous batching.

This is the in-process replacement of the engine subprocess the reference spawns per model
(llm/server.go:59-78 lists the calls: Load, Ping, Completion, Embedding, Tokenize, Detokenize, Close,
MemorySize ...).  Semantics kept from there:

* ``num_parallel`` slots share a cache of ``num_ctx`` tokens each (llm/llama_server.go:375-376);
* a request reuses the slot whose cached tokens share the longest prefix with its prompt and always
  re-evaluates at least one token (``cache_prompt``, llm/llama_server.go:1562);
* when the context fills up, either the oldest half after ``num_keep`` is dropped (context shift,
  llm/llama_server.go:321-331) or generation ends with ``done_reason = "length"`` (:1713-1727);
* open-ended generation is bounded at 10 x num_ctx tokens (:106-118) and a run of more than 30
  identical tokens aborts the request (:1692-1703);
* final chunk carries prompt/eval counts and durations (:1503-1513, :1719-1727).
"""
from __future__ import annotations

import contextlib
import os
import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Iterator, Sequence

import torch

from ..text.tokenizer import Tokenizer, tokenizer_from_gguf
from .backend import make_backend, open_model
from .sampler import Sampler, SamplingParams, TokenLogprob


@dataclass
class RunnerOptions:
    num_ctx: int = 4096
    num_batch: int = 512
    num_parallel: int = 1
    kv_cache_type: str = "f16"
    device: str = "auto"
    flash_attention: bool = True
    tp: int = 1
    gpu_ids: tuple = ()               # device indices chosen by the scheduler (empty: devices 0..tp-1 / the current device)
    adapter_paths: tuple = ()         # LoRA adapter files merged into the weights at load time (Modelfile ADAPTER)
    draft_path: str = ""              # a smaller model of the same vocabulary that drafts tokens (Modelfile DRAFT)
    draft_num_predict: int = 4        # tokens drafted per verification pass (api/types.go:1119)
    shift_mode: str = "rotate"        # context shift: "rotate" re-rotates the cached keys in place, "recompute" evaluates the kept tokens again


@dataclass
class CompletionRequest:
    prompt: str | Sequence[int] = ""
    sampling: SamplingParams = field(default_factory=SamplingParams)
    num_predict: int = -1
    num_keep: int = 4
    stop: list[str] = field(default_factory=list)
    grammar: str | None = None
    grammar_after: str = ""           # the grammar starts to constrain only after this text was generated (end of a reasoning block)
    truncate: bool = True
    shift: bool = True
    cache_prompt: bool = True
    add_special: bool = True
    embedding: bool = False
    ignore_eos: bool = False
    preserved_tokens: bool = True     # render special tokens into the text stream (harmony needs them)
    images: list = field(default_factory=list)   # encoded images (bytes); image N replaces the marker "[img-N]" of a text prompt


@dataclass
class CompletionChunk:
    content: str = ""
    tokens: list[int] = field(default_factory=list)
    done: bool = False
    done_reason: str = ""
    prompt_eval_count: int = 0
    prompt_eval_duration: float = 0.0
    eval_count: int = 0
    eval_duration: float = 0.0
    cached_tokens: int = 0
    logprobs: list[TokenLogprob] = field(default_factory=list)
    embedding: list[float] | None = None
    error: str | None = None


class RunnerError(RuntimeError):
    def __init__(self, msg: str, status: int = 500):
        super().__init__(msg)
        self.status = status


class _Seq:
    def __init__(self, req: CompletionRequest, prompt: list[int]):
        self.req = req
        self.prompt = prompt
        self.slot = -1
        self.n_past = 0                 # tokens whose K/V are in the cache
        self.cached = 0
        self.generated: list[int] = []
        self.out: "queue.Queue[CompletionChunk]" = queue.Queue()
        self.state = "pending"          # pending -> prefill -> decode -> done
        self.sampler: Sampler | None = None
        self.grammar = None
        self.grammar_pending = ""       # grammar text waiting for ``grammar_after`` to appear in the output
        self.gate_text = ""
        self.next_token = -1
        self.pending_bytes = b""
        self.held_text = ""
        self.text_len = 0
        self.t_prefill = 0.0
        self.t_decode = 0.0
        self.t_submit = time.perf_counter()
        self.t_queue = 0.0              # waiting for a slot
        self.t_first = 0.0              # submit -> first sampled token
        self.d_past = 0                 # tokens whose K/V are in the draft model's cache
        self.n_decoded = 0
        self.n_prompt_eval = 0
        self.cancelled = False
        self.repeat_run = 0
        self.logprobs: list[TokenLogprob] = []
        self.limit = 0
        self.pixels: list[tuple[int, torch.Tensor]] = []    # (first prompt index, preprocessed image) until the tower has run
        self.image_rows: dict[int, torch.Tensor] = {}      # prompt index -> embedding row (image positions)
        self.spans: list[tuple[int, int]] = []              # prompt index ranges of the images: bidirectional attention inside


class Runner:
    PREFIX_COPY_MIN = 16              # a prefix held by another slot is copied when it is at least this much longer than the slot's own
    def __init__(self, model_path: str, opts: RunnerOptions | None = None, backend=None):
        self.opts = opts or RunnerOptions()
        self.path = model_path
        t0 = time.time()
        self.gguf = open_model(model_path) if model_path else None     # a ready backend may come without a file
        self._tp_group = None
        if backend is None and self._tp_devices():
            # the model is split over several GPUs: this process leads, one spawned follower per further GPU repeats its calls
            from ..parallel.launcher import TPGroup
            self._tp_group = TPGroup(model_path, self._tp_devices(), max_chunk=max(512, min(int(self.opts.num_batch), 2048)),
                                    kv_type=self.opts.kv_cache_type or "f16", adapters=tuple(self.opts.adapter_paths or ()))
            backend = self._tp_group.backend
        elif backend is None and self._pp_devices():
            # several GPUs, but the tensor-parallel split does not take this model: consecutive layers on consecutive GPUs
            from .pipeline import PipelineBackend
            src = None
            if self.opts.adapter_paths:
                from ..models.lora import LoraTensors
                src = LoraTensors(self.gguf, self.opts.adapter_paths)
            try:
                backend = PipelineBackend(self.gguf, self._pp_devices(), opts=self.opts, tensors=src)
            finally:
                if src is not None:
                    src.close()
        if backend is None:
            with self._on(self.opts.device):
                backend = make_backend(self.gguf, self.opts.device, opts=self.opts, adapters=tuple(self.opts.adapter_paths or ()))
        self.backend = backend
        # kernels are launched on the current device's stream: the loop thread and the calls below make the backend's
        # device current (a layer pipeline switches devices itself)
        dev = str(getattr(self.backend, "device", "")) if getattr(self.backend, "name", "") != "b200-pp" else ""
        self._cuda_device = dev if dev.startswith("cuda") else ""
        self.cfg = self.backend.cfg
        try:
            self.tokenizer: Tokenizer | None = tokenizer_from_gguf(self.gguf.kv) if self.gguf is not None else None
        except (ValueError, NotImplementedError):
            self.tokenizer = None
        n_ctx = max(4, int(self.opts.num_ctx))
        if self.cfg.ctx_train:
            n_ctx = min(n_ctx, self.cfg.ctx_train)          # llm/server.go:111-116
        self.n_ctx = n_ctx
        self.n_slots = max(1, int(self.opts.num_parallel))
        with self._on(self._cuda_device):
            self.backend.alloc(self.n_slots, self.n_ctx)
            self.draft = None
            if self.opts.draft_path and int(self.opts.draft_num_predict) > 0 and getattr(self.backend, "supports_verify", False):
                self._load_draft()
        self.slot_tokens: list[list[int]] = [[] for _ in range(self.n_slots)]
        self.slot_seq: list[_Seq | None] = [None] * self.n_slots
        self.slot_used_at = [0.0] * self.n_slots
        self.pending: list[_Seq] = []
        self.cv = threading.Condition()
        self.closed = False
        self.error: str | None = None
        self.load_duration = time.time() - t0
        # totals since load, written by the loop thread only (read by /metrics)
        self.stats: dict[str, float] = {k: 0 for k in (
            "requests", "prompt_tokens", "cached_prompt_tokens", "generated_tokens", "queue_seconds", "prefill_seconds",
            "decode_seconds", "ttft_seconds", "decode_steps", "decode_step_sequences", "context_shifts", "draft_tokens",
            "draft_accepted_tokens")}
        self.done_reasons: dict[str, int] = {}
        self._vision = None           # the vision tower, loaded with the first image
        self._vision_cfg = None       # its hyper-parameters (False: the model takes no images)
        self._nvtx = bool(os.environ.get("B200_NVTX")) and str(getattr(self.backend, "device", "cpu")).startswith("cuda")
        self.thread = threading.Thread(target=self._loop, name="runner-loop", daemon=True)
        self.thread.start()

    def _load_draft(self) -> None:
        """Speculative decoding: the draft model runs on the same device with its own slot-partitioned cache.  A draft
        whose vocabulary differs cannot propose ids of the target model and is ignored."""
        g = open_model(self.opts.draft_path)
        dev = str(getattr(self.backend, "device", self.opts.device))
        draft = make_backend(g, dev if dev.startswith("cuda") else "cpu", opts=self.opts) if dev.startswith("cuda") \
            else make_backend(g, "cpu")
        if draft.cfg.vocab_size != self.cfg.vocab_size:
            draft.close()
            return
        draft.alloc(self.n_slots, self.n_ctx)
        self.draft = draft

    # -- public calls -------------------------------------------------------------------------------
    def ping(self) -> bool:
        if self._tp_group is not None and not self._tp_group.alive():
            return False          # a follower process of the tensor-parallel group is gone: the scheduler reloads the model
        return not self.closed and self.thread.is_alive() and self.error is None

    def tokenize(self, text: str, add_special: bool = False, parse_special: bool = True) -> list[int]:
        if self.tokenizer is None:
            raise RunnerError("model has no tokenizer", 400)
        return self.tokenizer.encode(text, add_special=add_special, parse_special=parse_special)

    def detokenize(self, tokens: Sequence[int]) -> str:
        if self.tokenizer is None:
            raise RunnerError("model has no tokenizer", 400)
        return self.tokenizer.decode(tokens)

    def memory(self) -> dict:
        w, kv = self.backend.weight_bytes(), self.backend.kv_bytes()
        if self.draft is not None:
            w, kv = w + self.draft.weight_bytes(), kv + self.draft.kv_bytes()
        on_gpu = getattr(self.backend, "name", "torch") != "torch" or str(getattr(self.backend, "device", "cpu")).startswith("cuda")
        return {"weights": w, "kv": kv, "total": w + kv, "vram": (w + kv) if on_gpu else 0}

    def completion(self, req: CompletionRequest) -> Iterator[CompletionChunk]:
        seq = self.submit(req)
        try:
            while True:
                ch = seq.out.get()
                if ch.error:
                    raise RunnerError(ch.error)
                yield ch
                if ch.done:
                    return
        finally:
            seq.cancelled = True
            with self.cv:
                self.cv.notify_all()

    def submit(self, req: CompletionRequest) -> _Seq:
        if self.closed:
            raise RunnerError("runner is closed")
        pixels: list[tuple[int, torch.Tensor]] = []
        spans: list[tuple[int, int]] = []
        if isinstance(req.prompt, str):
            if req.images:
                toks, pixels, spans = self._tokenize_with_images(req)
            else:
                toks = self.tokenize(req.prompt, add_special=req.add_special)
        else:
            toks = [int(t) for t in req.prompt]
        if req.embedding and self.tokenizer is not None and self.tokenizer.add_eos is False and self.cfg.pooling == "last":
            if self.tokenizer.eos >= 0 and (not toks or toks[-1] != self.tokenizer.eos):
                toks = toks + [self.tokenizer.eos]
        if not toks:
            toks = [self.tokenizer.bos if self.tokenizer and self.tokenizer.bos >= 0 else 0]
        limit = self.n_ctx - 1
        if len(toks) > limit:
            if not req.truncate or req.embedding:
                raise RunnerError("the prompt is longer than the context length currently available to the model; shorten the "
                                  "prompt, adjust the context length in settings, or use a model with a longer context length", 400)
            if pixels:
                raise RunnerError("the prompt and its images are longer than the context length currently available to the model", 400)
            keep = min(max(req.num_keep, 0), limit // 2)
            toks = toks[:keep] + toks[len(toks) - (limit - keep):]
        seq = _Seq(req, toks)
        seq.pixels, seq.spans = pixels, spans
        with self.cv:
            self.pending.append(seq)
            self.cv.notify_all()
        return seq

    # -- images ---------------------------------------------------------------------------------------
    def vision(self):
        """The vision hyper-parameters of the model when this runner takes images (the file carries a tower and the back end takes
        embedding rows), else None.  Reads metadata only: safe from any thread."""
        if self._vision_cfg is None and self.gguf is not None and getattr(self.backend, "supports_embeds", False):
            from ..models.vision import vision_config_from_gguf
            self._vision_cfg = vision_config_from_gguf(self.gguf) or False
        return self._vision_cfg or None

    def _tower(self):
        """The vision tower on the model's device, loaded with the first image.  Runner thread only: loading and encoding
        allocate device memory, which must not happen on another thread while this one may be capturing a CUDA graph."""
        if self._vision is None:
            from ..models.vision import load_tower
            dev = self._cuda_device if self._cuda_device.startswith("cuda") else "cpu"
            self._vision = load_tower(self.gguf, dev)
        return self._vision

    def _encode_images(self, s: "_Seq") -> None:
        """Turn the pixels of a sequence's images into embedding rows (once, before its first prefill chunk)."""
        tower = self._tower()
        for lo, px in s.pixels:
            emb = tower.project(tower.patches(px))
            for j in range(emb.shape[0]):
                s.image_rows[lo + j] = emb[j]
        s.pixels = []

    def _tokenize_with_images(self, req: CompletionRequest):
        """Prompt text with ``[img-N]`` markers (server/prompt.go:96-133 writes them) -> token ids in which every image is a block
        ``\n\n <start_of_image> soft tokens <end_of_image> \n\n``; the soft positions carry ids below zero that are derived from
        the image's bytes (equal images share cached prefixes, different ones never do) and take their input from the vision
        tower's projection.  Returns (ids, {prompt index: embedding row}, [(first, last + 1) of each image])."""
        import hashlib
        import re
        vc = self.vision()
        if vc is None:
            raise RunnerError("this model does not take images", 400)
        from ..models.vision import preprocess
        tk = self.tokenizer
        boi, eoi = tk.vocab.get("<start_of_image>"), tk.vocab.get("<end_of_image>")
        parts = re.split(r"\[img-(\d+)\]", req.prompt)
        if len(parts) == 1:               # no marker at all: the images go in front, in order
            parts = sum([["", str(i)] for i in range(len(req.images))], []) + parts
        toks: list[int] = []
        pixels: list[tuple[int, torch.Tensor]] = []
        spans: list[tuple[int, int]] = []
        first = True
        for i, part in enumerate(parts):
            if i % 2 == 0:
                if part or first:
                    toks += self.tokenize(part, add_special=req.add_special and first)
                    first = False
                continue
            n = int(part)
            if not 0 <= n < len(req.images):
                raise RunnerError(f"the prompt names image {n} but the request has {len(req.images)}", 400)
            data = req.images[n]
            try:
                px = preprocess(data, vc.image_size)
            except Exception as e:
                raise RunnerError(f"image {n} could not be read: {e}", 400)
            h = int.from_bytes(hashlib.sha256(data).digest()[:4], "little")
            if first:
                toks += self.tokenize("", add_special=req.add_special)
                first = False
            toks += self.tokenize("\n\n", add_special=False)
            if boi is not None:
                toks.append(boi)
            lo = len(toks)
            pixels.append((lo, px))
            toks += [-(1 + ((h * 1000003 + j) & 0x3FFFFFFF)) for j in range(vc.tokens_per_image)]
            spans.append((lo, len(toks)))
            if eoi is not None:
                toks.append(eoi)
            toks += self.tokenize("\n\n", add_special=False)
        return toks, pixels, spans

    def embedding(self, text: str | Sequence[int]) -> tuple[list[float], int]:
        seq = self.submit(CompletionRequest(prompt=text, embedding=True, truncate=False))
        ch = seq.out.get()
        if ch.error:
            raise RunnerError(ch.error)
        return ch.embedding or [], ch.prompt_eval_count

    def _tp_devices(self) -> list[int]:
        """GPUs of a tensor-parallel group for this model ([] = single device): ``tp`` option or B200_TP, when the split divides the model."""
        from .. import envconfig
        tp = int(self.opts.tp) if int(self.opts.tp) > 1 else envconfig.tp_degree()
        if tp < 2 or self.gguf is None or str(self.opts.device).startswith("cpu"):
            return []
        import torch
        if not torch.cuda.is_available() or torch.cuda.device_count() < tp:
            return []
        try:
            from ..models.config import config_from_gguf
            from ..parallel.tp_engine import shard_plan
            cfg = config_from_gguf(self.gguf)
            shard_plan(cfg, tp, {n: t.dtype for n, t in self.gguf.tensors.items()})
            if cfg.sandwich_norm or cfg.d_model > 8192:
                return []
        except (ValueError, NotImplementedError):
            return []
        return self._pick(tp)

    def _pick(self, n: int) -> list[int]:
        """``n`` device indices: the scheduler's choice when it names enough devices, else 0..n-1."""
        ids = [int(i) for i in (self.opts.gpu_ids or ())]
        return ids[:n] if len(ids) >= n else list(range(n))

    def _pp_devices(self) -> list[int]:
        """GPUs of a layer pipeline ([] = none): B200_PP, or the GPUs meant for a tensor-parallel group that cannot be formed."""
        from .. import envconfig
        n = envconfig.pp_degree() or (int(self.opts.tp) if int(self.opts.tp) > 1 else envconfig.tp_degree())
        if n < 2 or self.gguf is None or str(self.opts.device).startswith("cpu"):
            return []
        import torch
        if not torch.cuda.is_available() or torch.cuda.device_count() < n:
            return []
        from ..models.config import config_from_gguf
        from .b200 import supports
        cfg = config_from_gguf(self.gguf)
        return self._pick(n) if supports(cfg) and cfg.n_layers >= n else []

    def close(self) -> None:
        with self.cv:
            self.closed = True
            self.cv.notify_all()
        self.thread.join(timeout=30)
        if self._tp_group is not None:
            self._tp_group.close()
        else:
            self.backend.close()
        if self.draft is not None:
            self.draft.close()
        if self.gguf is not None:
            self.gguf.close()

    # -- batching loop -------------------------------------------------------------------------------
    @staticmethod
    def _on(device: str):
        """Context that makes ``device`` ("cuda:N") the current CUDA device; a no-op for anything else."""
        if isinstance(device, str) and device.startswith("cuda:") and torch.cuda.is_available():
            return torch.cuda.device(torch.device(device))
        return contextlib.nullcontext()

    def _loop(self) -> None:
        try:
            if self._cuda_device.startswith("cuda:") and torch.cuda.is_available():
                torch.cuda.set_device(torch.device(self._cuda_device))
            while True:
                with self.cv:
                    while not self.closed and not self.pending and not any(self.slot_seq):
                        self.cv.wait(timeout=0.5)
                    if self.closed:
                        break
                    self._admit()
                self._step()
        except Exception as e:  # a failed step poisons the runner; the scheduler replaces it
            import traceback
            self.error = f"{type(e).__name__}: {e}"
            traceback.print_exc()
            for s in list(self.slot_seq) + list(self.pending):
                if s is not None:
                    s.out.put(CompletionChunk(done=True, error=self.error))
            self.closed = True
        finally:
            for s in list(self.slot_seq) + list(self.pending):
                if s is not None and s.state != "done":
                    s.out.put(CompletionChunk(done=True, error=self.error or "runner closed"))

    def _admit(self) -> None:
        while self.pending:
            free = [i for i in range(self.n_slots) if self.slot_seq[i] is None]
            if not free:
                return
            seq = self.pending.pop(0)
            if seq.cancelled:
                continue
            best, best_lcp = free[0], -1
            for i in free:
                lcp = _common_prefix(self.slot_tokens[i], seq.prompt) if seq.req.cache_prompt else 0
                if lcp > best_lcp or (lcp == best_lcp and self.slot_used_at[i] < self.slot_used_at[best]):
                    best, best_lcp = i, lcp
            reuse = max(0, min(best_lcp, len(seq.prompt) - 1))   # always evaluate at least one token
            if seq.req.embedding or not self.cfg.causal:
                reuse = 0
            elif seq.req.cache_prompt and hasattr(self.backend, "copy_rows"):
                # a longer prefix of this prompt may sit in another slot, busy or not: its cache rows are copied over
                # (x/mlxrunner/prefix_cache.go:86-140 keeps such prefixes in a trie of snapshots; here the slots are the store)
                donor, donor_lcp = -1, reuse + self.PREFIX_COPY_MIN - 1
                for i in range(self.n_slots):
                    if i == best:
                        continue
                    other = self.slot_seq[i]
                    valid = self.slot_tokens[i] if other is None else self.slot_tokens[i][:other.n_past]
                    lcp = min(_common_prefix(valid, seq.prompt), len(seq.prompt) - 1)
                    if lcp > donor_lcp:
                        donor, donor_lcp = i, lcp
                if donor >= 0:
                    self.backend.copy_rows(donor, best, donor_lcp)
                    self.slot_tokens[best] = list(seq.prompt[:donor_lcp])
                    reuse = donor_lcp
                    self.stats["prefix_copies"] = self.stats.get("prefix_copies", 0) + 1
                    self.stats["prefix_copied_tokens"] = self.stats.get("prefix_copied_tokens", 0) + donor_lcp
            seq.slot, seq.n_past, seq.cached = best, reuse, reuse
            seq.d_past = 0
            seq.t_queue = time.perf_counter() - seq.t_submit
            del self.slot_tokens[best][reuse:]
            self.slot_seq[best] = seq
            seq.state = "prefill"
            r = seq.req
            try:
                seq.sampler = Sampler(r.sampling, self.cfg.vocab_size, self.n_ctx, history=seq.prompt)
                if r.grammar and r.grammar_after and self.tokenizer is not None:
                    seq.grammar_pending = r.grammar          # free-form reasoning first, constrained answer afterwards
                elif r.grammar:
                    from .grammar import Grammar
                    seq.grammar = Grammar(r.grammar, self.tokenizer)
            except Exception as e:      # a bad grammar or sampler setting is this request's problem only
                self._fail(seq, e)
                continue
            seq.limit = r.num_predict if r.num_predict >= 0 else 10 * self.n_ctx

    def _step(self) -> None:
        active = [s for s in self.slot_seq if s is not None]
        for s in active:
            if s.cancelled and s.state != "done":
                self._finish(s, "cancelled")
        # one prefill pass per iteration keeps decode latency of the other slots bounded; the pass takes rows of every
        # sequence that is waiting for its prompt, up to num_batch rows in all, when the backend can run them as one matrix
        waiting = [s for s in active if s.state == "prefill"]
        if len(waiting) > 1 and hasattr(self.backend, "prefill_many") and not any(s.req.embedding or s.image_rows or s.pixels for s in waiting):
            with self._range("prefill_batch"):
                self._prefill_batch(waiting)
        elif waiting:
            self._prefill_chunk(waiting[0])
        dec = [s for s in self.slot_seq if s is not None and s.state == "decode"]
        if dec:
            self._decode(dec)

    def _range(self, name: str):
        """NVTX range around a phase of the loop when B200_NVTX is set (shows up in Nsight timelines); a no-op otherwise."""
        if not self._nvtx:
            return contextlib.nullcontext()
        return torch.cuda.nvtx.range(name)

    def _prefill_chunk(self, s: _Seq) -> None:
        with self._range("prefill_chunk"):
            self._prefill_chunk_inner(s)

    def _prefill_chunk_inner(self, s: _Seq) -> None:
        t0 = time.perf_counter()
        remaining = len(s.prompt) - s.n_past
        n = min(remaining, max(1, self.opts.num_batch))
        for lo, hi in s.spans:            # the rows of an image attend to each other in both directions: one chunk holds them all
            if lo < s.n_past + n < hi:
                n = lo - s.n_past if lo > s.n_past else hi - s.n_past      # stop in front of the image, or take all of it
        chunk = s.prompt[s.n_past:s.n_past + n]
        last = n == remaining
        if s.req.embedding:
            hid = self.backend.hidden(s.slot, s.prompt)
            vec = _pool(hid.float(), self.cfg.pooling)
            _sync(hid)
            s.n_prompt_eval = len(s.prompt)
            s.out.put(CompletionChunk(done=True, done_reason="stop", embedding=vec.tolist(), prompt_eval_count=len(s.prompt),
                                      prompt_eval_duration=time.perf_counter() - t0))
            self.slot_tokens[s.slot] = []
            self._release(s)
            return
        if s.pixels:
            self._encode_images(s)
        if s.image_rows:
            rows = [i for i in range(n) if s.n_past + i in s.image_rows]
            embeds = (rows, torch.stack([s.image_rows[s.n_past + i] for i in rows])) if rows else None
            logits = self.backend.prefill(s.slot, chunk, s.n_past, need_logits=last, embeds=embeds, spans=s.spans)
        else:
            logits = self.backend.prefill(s.slot, chunk, s.n_past, need_logits=last)
        s.n_past += n
        s.n_prompt_eval += n
        self.slot_tokens[s.slot].extend(chunk)
        if last:
            s.state = "decode"
            self._sample_accept(s, logits)       # reads the logits: the chunk has finished on the device when this returns
            now = time.perf_counter()
            s.t_prefill += now - t0              # prompt-eval time includes the device's work, not only the host's enqueueing
            s.t_first = now - s.t_submit
        else:
            _sync(None)
            s.t_prefill += time.perf_counter() - t0

    def _prefill_batch(self, seqs: list[_Seq]) -> None:
        """One pass over prompt rows of several sequences: the row budget (num_batch) is filled in arrival order, so the request that
        came first reaches its first token first and short prompts ride along in what a longer one leaves over (the order in which
        the reference's runner packs the prompts of its slots into a batch)."""
        t0 = time.perf_counter()
        budget = max(1, self.opts.num_batch)
        left = {id(s): len(s.prompt) - s.n_past for s in seqs}
        take = {id(s): 0 for s in seqs}
        for s in seqs:
            if budget == 0:
                break
            take[id(s)] = min(left[id(s)], budget)
            budget -= take[id(s)]
        part = [s for s in seqs if take[id(s)] > 0]
        segs = [(s.slot, s.prompt[s.n_past:s.n_past + take[id(s)]], s.n_past) for s in part]
        last = [take[id(s)] == left[id(s)] for s in part]
        outs = self.backend.prefill_many(segs, last)
        if not any(last):
            _sync(None)
        self.stats["prefill_batches"] = self.stats.get("prefill_batches", 0) + 1
        for s, (_, chunk, _), done, logits in zip(part, segs, last, outs):
            s.n_past += len(chunk)
            s.n_prompt_eval += len(chunk)
            self.slot_tokens[s.slot].extend(chunk)
            if done:
                s.state = "decode"
                self._sample_accept(s, logits)   # reads the logits: the pass has finished on the device
                s.t_first = time.perf_counter() - s.t_submit
            s.t_prefill += time.perf_counter() - t0

    def _decode(self, seqs: list[_Seq]) -> None:
        with self._range("decode_step"):
            self._decode_inner(seqs)

    def _decode_inner(self, seqs: list[_Seq]) -> None:
        t0 = time.perf_counter()
        ready: list[_Seq] = []
        for s in seqs:
            if s.n_past + 1 > self.n_ctx:
                if not self._shift(s):
                    continue
            ready.append(s)
        if not ready:
            return
        slots = [s.slot for s in ready]
        toks = [s.next_token for s in ready]
        poss = [s.n_past for s in ready]
        plain = all(s.sampler.p.greedy and not s.sampler.p.has_penalties and s.grammar is None and not s.sampler.p.logprobs for s in ready)
        if self.draft is not None and plain and len(ready) == 1 and self._speculate(ready[0], t0):
            return
        fast = hasattr(self.backend, "decode_argmax") and plain
        if fast:
            out = self.backend.decode_argmax(slots, toks, poss)
            sampled = [(int(t), None) for t in out]
            for s, (t, _) in zip(ready, sampled):
                s.sampler.accept(t)
        else:
            logits = self.backend.decode(slots, toks, poss)
            sampled = [None] * len(ready)        # drawn per sequence below, so that one failing sampler stops one sequence
        dt = time.perf_counter() - t0
        self.stats["decode_steps"] += 1
        self.stats["decode_step_sequences"] += len(ready)
        for i, s in enumerate(ready):
            self.slot_tokens[s.slot].append(s.next_token)
            s.n_past += 1
            s.t_decode += dt
            s.n_decoded += 1
            if sampled[i] is None:
                self._sample_accept(s, logits[i])
            else:
                self._sample_accept(s, None, sampled[i])

    def _sample_accept(self, s: _Seq, logits, drawn: tuple | None = None) -> None:
        """Draw the next token of one sequence (unless ``drawn`` already holds it) and process it.

        Errors raised here come from this sequence's own sampler, grammar or stop handling (for instance a grammar
        that rejects every token the vocabulary offers): they end this sequence with an error chunk and leave the
        other slots running.  Device errors are not caught: they poison the runner and the scheduler replaces it.
        """
        try:
            tok, lp = drawn if drawn is not None else s.sampler.sample(logits, s.grammar.allows if s.grammar else None)
            self._accept(s, tok, lp)
        except Exception as e:
            if _is_device_error(e):
                raise
            self._fail(s, e)

    def _fail(self, s: _Seq, e: Exception) -> None:
        """End one sequence with an error chunk and free its slot."""
        if s.state == "done":
            return
        self.stats["failed_requests"] = self.stats.get("failed_requests", 0) + 1
        s.out.put(CompletionChunk(done=True, error=f"{type(e).__name__}: {e}"))
        if s.slot >= 0:
            self.slot_tokens[s.slot] = self.slot_tokens[s.slot][:s.n_past]
        self._release(s)

    def _speculate(self, s: _Seq, t0: float) -> bool:
        """One speculative step of a greedy sequence: the draft model proposes ``k`` tokens one by one, the target model
        scores the pending token and all proposals in one pass, and the longest prefix of proposals that the target
        would have produced itself is kept, plus the target's own next token.  Both caches are indexed by position, so
        rows written for rejected proposals are simply overwritten later.  Returns False when the step has to be an
        ordinary one (no room left in the context)."""
        k = int(self.opts.draft_num_predict)
        if s.n_past + k + 1 > self.n_ctx or len(s.generated) + k + 1 > s.limit:
            return False
        d, slot = self.draft, s.slot
        hist = self.slot_tokens[slot]
        if s.d_past < s.n_past:            # bring the draft cache up to date (the whole prompt at the first step)
            pos = s.d_past
            while pos < s.n_past:
                chunk = hist[pos:pos + max(1, self.opts.num_batch)]
                d.prefill(slot, chunk, pos, need_logits=False)
                pos += len(chunk)
            s.d_past = s.n_past
        proposals: list[int] = []
        tok = s.next_token
        for i in range(k):
            if hasattr(d, "decode_argmax"):
                tok = int(d.decode_argmax([slot], [tok], [s.n_past + i])[0])
            else:
                tok = int(d.decode([slot], [tok], [s.n_past + i])[0].argmax())
            proposals.append(tok)
        logits = self.backend.verify(slot, [s.next_token] + proposals, s.n_past)
        target = logits.argmax(-1).tolist()                 # target[i]: the token after position n_past + i
        n_ok = 0
        while n_ok < k and proposals[n_ok] == target[n_ok]:
            n_ok += 1
        produced = target[:n_ok + 1]
        dt = time.perf_counter() - t0
        st = self.stats
        st["decode_steps"] += 1
        st["decode_step_sequences"] += 1
        st["draft_tokens"] += k
        st["draft_accepted_tokens"] += n_ok
        s.d_past = s.n_past + min(n_ok + 1, k)               # draft inputs were the pending token and proposals 1..k-1
        s.t_decode += dt
        for tok in produced:
            hist.append(s.next_token)
            s.n_past += 1
            s.n_decoded += 1
            s.sampler.accept(tok)
            self._accept(s, tok, None)
            if s.state == "done":
                break
        return True

    def _shift(self, s: _Seq) -> bool:
        """Context is full: drop half of the tokens after ``num_keep`` and rebuild the cache for the rest."""
        if not s.req.shift:
            self._finish(s, "length")
            return False
        keep = min(max(s.req.num_keep, 0), self.n_ctx // 2)
        toks = self.slot_tokens[s.slot]
        discard = max(1, (len(toks) - keep) // 2)
        new = toks[:keep] + toks[keep + discard:]
        if hasattr(self.backend, "shift") and self.opts.shift_mode != "recompute":
            # the cache rows of the dropped tokens are removed and the keys behind them re-rotated to their new positions
            self.backend.shift(s.slot, keep, discard, len(toks))
        else:
            self.slot_tokens[s.slot] = new[:keep]
            tail = new[keep:]
            pos = keep
            while tail:
                chunk, tail = tail[: self.opts.num_batch], tail[self.opts.num_batch:]
                self.backend.prefill(s.slot, chunk, pos, need_logits=False)
                pos += len(chunk)
        self.slot_tokens[s.slot] = new
        s.n_past = len(new)
        s.d_past = 0                     # positions moved: the draft cache is rebuilt at the next speculative step
        self.stats["context_shifts"] += 1
        return True

    def _accept(self, s: _Seq, tok: int, lp: TokenLogprob | None) -> None:
        """Handle a freshly sampled token: stop conditions, detokenise, stream."""
        tk = self.tokenizer
        s.generated.append(tok)
        if s.grammar is not None:
            s.grammar.accept(tok)
        elif s.grammar_pending and tk is not None and 0 <= tok < tk.n_vocab:
            s.gate_text = (s.gate_text + tk.token_bytes(tok).decode("utf-8", "ignore"))[-4 * len(s.req.grammar_after) - 64:]
            if s.req.grammar_after in s.gate_text:
                from .grammar import Grammar
                s.grammar, s.grammar_pending = Grammar(s.grammar_pending, tk), ""
        if s.next_token == tok:
            s.repeat_run += 1
        else:
            s.repeat_run = 0
        s.next_token = tok
        if lp is not None:
            s.logprobs.append(lp)
        if tk is not None and tk.is_eog(tok) and not s.req.ignore_eos:
            s.generated.pop()
            self._flush(s, final=True)
            self._finish(s, "stop")
            return
        piece = b""
        if tk is not None:
            if 0 <= tok < tk.n_vocab and tk.types[tok] == 3 and not s.req.preserved_tokens:
                piece = b""               # control tokens are not part of the visible text; user-defined tokens are
            else:
                piece = tk.token_bytes(tok) if 0 <= tok < tk.n_vocab else b""
        s.pending_bytes += piece
        text, s.pending_bytes = _valid_utf8_prefix(s.pending_bytes)
        stopped = self._emit(s, text, [tok])
        if stopped:
            self._finish(s, "stop")
        elif s.grammar is not None and s.grammar.done():
            self._flush(s, final=True)
            self._finish(s, "stop")
        elif len(s.generated) >= s.limit:
            self._flush(s, final=True)
            self._finish(s, "length")
        elif s.repeat_run > 30:
            self._flush(s, final=True)
            self._finish(s, "stop")

    def _emit(self, s: _Seq, text: str, toks: list[int]) -> bool:
        """Stream ``text`` while holding back anything that may still turn into a stop string."""
        buf = s.held_text + text
        for st in s.req.stop:
            if st and st in buf:
                buf = buf[: buf.index(st)]
                s.held_text = ""
                if buf:
                    s.out.put(CompletionChunk(content=buf, tokens=toks, logprobs=self._take_lp(s)))
                return True
        hold = 0
        for st in s.req.stop:
            for k in range(min(len(st) - 1, len(buf)), 0, -1):
                if buf.endswith(st[:k]):
                    hold = max(hold, k)
                    break
        out, s.held_text = (buf[: len(buf) - hold], buf[len(buf) - hold:]) if hold else (buf, "")
        if out or toks:
            s.out.put(CompletionChunk(content=out, tokens=toks, logprobs=self._take_lp(s)))
        return False

    def _take_lp(self, s: _Seq) -> list[TokenLogprob]:
        lps, s.logprobs = s.logprobs, []
        return lps

    def _flush(self, s: _Seq, final: bool = False) -> None:
        text = s.held_text
        if final and s.pending_bytes:
            text += s.pending_bytes.decode("utf-8", errors="replace")
            s.pending_bytes = b""
        s.held_text = ""
        if text:
            s.out.put(CompletionChunk(content=text, logprobs=self._take_lp(s)))

    def _finish(self, s: _Seq, reason: str) -> None:
        if s.state == "done":
            return
        st = self.stats
        st["requests"] += 1
        st["prompt_tokens"] += len(s.prompt)
        st["cached_prompt_tokens"] += s.cached
        st["generated_tokens"] += len(s.generated)
        st["queue_seconds"] += s.t_queue
        st["prefill_seconds"] += s.t_prefill
        st["decode_seconds"] += s.t_decode
        st["ttft_seconds"] += s.t_first
        self.done_reasons[reason] = self.done_reasons.get(reason, 0) + 1
        s.out.put(CompletionChunk(done=True, done_reason=reason, prompt_eval_count=len(s.prompt),
                                  prompt_eval_duration=s.t_prefill, eval_count=len(s.generated), eval_duration=s.t_decode,
                                  cached_tokens=s.cached, logprobs=self._take_lp(s)))
        self._release(s)

    def _release(self, s: _Seq) -> None:
        s.state = "done"
        if s.slot >= 0 and self.slot_seq[s.slot] is s:
            self.slot_seq[s.slot] = None
            self.slot_used_at[s.slot] = time.time()


def _is_device_error(e: Exception) -> bool:
    """True for failures of the backend itself (CUDA runtime, kernel library, exchange time-outs) as opposed to host-side
    per-request logic."""
    from ..ops.cuda import CudaKernelError
    if isinstance(e, CudaKernelError):
        return True
    msg = str(e)
    return isinstance(e, RuntimeError) and ("CUDA" in msg or "cuda" in msg or "tensor-parallel exchange" in msg)


def _common_prefix(a: Sequence[int], b: Sequence[int]) -> int:
    n = min(len(a), len(b))
    i = 0
    while i < n and a[i] == b[i]:
        i += 1
    return i


def _valid_utf8_prefix(b: bytes) -> tuple[str, bytes]:
    """Split ``b`` into the longest decodable prefix and the incomplete trailing sequence."""
    if not b:
        return "", b""
    cut = len(b)
    for back in range(1, min(4, len(b)) + 1):
        c = b[-back]
        if c & 0xC0 == 0x80:
            continue
        need = 1 if c < 0x80 else 2 if c >> 5 == 0b110 else 3 if c >> 4 == 0b1110 else 4 if c >> 3 == 0b11110 else 1
        if need > back:
            cut = len(b) - back
        break
    return b[:cut].decode("utf-8", errors="replace"), b[cut:]


def _pool(hid: torch.Tensor, mode: str) -> torch.Tensor:
    if mode == "cls":
        return hid[0]
    if mode == "last":
        return hid[-1]
    return hid.mean(0)


def _sync(t) -> None:
    if torch.cuda.is_available():
        torch.cuda.synchronize()
