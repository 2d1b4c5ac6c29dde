"""The Python entry point, in the manner of the reference's engine and serving loop
(include/zedinfer/engine.hpp:85-202, include/zedinfer/serving_loop.hpp:31-81):

    engine = InferenceEngine.create(model_path, SchedulerConfig(...), dtype="bfloat16")
    result = engine.generate_tokens(prompt_ids, GenerationConfig(max_new_tokens=32))
    future = engine.submit_async(InferenceRequest(prompt_ids, config)); engine.run_loop(); future.result()

Requests are token ids in, token ids out: tokenizer and chat templates are not part of this engine.
"""
from __future__ import annotations

import os
import time
from typing import Callable, List, Optional, Sequence, Tuple

import torch

from ..config.engine_config import GenerationConfig, SchedulerConfig, sampling_defaults
from ..sampling.sampler import Sampler, fresh_seed
from ..cache.pool import OutOfPages
from .core import EngineCore, StepEntry
from .request import GenerationResult, InferenceRequest, RequestPhase
from .scheduler import ScheduledBatch, Scheduler


class RequestFuture:
    """Handle returned by :meth:`InferenceEngine.submit_async`; ``result()`` is ready once the request finished."""

    def __init__(self, request: InferenceRequest):
        self.request = request

    def done(self) -> bool:
        return self.request.phase == RequestPhase.COMPLETE

    def result(self) -> GenerationResult:
        if not self.done():
            raise RuntimeError("the request has not finished; drive the engine with step() or run_loop()")
        return self.request.result()


class InferenceEngine:
    def __init__(self, core: EngineCore, scheduler_config: SchedulerConfig):
        self.core = core
        self.scheduler_config = scheduler_config
        core.cuda_graphs = bool(scheduler_config.cuda_graphs)
        self.scheduler = Scheduler(scheduler_config, core.cache, core.max_seq_len, core.spec.eos_token_ids)
        self.sampler = Sampler(core.device, core)
        self.steps_run = 0
        self.steps_run_ahead = 0
        self.on_step: Optional[Callable[[ScheduledBatch], None]] = None
        # how a request is sampled that brings no sampling options of its own (GenerationConfig.has_sampling_override)
        self.default_generation = GenerationConfig(use_argmax=True, has_sampling_override=True)
        self._pending: Optional[Tuple[ScheduledBatch, object]] = None     # a launched step whose tokens are on their way

    @classmethod
    def create(cls, model_path: str, scheduler_config: Optional[SchedulerConfig] = None, dtype="bfloat16",
               device="cuda:0", random_seed: Optional[int] = None) -> "InferenceEngine":
        """``model_path``: a folder with config.json and *.safetensors.  With ``random_seed`` it may be a config.json
        alone (or a folder that holds one): the weights are then drawn on the device from that seed, which is how
        shapes too large to write out as a folder are measured."""
        cfg = scheduler_config or SchedulerConfig()
        cfg.validate()
        sizes = dict(page_size=cfg.kv_block_size, num_pages=cfg.num_kv_pages,
                     gpu_memory_utilization=cfg.gpu_memory_utilization, max_requests=cfg.max_batch_requests,
                     max_seq_len=cfg.max_seq_len, device=device, max_step_tokens=cfg.max_batch_tokens,
                     count_generated=True)
        if random_seed is None:
            core = EngineCore(model_path, dtype, **sizes)
        else:
            from ..config.registry import read_config_json
            core = EngineCore(None, dtype, config=read_config_json(model_path), random_seed=int(random_seed), **sizes)
        engine = cls(core, cfg)
        engine.default_generation = sampling_defaults(model_path)      # the folder's generation_config.json, if any
        if os.environ.get("ZEDINFER_DISABLE_WARMUP") is None:            # as the reference (src/zedinfer/engine.cpp:506-516)
            engine.warmup()
        return engine

    def warmup(self) -> None:
        """A short prompt and a few decode steps of random ids: kernel libraries are compiled and loaded and the
        decode step for one request is captured before the first real request comes.  Skipped when the pool is too
        small for it; a failure here is left for the first request to report."""
        c = self.core.cache
        room = min(self.core.max_seq_len, min(c.free_pages()) * c.page_size if c.groups else self.core.max_seq_len)
        n = min(16, room - 4)
        if n < 2:
            return
        try:
            self.profile(n, 3)
        except (OutOfPages, ValueError):
            pass

    # ---- intake -----------------------------------------------------------------------------
    def submit_async(self, request: InferenceRequest) -> RequestFuture:
        request.config = request.config.with_sampling_of(self.default_generation)
        request.sample_seed = request.config.seed if request.config.seed != 0 else fresh_seed()
        request.arrival_time = time.perf_counter()
        self.scheduler.submit(request)
        return RequestFuture(request)

    def generate_tokens(self, input_ids: Sequence[int], config: Optional[GenerationConfig] = None,
                        stream_callback=None) -> GenerationResult:
        """Run one request to its end on the caller's thread (src/zedinfer/serving_loop.cpp:97-107)."""
        fut = self.submit_async(InferenceRequest(list(input_ids), config, stream_callback))
        while not fut.done():
            if not self.step():
                break
        return fut.result()

    def generate_batch(self, prompts: Sequence[Sequence[int]], config: Optional[GenerationConfig] = None
                       ) -> List[GenerationResult]:
        futs = [self.submit_async(InferenceRequest(list(p), config)) for p in prompts]
        self.run_loop()
        return [f.result() for f in futs]

    # ---- the loop ---------------------------------------------------------------------------
    def has_work(self) -> bool:
        return self._pending is not None or self.scheduler.has_work()

    def run_loop(self) -> None:
        """Step until every submitted request has finished (src/zedinfer/serving_loop.cpp:424-430)."""
        while self.has_work():
            self.step()

    def entries_for(self, batch: ScheduledBatch) -> List[StepEntry]:
        entries = [StepEntry(r.request_id, [r.output_ids[-1]], [0]) for r in batch.decode_requests]
        for r, start, size, completes in zip(batch.prefill_requests, batch.prefill_chunk_starts,
                                             batch.prefill_chunk_sizes, batch.prefill_completes):
            seq = r.sequence()
            want = [size - 1] if completes else []
            entries.append(StepEntry(r.request_id, seq[start:start + size], want))
        return entries

    def step(self) -> bool:
        """schedule → forward → sample → process results.  Returns False when there was nothing to do.

        While a steady decode runs (the same requests step after step, nothing waiting), the next step is launched
        before this one's tokens have reached the host: it takes them on the device.  The host then reads this
        step's tokens while the GPU already works, so its bookkeeping costs no GPU time.  A request that ends with
        this step's token has a row in the step launched ahead; that row's result is dropped.
        """
        pending = self._pending
        self._pending = None
        if pending is None:
            batch = self.scheduler.schedule()
            if batch.empty():
                return self.scheduler.has_work()
            if self.on_step is not None:
                self.on_step(batch)
            try:
                entries = self.entries_for(batch)
                chosen = None
                if not batch.prefill_requests and batch.decode_requests:
                    # step and choice in one graph, where that goes: greedy rows by argmax, else each row's own draw
                    sampling = None
                    fused = True
                    if not all(r.config.use_argmax for r in batch.decode_requests):
                        sampling = self.sampler.params(batch.decode_requests)
                        fused = sampling is not None
                    picked = self.core.step_greedy(entries, sampling) if fused else None
                    if picked is not None:
                        chosen = self.sampler.from_step(picked, len(entries))
                        chosen.drawn = sampling is not None
                        if sampling is not None:
                            self.sampler.counted(batch.decode_requests)
                if chosen is None:
                    logits = self.core.step(entries)
                    rows = batch.rows_wanted()
                    chosen = self.sampler.launch(logits, [r for r, _ in rows]) if rows else None
            except Exception as e:                       # keep serving: fail what was in the step
                self.scheduler.fail_batch(batch, f"step failed: {e}")
                if isinstance(e, (torch.cuda.OutOfMemoryError, KeyboardInterrupt)):
                    raise
                return True
            pending = (batch, chosen)
        batch, chosen = pending
        try:
            if chosen is not None and self._may_run_ahead(batch):
                self._pending = self._launch_ahead(batch, chosen)
            tokens = chosen.wait() if chosen is not None else []
        except Exception as e:
            self._pending = None
            self.scheduler.fail_batch(batch, f"step failed: {e}")
            if isinstance(e, (torch.cuda.OutOfMemoryError, KeyboardInterrupt)):
                raise
            return True
        self.scheduler.process_results(batch, tokens)
        self.steps_run += 1
        return True

    def _may_run_ahead(self, batch: ScheduledBatch) -> bool:
        """A pure decode step whose requests all go on unless this step's token ends them, and nothing is waiting."""
        if not self.scheduler_config.run_ahead or not self.core.cuda_graphs or batch.prefill_requests:
            return False
        if self.scheduler.waiting or len(batch.decode_requests) != len(self.scheduler.active):
            return False
        for r in batch.decode_requests:
            if r.cancelled or r.phase == RequestPhase.COMPLETE or len(r.output_ids) + 2 > r.max_new_tokens:
                return False
            if not r.config.use_argmax and r.config.repetition_penalty != 1.0 and self.sampler.core is None:
                return False          # the penalty needs the generated tokens on the host
        return True

    def _launch_ahead(self, batch: ScheduledBatch, chosen) -> Optional[Tuple[ScheduledBatch, object]]:
        fused = chosen.chosen_with_step
        sampling = None
        if fused and getattr(chosen, "drawn", False):
            sampling = self.sampler.params(batch.decode_requests, ahead=1)
            if sampling is None:
                return None
        out = self.core.step_ahead([r.request_id for r in batch.decode_requests], None if fused else chosen.device_tokens,
                                   greedy=fused, sampling=sampling)
        if out is None:
            return None
        nxt = ScheduledBatch(decode_requests=list(batch.decode_requests))
        if self.on_step is not None:
            self.on_step(nxt)
        self.steps_run_ahead += 1
        if fused:
            pending = self.sampler.from_step(out, len(nxt.decode_requests))
            pending.drawn = sampling is not None
            if sampling is not None:
                self.sampler.counted(nxt.decode_requests)
            return nxt, pending
        return nxt, self.sampler.launch(out, nxt.decode_requests, ahead=1)

    # ---- measurement (src/zedinfer/profiler.cpp:119-162) ------------------------------------
    def profile(self, prefill_len: int, decode_len: int, seed: int = 12345) -> Tuple[float, float]:
        """One request of random ids: milliseconds for the prompt, and for ``decode_len - 1`` decode steps."""
        g = torch.Generator().manual_seed(seed)
        vocab = self.core.spec.vocab_size
        lo, hi = (100, vocab - 100) if vocab > 300 else (0, vocab)
        ids = torch.randint(lo, hi, (prefill_len,), generator=g).tolist()
        rid = ("profile", time.perf_counter_ns())
        start, mid, end = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        out = torch.empty(1, dtype=torch.int32, device=self.core.device)
        try:
            torch.cuda.synchronize()
            start.record()
            bound = self.core.cache.step_bound or prefill_len      # portions, where the pools ask for them
            for at in range(0, prefill_len, bound):
                part = ids[at:at + bound]
                logits = self.core.step([StepEntry(rid, part, [len(part) - 1] if at + bound >= prefill_len else [])])
            from .. import ops
            ops.argmax(logits, out)
            tok = int(out.item())
            mid.record()
            for _ in range(decode_len - 1):
                logits = self.core.step([StepEntry(rid, [tok], [0])])
                ops.argmax(logits, out)
                tok = int(out.item())
            end.record()
            self.core.check_kernels()
        finally:
            self.core.end(rid)
        return start.elapsed_time(mid), mid.elapsed_time(end)

    def cache_stats(self) -> dict:
        c = self.core.cache
        pool = sum(g.tensor.numel() * g.tensor.element_size() for g in c.groups if g.tensor is not None)
        return {"page_size": c.page_size, "pages_per_group": [g.num_pages for g in c.groups], "pool_tokens": c.num_pages * c.page_size, "pool_bytes": pool, "free_pages": c.free_pages(),
                "live_requests": c.num_live, "groups": len(c.groups), "preemptions": self.scheduler.num_preemptions}
