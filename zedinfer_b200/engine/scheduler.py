"""Continuous batching above the step function: admission, portions of prompts under a token
budget, decoding, finishing and freeing.

Policy of the reference (src/zedinfer/scheduler.cpp:267-394): every step first gives each
running request one decode token while the token budget lasts; then requests are admitted from
the head of the waiting queue only (FIFO, no skipping), their prompts cut into portions under
``min(remaining budget, max_prefill_tokens)``; a request whose prompt is not finished stays at the
head and blocks admission, so at most one request is in mid-prompt.  A request is admitted when
pages for its whole prompt (plus ``generation_reserve``) are free, and takes them at once.  A
request that can never be admitted, because nothing else is running that could give pages back,
fails right away (tests/zedinfer/test_scheduler_sampling.cpp:104-131 of the reference).

When pages run out while decoding, the reference fails the request
(src/zedinfer/scheduler.cpp:293-318).  Here that is ``on_exhaust="fail"``; the default
``"preempt"`` takes the youngest running request off the GPU instead: its pages are freed, and it
goes back to the head of the queue (behind a request that is in the middle of its prompt, which holds
its pages) with prompt := prompt + generated, to be recomputed when pages are free again.  Older
requests therefore always finish.

The scheduler decides on the host and never touches the device: it works against the cache
manager's bookkeeping, so it is tested without a GPU.
"""
from __future__ import annotations

import collections
import os
import sys
import threading
import time
from dataclasses import dataclass, field
from typing import Deque, List, Optional, Sequence, Tuple

from ..cache.manager import CacheManager

# ZEDINFER_DUMP_TOKEN_IDS=1: every committed token id goes to stderr (src/zedinfer/scheduler.cpp:561-564); read once
_DUMP_TOKEN_IDS = os.environ.get("ZEDINFER_DUMP_TOKEN_IDS", "")[:1] == "1"
from ..cache.pool import OutOfPages
from ..config.engine_config import SchedulerConfig, resolve_max_new_tokens
from .request import InferenceRequest, RequestPhase


@dataclass
class ScheduledBatch:
    """What one step holds: decode requests first, then prompt portions (batch_context.cpp:25-82)."""
    decode_requests: List[InferenceRequest] = field(default_factory=list)
    prefill_requests: List[InferenceRequest] = field(default_factory=list)
    prefill_chunk_starts: List[int] = field(default_factory=list)
    prefill_chunk_sizes: List[int] = field(default_factory=list)
    prefill_completes: List[bool] = field(default_factory=list)     # this portion ends the request's sequence

    def empty(self) -> bool:
        return not self.decode_requests and not self.prefill_requests

    def num_tokens(self) -> int:
        return len(self.decode_requests) + sum(self.prefill_chunk_sizes)

    def rows_wanted(self) -> List[Tuple[InferenceRequest, bool]]:
        """(request, is_prefill) for each logits row the step returns, in order."""
        rows = [(r, False) for r in self.decode_requests]
        for r, completes in zip(self.prefill_requests, self.prefill_completes):
            if completes:
                rows.append((r, True))
        return rows


class Scheduler:
    def __init__(self, config: SchedulerConfig, cache: CacheManager, max_seq_len: int,
                 stop_token_ids: Sequence[int] = ()):
        config.validate()
        self.config = config
        self.cache = cache
        self.max_seq_len = int(max_seq_len)
        self.stop_token_ids = frozenset(int(t) for t in stop_token_ids)
        self.waiting: Deque[InferenceRequest] = collections.deque()
        self.active: List[InferenceRequest] = []
        self.finished: List[InferenceRequest] = []
        self._lock = threading.Lock()
        self.num_preemptions = 0

    # ---- intake ---------------------------------------------------------------------------
    def submit(self, req: InferenceRequest) -> None:
        req.config.validate()
        if not req.input_ids:
            raise ValueError("a request needs at least one prompt token")
        req.max_new_tokens = resolve_max_new_tokens(req.config.max_new_tokens, len(req.input_ids), self.max_seq_len)
        with self._lock:
            if len(self.waiting) >= self.config.max_queue_size:
                raise RuntimeError("Queue full")
            self.waiting.append(req)

    def has_work(self) -> bool:
        return bool(self.waiting) or bool(self.active)

    # ---- finishing ------------------------------------------------------------------------
    def _release(self, req: InferenceRequest) -> None:
        if req.cache is not None:
            self.cache.close(req.cache)
            req.cache = None

    def _complete(self, req: InferenceRequest, reason: str, error: Optional[str] = None) -> None:
        req.phase = RequestPhase.COMPLETE
        req.finish_reason, req.error = reason, error
        now = time.perf_counter()
        req.stats.generated_tokens = len(req.output_ids)
        req.stats.total_time_ms = (now - req.arrival_time) * 1000.0
        if req.first_token_time is not None:
            req.stats.decode_time_ms = (now - req.first_token_time) * 1000.0
        self._release(req)
        self.finished.append(req)

    def _preempt(self, req: InferenceRequest) -> None:
        """Take a running request off the GPU; it will be recomputed from prompt + generated."""
        self._release(req)
        req.phase = RequestPhase.WAITING
        req.prefill_progress = 0
        req.stats.preemptions += 1
        self.num_preemptions += 1
        self.active.remove(req)
        # to the head of the queue, but behind a request that is in the middle of its prompt: that one holds its
        # pages and is the only one the admission looks at, so it has to stay first or neither could go on
        with self._lock:
            at = 0
            while at < len(self.waiting) and self.waiting[at].cache is not None:
                at += 1
            self.waiting.insert(at, req)

    def cancel(self, req: InferenceRequest) -> None:
        req.cancelled = True

    # ---- one scheduling decision ------------------------------------------------------------
    def _tokens_to_reserve(self, req: InferenceRequest) -> int:
        left_to_generate = max(0, req.max_new_tokens - len(req.output_ids))
        return len(req.sequence()) + min(left_to_generate, self.config.generation_reserve)

    def can_admit(self, req: InferenceRequest) -> bool:
        if req.cache is None and not self.cache.can_open():
            return False
        return self.cache.can_ensure(req.cache, self._tokens_to_reserve(req))

    def schedule(self) -> ScheduledBatch:
        batch = ScheduledBatch()
        token_budget = self.config.max_batch_tokens

        # 1. decode first
        for req in list(self.active):
            if token_budget <= 0:
                break
            if req.phase == RequestPhase.COMPLETE or req not in self.active:
                continue
            if req.cancelled:
                self.active.remove(req)
                self._complete(req, "cancelled")
                continue
            while True:
                try:
                    self.cache.ensure(req.cache, req.cache.length + 1)
                    batch.decode_requests.append(req)
                    token_budget -= 1
                    break
                except OutOfPages as e:
                    if self.config.on_exhaust == "fail":
                        self.active.remove(req)
                        self._complete(req, "error", f"KV cache exhausted during decode for request "
                                                     f"{req.request_id}: {e}")
                        break
                    victim = self.active[-1]                 # the youngest running request
                    if victim in batch.decode_requests:
                        batch.decode_requests.remove(victim)
                        token_budget += 1
                    self._preempt(victim)
                    if victim is req:
                        break

        # 2. admit from the head of the queue
        prefill_budget = min(token_budget, self.config.max_prefill_tokens)
        with self._lock:
            while self.waiting and prefill_budget > 0:
                req = self.waiting[0]
                if req.cancelled:
                    self.waiting.popleft()
                    self._complete(req, "cancelled")
                    continue
                # Requests whose prompt ends in this step are in ``active`` already.  (The reference adds the step's
                # prompt portions to that number once more, src/zedinfer/scheduler.cpp:338-341, and so admits half of
                # the free places per step; the limit means the same here, the queue just empties sooner.)
                if len(self.active) >= self.config.max_batch_requests:
                    break
                if req.cache is None:
                    if not self.can_admit(req):
                        nothing_running = batch.empty() and not self.active
                        if nothing_running:
                            self.waiting.popleft()
                            self._complete(req, "error",
                                           f"Cannot admit request {req.request_id}: prompt={len(req.sequence())} "
                                           f"tokens, free pages={self.cache.free_pages()}")
                            continue
                        break
                    req.cache = self.cache.open(req.request_id)
                    self.cache.ensure(req.cache, self._tokens_to_reserve(req))
                    if req.first_scheduled_time is None:
                        req.first_scheduled_time = time.perf_counter()
                        req.stats.queue_time_ms = (req.first_scheduled_time - req.arrival_time) * 1000.0
                seq_len = len(req.sequence())
                chunk = min(seq_len - req.prefill_progress, prefill_budget)
                batch.prefill_requests.append(req)
                batch.prefill_chunk_starts.append(req.prefill_progress)
                batch.prefill_chunk_sizes.append(chunk)
                batch.prefill_completes.append(req.prefill_progress + chunk >= seq_len)
                prefill_budget -= chunk
                req.phase = RequestPhase.PREFILL
                if req.prefill_progress + chunk >= seq_len:
                    self.waiting.popleft()
                    self.active.append(req)
                else:
                    break
        return batch

    # ---- after the step ---------------------------------------------------------------------
    def process_results(self, batch: ScheduledBatch, tokens: Sequence[int]) -> List[InferenceRequest]:
        """``tokens``: one sampled token per row of ``batch.rows_wanted()``.  Returns the requests that finished."""
        rows = batch.rows_wanted()
        if len(tokens) != len(rows):
            raise ValueError(f"{len(rows)} sampled tokens expected, got {len(tokens)}")
        before = len(self.finished)
        now = time.perf_counter()
        for req, start, size in zip(batch.prefill_requests, batch.prefill_chunk_starts, batch.prefill_chunk_sizes):
            req.prefill_progress = start + size
        for (req, was_prefill), tok in zip(rows, tokens):
            if req.phase == RequestPhase.COMPLETE:
                continue
            tok = int(tok)
            if was_prefill:
                req.phase = RequestPhase.DECODE
                if req.first_token_time is None:
                    req.first_token_time = now
                    req.stats.prefill_time_ms = (now - (req.first_scheduled_time or req.arrival_time)) * 1000.0
            req.output_ids.append(tok)
            if _DUMP_TOKEN_IDS:
                print(f"[token] request={req.request_id} index={len(req.output_ids) - 1} id={tok}", file=sys.stderr)
            req.prefill_progress = len(req.sequence()) - 1        # all but the token just sampled are cached
            if req.stream_callback is not None:
                try:
                    req.stream_callback(tok)
                except Exception as e:             # the caller's code: this request ends, the others go on
                    if req in self.active:
                        self.active.remove(req)
                    with self._lock:
                        if req in self.waiting:
                            self.waiting.remove(req)
                    self._complete(req, "error", f"stream callback raised: {e!r}")
                    continue
            if req.cancelled:
                self._finish_active(req, "cancelled")
            elif tok in self.stop_token_ids and not req.config.ignore_eos:
                self._finish_active(req, "stop")
            elif len(req.output_ids) >= req.max_new_tokens:
                self._finish_active(req, "length")
        return self.finished[before:]

    def _finish_active(self, req: InferenceRequest, reason: str) -> None:
        if req in self.active:
            self.active.remove(req)
        self._complete(req, reason)

    def fail_batch(self, batch: ScheduledBatch, message: str) -> None:
        """The step raised: fail what was in it and keep serving (src/zedinfer/serving_loop.cpp:467-495)."""
        for req in batch.decode_requests + batch.prefill_requests:
            if req.phase == RequestPhase.COMPLETE:
                continue
            if req in self.active:
                self.active.remove(req)
            with self._lock:
                if req in self.waiting:
                    self.waiting.remove(req)
            self._complete(req, "error", message)
