"""The step function: one batch of (request, its next tokens) through the model, from the cache.

:class:`EngineCore` owns the model, the cache manager and the device-side descriptor of a
step.  ``step(entries)`` takes any mix of prompt portions and single decoded tokens, cut
anywhere; it runs only the tokens it is given, appends their keys and values to the pages of
their requests, and returns float32 logits at the places asked for.  Generation, trace replay
and the benchmark all go through this one function.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import ops
from ..cache.manager import CacheManager, RequestCache, StateNeed
from ..config.registry import load_model_config
from ..parts.base import StepContext
from ..weights.loader import load_weights
from ..weights.random_init import random_tensors
from .descriptor import pack_step, step_padding, step_signature
from .model import Model

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def parse_dtype(dtype) -> torch.dtype:
    if dtype not in _DTYPES:
        raise ValueError(f"dtype must be 'bfloat16' or 'float32', got {dtype!r}")
    return _DTYPES[dtype]


@dataclass
class StepEntry:
    """A request's next tokens in one step, and the places (indices into ``tokens``) whose logits are wanted."""
    request_id: object
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)


def require_gpu(device) -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("zedinfer_b200 runs on an NVIDIA GPU only: no CUDA device is visible, "
                           "and there is no CPU path")
    dev = torch.device(device)
    if dev.type != "cuda":
        raise RuntimeError(f"zedinfer_b200 runs on an NVIDIA GPU only, not on {dev}")
    return dev


class PinnedStaging:
    """A few pinned staging buffers; a buffer is reused only after the copy out of it has finished."""

    def __init__(self, n: int = 4):
        self.bufs: List[Optional[torch.Tensor]] = [None] * n
        self.events: List[Optional[torch.cuda.Event]] = [None] * n
        self.i = 0
        self.bytes_staged = 0

    def stage_into(self, host: np.ndarray, dst: torch.Tensor) -> None:
        """Copy ``host`` into the device tensor ``dst`` (same length) through a pinned buffer."""
        i = self.i
        self.i = (i + 1) % len(self.bufs)
        if self.events[i] is not None:
            self.events[i].synchronize()
        buf = self.bufs[i]
        if buf is None or buf.numel() < host.size:
            buf = torch.empty(max(host.size, 4096), dtype=torch.int32).pin_memory()
            self.bufs[i] = buf
        buf[:host.size].numpy()[:] = host
        self.bytes_staged += host.size * 4
        dst.copy_(buf[:host.size], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.events[i] = ev

    def stage(self, host: np.ndarray, device: torch.device) -> torch.Tensor:
        i = self.i
        self.i = (i + 1) % len(self.bufs)
        if self.events[i] is not None:
            self.events[i].synchronize()
        buf = self.bufs[i]
        if buf is None or buf.numel() < host.size:
            buf = torch.empty(max(host.size, 4096), dtype=torch.int32).pin_memory()
            self.bufs[i] = buf
        buf[:host.size].numpy()[:] = host
        self.bytes_staged += host.size * 4
        dev = torch.empty(host.size, dtype=torch.int32, device=device)
        dev.copy_(buf[:host.size], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.events[i] = ev
        return dev


def build_step_context(entries: Sequence[StepEntry], rcs: Sequence[RequestCache], cache: CacheManager,
                       table_width: int, dtype: torch.dtype, device: torch.device, vocab: int,
                       ring: "PinnedStaging", pad_segments: int = 0,
                       into: Optional[torch.Tensor] = None, pos_width: int = 1
                       ) -> Tuple[StepContext, Optional[torch.Tensor]]:
    """Flatten the entries into one device descriptor (a single host-to-device copy; the layout is
    ``descriptor.pack_step``'s).  ``into``: a device buffer to hold the descriptor (a captured step's static buffer)
    instead of a fresh one; its length must fit."""
    n_groups = len(cache.groups)
    host, lay = pack_step([e.request_id for e in entries], [e.tokens for e in entries], [e.want for e in entries],
                          [rc.length for rc in rcs], [rc.slot for rc in rcs], [rc.tables for rc in rcs], n_groups,
                          table_width, vocab, cache.scratch_pages, ops.PREFILL_TILE_ROWS, pad_segments,
                          pos_width)
    n_seg, n_tok, width, total = lay.n_seg, lay.n_tok, lay.width, lay.total
    off_ids, off_pos, off_seg, off_want = lay.off_ids, lay.off_pos, lay.off_seg, lay.off_want
    off_slots, off_tiles, off_tab = lay.off_slots, lay.off_tiles, lay.off_tab
    n_want, n_real_want, n_tiles, lead = lay.n_want, lay.n_real_want, lay.n_tiles, lay.lead
    seg_start, seg_len, seg_pos0, slots, max_kv = lay.seg_start, lay.seg_len, lay.seg_pos0, lay.slots, lay.max_kv
    if into is None:
        dev = ring.stage(host, device)
    else:
        if into.numel() != total:
            raise ValueError(f"the step's descriptor has {total} entries, the static buffer {into.numel()}")
        ring.stage_into(host, into)
        dev = into
    tables = [dev[off_tab + g * n_seg * width: off_tab + (g + 1) * n_seg * width].view(n_seg, width)
              for g in range(n_groups)]
    ctx = StepContext(
        n_tokens=n_tok, n_segments=n_seg, dtype=dtype, device=device,
        token_ids=dev[off_ids: off_ids + n_tok], positions=dev[off_pos: off_pos + n_tok],
        tok_seg=dev[off_seg: off_seg + n_tok], tables=tables, slots=dev[off_slots: off_slots + n_seg],
        position_axes=dev[off_pos: off_pos + pos_width * n_tok].view(pos_width, n_tok),
        seg_start_host=seg_start, seg_len_host=seg_len, seg_pos0_host=seg_pos0, slots_host=slots,
        decode_only=all(k == 1 for k in seg_len), max_kv_len=max(max_kv, 1))
    ctx.extras["attn_tiles"] = dev[off_tiles: off_tiles + 3 * n_tiles].view(n_tiles, 3)
    ctx.extras["leading_singles"] = lead
    ctx.extras["real_want"] = n_real_want
    ctx.extras["descriptor_len"] = total
    want = dev[off_want: off_want + n_want] if n_want else None
    return ctx, want



class _SeenStep:
    """What is known of a step shape that has no graph: appearances, and the first one's timing."""
    __slots__ = ("count", "host_ms", "events", "gpu_bound")

    def __init__(self):
        self.count, self.host_ms, self.events, self.gpu_bound = 0, 0.0, None, None


COUNTS_KEY = ("sampler", "generated_counts")      # the cache key of the sampler's per-request state


class EngineCore:
    def __init__(self, model_dir: Optional[str], dtype="bfloat16", *, page_size: int = 16,
                 num_pages: Optional[int] = None, max_tokens: Optional[int] = None,
                 gpu_memory_utilization: float = 0.9, max_requests: int = 64, max_seq_len: Optional[int] = None,
                 device="cuda:0", cuda_graphs: bool = False, config: Optional[dict] = None,
                 random_seed: Optional[int] = None, max_step_tokens: Optional[int] = None,
                 init_scale: float = 1.0, count_generated: bool = False):
        """``num_pages``: pages of each cache group that keeps all keys; ``max_tokens``: size the pool for that many
        cached tokens instead; neither: whatever ``gpu_memory_utilization`` of the device leaves after the weights.
        ``max_step_tokens``: the caller's promise that no step brings more tokens of one request than this (a
        scheduler's token budget); groups of layers with a window then get pools only as large as ``max_requests``
        requests can fill, and the memory goes to the other groups.

        ``count_generated``: every request gets a slot of fixed-size state of the sampler's: how often it has
        generated each token of the vocabulary (int32 ``[vocab]``, ``generated_counts``), zero when the request
        starts.  The repetition penalty then works from that table on the device.  At most ``max_requests`` requests
        are live at a time then.

        ``model_dir=None`` with ``config`` (a config.json dict) and ``random_seed`` builds the model with
        random weights drawn on the device, without a folder (benchmarks of large shapes); the values are those
        that ``write_random_model(config, random_seed, ..., init_scale=init_scale)`` writes (weights/random_init.py)."""
        self.device = require_gpu(device)
        self.dtype = parse_dtype(dtype)
        torch.cuda.set_device(self.device)
        if model_dir is not None:
            self.arch, self.config, self.spec = load_model_config(model_dir)
            self.model = Model(self.spec)
            tensors = load_weights(model_dir, self.model.tensor_specs(), self.dtype, self.device)
        else:
            if config is None or random_seed is None:
                raise ValueError("without a model folder, give config= and random_seed=")
            from ..config.registry import resolve_architecture
            self.arch = resolve_architecture(config)
            self.config = self.arch.parse(config)
            self.spec = self.arch.build_spec(self.config)
            self.model = Model(self.spec)
            tensors = random_tensors(self.model.tensor_specs(), random_seed, self.dtype, init_scale=init_scale,
                                     device=self.device)
        self.model.bind(tensors, self.dtype, self.device)
        del tensors
        self.page_size = int(page_size)
        self.max_seq_len = min(int(max_seq_len or self.spec.max_position_embeddings),
                               self.spec.max_position_embeddings)
        needs = list(self.model.cache_needs())
        if count_generated:
            needs.append((COUNTS_KEY, StateNeed((self.spec.vocab_size,), torch.int32)))
        self.cache = CacheManager(needs, self.page_size, max_requests=max_requests, max_step_tokens=max_step_tokens)
        if num_pages is None and max_tokens is not None:
            num_pages = (int(max_tokens) + self.page_size - 1) // self.page_size
        if num_pages is None:
            torch.cuda.empty_cache()        # what loading freed again (tensors stacked into one) is free for the pool
            free, total = torch.cuda.mem_get_info(self.device)
            budget = int(total * gpu_memory_utilization) - (total - free)
            # leave room for the activations of a step
            budget -= 2 << 30
            num_pages = self.cache.pages_for_budget(max(budget, 0), self.dtype)
            per_request = (self.max_seq_len + self.page_size - 1) // self.page_size
            num_pages = min(num_pages, per_request * max_requests)
            if num_pages <= 0:
                raise RuntimeError("no device memory left for the cache after the weights "
                                   f"(free {free >> 20} MiB of {total >> 20} MiB, utilization {gpu_memory_utilization})")
        self.cache.allocate_device(int(num_pages), self.dtype, self.device)
        self.views = {call: self.cache.view_for_call(call) for call, _ in self.model.cache_needs()}
        # int32 [max_requests, vocab] or None: see count_generated
        self.generated_counts = self.cache.view_for_call(COUNTS_KEY).tensor if count_generated else None
        self.table_width = max(1, (self.max_seq_len + self.page_size - 1) // self.page_size)
        self._ring = PinnedStaging()
        self.cuda_graphs = bool(cuda_graphs)
        self.max_requests = int(max_requests)
        self._decode_graphs: Dict[tuple, "DecodeGraph"] = {}
        # decode steps whose requests all stay below this length have a captured graph of their own (decode_graph)
        self._short_reach = self.max_seq_len
        if self.dtype == torch.bfloat16:
            self._short_reach = min(self.max_seq_len, ops.decode_attention_split_from() - 1)
        self._last_decode_graph = None          # the graph the step before ran on, if it was a captured decode step
        self._step_graphs: Dict[tuple, "StepGraph"] = {}
        self._step_seen: Dict[tuple, _SeenStep] = {}
        self._graph_pool = None
        self.capture_blockers = self.model.capture_blockers()     # the parts that keep steps from being captured, by name
        self.capture_safe = not self.capture_blockers

    @staticmethod
    def kernel_libraries(dtype) -> List[str]:
        """The kernel libraries a run in ``dtype`` loads, for building them ahead of the first step."""
        libs = ["elementwise", "gemm_simt", "attention_generic", "sampling"]
        if parse_dtype(dtype) == torch.bfloat16:
            libs += ["attention_mma", "gemm_smallm"]      # the tcgen05 libraries are built when a step first needs them
        return libs

    # ---- requests -------------------------------------------------------------------------
    def request(self, request_id) -> Optional[RequestCache]:
        return self.cache.get(request_id)

    def end(self, request_id) -> None:
        rc = self.cache.get(request_id)
        if rc is not None:
            self.cache.close(rc)

    # ---- the step -------------------------------------------------------------------------
    def build_context(self, entries: Sequence[StepEntry], rcs: Sequence[RequestCache],
                      pad_segments: int = 0, into: Optional[torch.Tensor] = None
                      ) -> Tuple[StepContext, Optional[torch.Tensor]]:
        """Flatten the entries into one device descriptor (a single host-to-device copy)."""
        return build_step_context(entries, rcs, self.cache, self.table_width, self.dtype, self.device,
                                  self.spec.vocab_size, self._ring, pad_segments, into, self.spec.position_width)

    # Steps that are not pure decode are launched kernel by kernel, which costs the host a few milliseconds whatever
    # their size.  Every launch of such a step depends on the step's counts alone, so a step whose counts come back
    # (the full-size portions of a long prompt, the same portion beside the same number of decoding requests) is
    # captured in a CUDA graph at its second appearance and replayed from then on.
    MAX_STEP_GRAPHS = 32
    GPU_BOUND_RATIO = 1.25          # device time over host launch time from which a step shape is left eager

    def _step_padding(self, entries: Sequence[StepEntry]) -> int:
        return step_padding([len(e.tokens) for e in entries])

    def _step_signature(self, entries: Sequence[StepEntry], pad: int) -> tuple:
        return step_signature([len(e.tokens) for e in entries], sum(len(e.want) for e in entries), pad,
                              ops.PREFILL_TILE_ROWS)

    def _eager_or_captured(self, entries: Sequence[StepEntry], rcs: Sequence[RequestCache]) -> Optional[torch.Tensor]:
        """A step whose counts recur is replayed as a CUDA graph, if that can gain anything: its first appearance
        runs eagerly between two events and with a clock on the host.  If the GPU took clearly longer over it than
        the host took to launch it, the host keeps ahead of the GPU anyway, and the shape stays eager for good (a
        capture costs several eager launches).  Else it is captured at its second appearance."""
        from .decode_graph import StepGraph
        if not (self.cuda_graphs and self.capture_safe):
            ctx, want = self.build_context(entries, rcs)
            return self.model.forward(ctx, self.views, want)
        pad = self._step_padding(entries)
        sig = self._step_signature(entries, pad)
        g = self._step_graphs.pop(sig, None)
        if g is None:
            seen = self._step_seen.get(sig)
            if seen is None:
                if len(self._step_seen) > 4096:
                    self._step_seen.clear()
                seen = self._step_seen[sig] = _SeenStep()
            if seen.gpu_bound is None and seen.events is not None and seen.events[1].query():
                seen.gpu_bound = seen.events[0].elapsed_time(seen.events[1]) > self.GPU_BOUND_RATIO * seen.host_ms
                seen.events = None
            if seen.count == 0 or seen.gpu_bound or (seen.gpu_bound is None and seen.events is not None):
                first = seen.count == 0
                seen.count += 1
                if first:
                    seen.events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                    seen.events[0].record()
                    t0 = time.perf_counter()
                ctx, want = self.build_context(entries, rcs, pad_segments=pad)     # the shape a capture would have
                logits = self.model.forward(ctx, self.views, want)
                if first:
                    seen.host_ms = (time.perf_counter() - t0) * 1000.0
                    seen.events[1].record()
                real = ctx.extras["real_want"]                                      # the rows of padding tokens are dropped
                return None if logits is None or real == 0 else logits[:real]
            while len(self._step_graphs) >= self.MAX_STEP_GRAPHS:                   # the least recently used one goes
                del self._step_graphs[next(iter(self._step_graphs))]
            g = StepGraph(self, entries, rcs, pad)
        self._step_graphs[sig] = g                                                  # most recently used: last
        return g.run(entries, rcs)

    def check_kernels(self) -> None:
        """Wait for the device and raise if a kernel with bounded waits gave up since the last check.  Steps do not
        wait for this themselves: the word travels with the sampled tokens, and whoever reads logits calls this."""
        ops._tc_launched.pop(self.device, None)
        code = ops.tcgen05_status(self.device)          # reads the word: waits for everything launched so far
        if code:
            raise ops.KernelError(f"a bounded wait ran out inside a kernel (code {code}); the step's output is not valid")

    def prepare(self, entries: Sequence[StepEntry]) -> List[RequestCache]:
        """Open new requests and make sure every entry has pages for its tokens; all or nothing."""
        seen = set()
        for e in entries:
            if e.request_id in seen:
                raise ValueError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            if len(e.tokens) == 0:
                raise ValueError(f"request {e.request_id!r} brings no tokens")
            if self.cache.step_bound is not None and len(e.tokens) > self.cache.step_bound:
                raise ValueError(f"request {e.request_id!r} brings {len(e.tokens)} tokens in one step; the pools of this "
                                 f"model's windowed layers were sized for at most {self.cache.step_bound} (max_step_tokens)")
        opened: List[RequestCache] = []
        rcs: List[RequestCache] = []
        try:
            for e in entries:
                rc = self.cache.get(e.request_id)
                if rc is None:
                    rc = self.cache.open(e.request_id)
                    opened.append(rc)
                new_len = rc.length + len(e.tokens)
                if new_len > self.max_seq_len:
                    raise ValueError(f"request {e.request_id!r} would reach {new_len} tokens; the context limit "
                                     f"is {self.max_seq_len}")
                self.cache.ensure(rc, new_len)
                rcs.append(rc)
        except Exception:
            for rc in opened:
                self.cache.close(rc)
            raise
        return rcs

    def decode_graph(self, n: int, greedy: bool = False, sample: bool = False, longest: int = 0) -> "DecodeGraph":
        """The captured decode step for ``n`` requests (bucket: the next power of two).  ``greedy``: the form that
        also chooses the most likely token of every row and hands it to the next step on the device; ``sample``: the
        same with a draw by each row's own options.  ``longest``: the longest context among the requests after the
        step.  While it stays below the length from which the decode attention shares a request among clusters, the
        step is a graph captured for that reach, without the kernel that adds the clusters' parts (0.07 ms of a
        28-layer step); a longer request moves the step to the graph captured for the core's longest sequence."""
        from .decode_graph import DecodeGraph
        bucket = 1
        while bucket < n:
            bucket *= 2
        bucket = min(bucket, max(self.max_requests, n))
        reach = self.max_seq_len
        if self._short_reach < self.max_seq_len and longest <= self._short_reach:
            reach = self._short_reach
        key = (bucket, "sample" if sample else bool(greedy), reach)
        g = self._decode_graphs.get(key)
        if g is None:
            g = DecodeGraph(self, bucket, loop=bool(greedy), sample=bool(sample), reach=reach)
            self._decode_graphs[key] = g
        return g

    def step_greedy(self, entries: Sequence[StepEntry], sampling=None) -> Optional[torch.Tensor]:
        """A decode-only step of requests that all take their most likely token: step and choice are one captured
        graph.  ``sampling``: ``(par, top_k)`` as ``DecodeGraph.set_sampling`` takes them; the rows are then drawn by
        their own options instead (the sampling kernel inside the graph).  Returns int32 ``[bucket + 1]`` on the device (bucket >= n): the requests' tokens in the first n places,
        the kernels' status word in the last; or None when the step is not of that kind (the caller then uses
        :meth:`step` and samples himself)."""
        if not (entries and self.cuda_graphs and self.capture_safe and len(entries) <= self.max_requests
                and all(len(e.tokens) == 1 and tuple(e.want) == (0,) for e in entries)):
            return None
        rcs = self.prepare(entries)
        g = self.decode_graph(len(entries), greedy=sampling is None, sample=sampling is not None,
                              longest=max(rc.length for rc in rcs) + 1)
        if sampling is not None:
            g.set_sampling(*sampling)
        g.run(entries, rcs)
        self._last_decode_graph = g
        for rc in rcs:
            self.cache.commit(rc, rc.length + 1)
        return self._chosen(g, len(entries))

    @staticmethod
    def _chosen(g: "DecodeGraph", n: int) -> torch.Tensor:
        return g.sampled            # [bucket + 1]: the first n entries are the requests' tokens, the last the status word

    def step_ahead(self, request_ids: Sequence, sampled: Optional[torch.Tensor], greedy: bool = False,
                   sampling=None) -> Optional[torch.Tensor]:
        """One more decode step for exactly the requests of the decode step just launched, fed on the device with
        the tokens that step chose (``sampled``, int32, one per request) so the host need not have read them yet.
        Returns the logits, or None when this cannot be done (other requests in the captured step's rows, no page
        left): the caller then takes the ordinary path.  ``greedy`` / ``sampling``: the step before came from
        :meth:`step_greedy` in that form (its graph has handed the tokens on itself); the return value is then as that
        method's."""
        from ..cache.pool import OutOfPages
        rcs = [self.cache.get(rid) for rid in request_ids]
        if (not rcs or any(rc is None for rc in rcs) or not self.cuda_graphs or not self.capture_safe
                or len(rcs) > self.max_requests):
            return None
        g = self.decode_graph(len(rcs), greedy=greedy and sampling is None, sample=sampling is not None,
                              longest=max(rc.length for rc in rcs) + 1)
        if (not g.holds(rcs) or g is not self._last_decode_graph
                or any(rc.length + 1 > self.max_seq_len for rc in rcs)):
            return None
        try:
            for rc in rcs:
                self.cache.ensure(rc, rc.length + 1)
        except OutOfPages:
            return None
        if sampling is not None:
            g.set_sampling(*sampling)
        logits = g.run_ahead(rcs, sampled)
        for rc in rcs:
            self.cache.commit(rc, rc.length + 1)
        return self._chosen(g, len(rcs)) if (greedy or sampling is not None) else logits

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run one batch; returns float32 logits ``[wanted, vocab]`` on the device, or None if nothing is wanted."""
        if not entries:
            return None
        rcs = self.prepare(entries)
        if (self.cuda_graphs and self.capture_safe and len(entries) <= self.max_requests
                and all(len(e.tokens) == 1 and tuple(e.want) == (0,) for e in entries)):
            g = self.decode_graph(len(entries), longest=max(rc.length for rc in rcs) + 1)
            logits = g.run(entries, rcs)
            self._last_decode_graph = g
        else:
            self._last_decode_graph = None
            logits = self._eager_or_captured(entries, rcs)
        for e, rc in zip(entries, rcs):
            self.cache.commit(rc, rc.length + len(e.tokens))
        return logits
