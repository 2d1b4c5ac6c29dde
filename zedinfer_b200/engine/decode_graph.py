"""A decode-only step captured as a CUDA graph.

A decode step launches a few hundred small kernels; issued one by one from the host they take
longer to launch than to run.  For every batch-size bucket the step is captured once over static
device buffers (token ids, positions, block tables) and replayed: the host then only refreshes
the buffers.  Requests missing from a bucket are padded with tokens that sit at position 0 of the
cache's scratch page, which nothing reads.  The captured work is the same ``Model.forward`` that
runs eagerly, so the two paths cannot drift apart.

``loop=True`` also captures the greedy choice and the hand-over of the chosen token to the next
step (ids := argmax, positions += 1), so that steps can be replayed back to back without the host;
the benchmark uses this to time the device alone.
"""
from __future__ import annotations

import contextlib
import gc
from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..parts.base import StepContext


@contextlib.contextmanager
def capturing(graph: "torch.cuda.CUDAGraph", pool=None):
    """``torch.cuda.graph`` with Python's cycle collector held still.  A collection that starts in the middle of a
    capture may destroy the CUDA graphs of an engine that is gone (they sit in reference cycles with it), and
    destroying a graph is not allowed while a stream captures: the capture is lost with "operation not permitted
    when stream is capturing".  So: collect first, then capture with the collector off."""
    gc.collect()
    was_enabled = gc.isenabled()
    gc.disable()
    try:
        with torch.cuda.graph(graph, pool=pool):
            yield
    finally:
        if was_enabled:
            gc.enable()


class DecodeGraph:
    def __init__(self, core, bucket: int, loop: bool = False, sample: bool = False, reach: Optional[int] = None):
        """``loop``: the graph also chooses a token per row and hands it to the next step on the device; the most
        likely token, or with ``sample`` a draw with the row's temperature, top-k, top-p and uniform number, which
        :meth:`set_sampling` brings before a replay (rows of temperature 0 take the most likely token).
        ``reach``: the longest context (after the step) that a request of a replay may have; the core's longest
        sequence if None.  Kernels plan their launches for it at capture."""
        self.core, self.bucket, self.loop, self.sample = core, bucket, loop or sample, sample
        self.reach = core.max_seq_len if reach is None else min(int(reach), core.max_seq_len)
        b, width, ng = bucket, core.table_width, len(core.cache.groups)
        pw = self.pos_width = core.spec.position_width          # position numbers per token, one run of b per axis
        self.off_ids, self.off_pos, self.off_seg = 0, b, (1 + pw) * b
        self.off_want, self.off_slots, self.off_tab = self.off_seg + b, self.off_seg + 2 * b, self.off_seg + 3 * b
        total = self.off_tab + ng * b * width
        self.host = np.zeros(total, dtype=np.int32)
        self.host[self.off_seg: self.off_seg + b] = np.arange(b)
        self.host[self.off_want: self.off_want + b] = np.arange(b)
        self._pad_rows(0)
        self.dev = torch.zeros(total, dtype=torch.int32, device=core.device)
        core._ring.stage_into(self.host, self.dev)
        self._slot_sig: List[Optional[tuple]] = [None] * b
        self._n_filled = 0
        d = self.dev
        tables = [d[self.off_tab + g * b * width: self.off_tab + (g + 1) * b * width].view(b, width) for g in range(ng)]
        self.ctx = StepContext(
            n_tokens=b, n_segments=b, dtype=core.dtype, device=core.device,
            token_ids=d[self.off_ids: self.off_ids + b], positions=d[self.off_pos: self.off_pos + b],
            tok_seg=d[self.off_seg: self.off_seg + b], tables=tables, slots=d[self.off_slots: self.off_slots + b],
            position_axes=d[self.off_pos: self.off_pos + pw * b].view(pw, b),
            seg_start_host=list(range(b)), seg_len_host=[1] * b, seg_pos0_host=[0] * b, slots_host=[-1] * b,
            decode_only=True, max_kv_len=self.reach)
        self.want = d[self.off_want: self.off_want + b]
        # loop: the tokens chosen by the step, and behind them the kernels' status word as the step left it
        self.sampled = torch.zeros(b + 1, dtype=torch.int32, device=core.device)
        # sample: temperature | top_p | uniform | repetition penalty (float32 bits) | top_k | slot of the request's
        # table of generated tokens (-1: none kept), one row of b each, sent in one copy
        self.par_host = np.zeros(6 * b, dtype=np.int32)
        self._blank_par()
        self.par = torch.zeros(6 * b, dtype=torch.int32, device=core.device)
        if sample:
            core._ring.stage_into(self.par_host, self.par)
        self.launches = 0
        # warm up on a side stream (loads the libraries, lets cuBLAS pick its kernels), then capture
        side = torch.cuda.Stream(device=core.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self._body()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        from ..ops import _lib
        before = _lib.launch_count()
        with capturing(self.graph):
            self.logits = self._body()
        self.launches = _lib.launch_count() - before

    def _body(self) -> torch.Tensor:
        logits = self.core.model.forward(self.ctx, self.core.views, self.want)
        if self.loop:
            b = self.bucket
            if self.sample:
                fl = self.par[:4 * b].view(torch.float32)
                counts, slots = self.core.generated_counts, self.par[5 * b:]
                if counts is not None:
                    ops.penalty_rows(logits, counts, slots, fl[3 * b:])
                ops.sample(logits, self.sampled[:b], fl[:b], self.par[4 * b: 5 * b], fl[b: 2 * b], fl[2 * b: 3 * b])
                if counts is not None:
                    ops.count_tokens(counts, slots, self.sampled[:b])
            else:
                ops.argmax(logits, self.sampled[:b])
            self.sampled[b:].copy_(ops.status_word(self.core.device))
            ops.advance_decode(self.ctx.token_ids, self.ctx.position_axes, self.sampled[:b])
        return logits

    def _blank_par(self) -> None:
        b, h = self.bucket, self.par_host
        h[:] = 0                                                  # temperature 0: greedy rows
        h[b: 2 * b] = np.float32(1.0).view(np.int32)              # top_p
        h[3 * b: 4 * b] = np.float32(1.0).view(np.int32)          # repetition penalty
        h[5 * b:] = -1                                            # no table of generated tokens

    def set_sampling(self, par: np.ndarray, ints: np.ndarray) -> None:
        """``par`` float32 ``[4, n]`` (temperature, top_p, uniform number, repetition penalty) and ``ints`` int32
        ``[2, n]`` (top_k, slot of the table of generated tokens or -1) for the first n rows of the next replay; the
        rows behind them are greedy."""
        b, n = self.bucket, par.shape[1]
        h = self.par_host
        self._blank_par()
        for k in range(4):
            h[k * b: k * b + n] = np.ascontiguousarray(par[k], dtype=np.float32).view(np.int32)
        h[4 * b: 4 * b + n] = ints[0]
        h[5 * b: 5 * b + n] = ints[1]
        self.core._ring.stage_into(h, self.par)

    def _pad_rows(self, first: int) -> None:
        b, width, ng = self.bucket, self.core.table_width, len(self.core.cache.groups)
        scratch = self.core.cache.scratch_pages
        h = self.host
        h[self.off_ids + first: self.off_ids + b] = 0
        for axis in range(self.pos_width):
            h[self.off_pos + axis * b + first: self.off_pos + (axis + 1) * b] = 0
        h[self.off_slots + first: self.off_slots + b] = -1
        for g in range(ng):
            base = self.off_tab + g * b * width
            rows = h[base: base + b * width].reshape(b, width)
            rows[first:, :] = scratch[g]       # wherever a padding row's position points (a looping graph moves it on)

    def _write_tables(self, i: int, rc) -> None:
        """Row ``i`` of every group's block table := the request's pages; entries that a window has passed and given
        back (-1) point at the scratch page, whose keys the kernels mask like any other outside the window."""
        b, width, h = self.bucket, self.core.table_width, self.host
        scratch = self.core.cache.scratch_pages
        for g in range(len(self.core.cache.groups)):
            tab = np.asarray(rc.tables[g], dtype=np.int32)
            base = self.off_tab + (g * b + i) * width
            h[base: base + tab.size] = np.where(tab < 0, scratch[g], tab)
            h[base + tab.size: base + width] = 0

    def fill(self, tokens: Sequence[int], rcs: Sequence, reserve_ahead: int = 0) -> None:
        """Refresh the static buffers for these requests (one token each) and upload what changed.

        Token ids and positions change every step and are always sent.  A row of block tables is rewritten only
        when another request sits in the slot or the request's tables changed (its ``version``), which for a
        steady decode is once every ``page_size`` steps; the tables go up only then.
        """
        n = len(rcs)
        b, width, ng = self.bucket, self.core.table_width, len(self.core.cache.groups)
        h = self.host
        vocab = self.core.spec.vocab_size
        toks = np.asarray(tokens, dtype=np.int64)
        if n and (toks.min() < 0 or toks.max() >= vocab):
            raise ValueError(f"token id outside [0, {vocab})")
        h[self.off_ids: self.off_ids + n] = toks
        for axis in range(self.pos_width):
            h[self.off_pos + axis * b: self.off_pos + axis * b + n] = [rc.length for rc in rcs]
        tables_dirty = False
        sigs = self._slot_sig
        for i, rc in enumerate(rcs):
            sig = (rc.request_id, rc.serial, rc.version)
            if sigs[i] == sig:
                continue
            sigs[i] = sig
            tables_dirty = True
            h[self.off_slots + i] = rc.slot
            self._write_tables(i, rc)
        if n != self._n_filled:
            self._pad_rows(n)
            for i in range(n, b):
                sigs[i] = None
            self._n_filled = n
            tables_dirty = True
        head = self.off_seg                                   # ids and positions
        if tables_dirty:
            self.core._ring.stage_into(h, self.dev)
        else:
            self.core._ring.stage_into(h[:head], self.dev[:head])

    def run(self, entries: Sequence, rcs: Sequence) -> torch.Tensor:
        self.fill([e.tokens[0] for e in entries], rcs)
        self.graph.replay()
        return self.logits[:len(entries)]

    def holds(self, rcs: Sequence) -> bool:
        """The last fill put exactly these requests into the first rows."""
        return len(rcs) == self._n_filled and all(sig is not None and sig[:2] == (rc.request_id, rc.serial)
                                                  for sig, rc in zip(self._slot_sig, rcs))

    def run_ahead(self, rcs: Sequence, sampled: torch.Tensor) -> torch.Tensor:
        """The step after the one just run, for the same requests, before the host knows their tokens: ids and
        positions move on the device (``sampled`` holds the tokens chosen by the last step); only block tables
        that changed go up."""
        n = len(rcs)
        b, width, ng = self.bucket, self.core.table_width, len(self.core.cache.groups)
        h = self.host
        dirty = False
        for i, rc in enumerate(rcs):
            sig = (rc.request_id, rc.serial, rc.version)
            if self._slot_sig[i] == sig:
                continue
            self._slot_sig[i] = sig
            dirty = True
            self._write_tables(i, rc)
        if dirty:
            head = self.off_seg                               # ids and positions stay as the device has them
            self.core._ring.stage_into(h[head:], self.dev[head:])
        if not self.loop:                                     # a looping graph has moved ids and positions on itself
            ops.advance_decode(self.ctx.token_ids, self.ctx.position_axes, sampled, n)
        self.graph.replay()
        return self.logits[:n]

    def replay(self) -> None:
        self.graph.replay()


class StepGraph:
    """Any step (portions of prompts, alone or beside decoding requests) captured as a CUDA graph.

    Everything the step's kernels are launched with depends on its counts only: tokens, segments, attention tiles
    and wanted rows.  Which token belongs to which request, the positions, the block tables and the tiles are
    data in the step's descriptor, which lives in a static device buffer here and is rewritten before each replay.
    The captured work is ``Model.forward``, as in the eager path.  All step graphs share one memory pool: they
    replay one at a time, and a step's logits are read before the next replay.
    """

    def __init__(self, core, entries: Sequence, rcs: Sequence, pad_segments: int = 0):
        self.core, self.pad = core, pad_segments
        probe_ctx, _ = core.build_context(entries, rcs, pad_segments=pad_segments)   # only to learn the descriptor's length
        self.dev = torch.zeros(probe_ctx.extras["descriptor_len"], dtype=torch.int32, device=core.device)
        self.ctx, self.want = core.build_context(entries, rcs, pad_segments=pad_segments, into=self.dev)
        if core._graph_pool is None:
            core._graph_pool = torch.cuda.graph_pool_handle()
        # the eager runs before this one loaded the libraries and let cuBLAS pick its kernels; capture
        torch.cuda.synchronize()
        ops._tc_launched.pop(core.device, None)
        self.graph = torch.cuda.CUDAGraph()
        with capturing(self.graph, pool=core._graph_pool):
            self.logits = core.model.forward(self.ctx, core.views, self.want)
        self.uses_status = bool(ops._tc_launched.get(core.device, False))

    def run(self, entries: Sequence, rcs: Sequence) -> Optional[torch.Tensor]:
        pad = self.ctx.n_segments - len(entries)      # same counts, so the same layout: the views are the captured ones
        ctx, _ = self.core.build_context(entries, rcs, pad_segments=pad, into=self.dev)
        if ctx.n_tokens != self.ctx.n_tokens or ctx.n_segments != self.ctx.n_segments:
            raise RuntimeError("a step was given to a graph captured for other counts")
        self.graph.replay()
        if self.uses_status:
            ops._tc_launched[self.core.device] = True
        real = ctx.extras["real_want"]                    # the rows of padding tokens are dropped
        return None if self.logits is None or real == 0 else self.logits[:real]
