"""Token choice for the rows of a step: greedy, or temperature with top-k / top-p and a
repetition penalty on the tokens generated so far (src/frontend/sampler/sampler.cpp:195-318).

Everything runs in the CUDA kernels of ``csrc/sampling.cu``; one device-to-host copy brings the
chosen tokens back.  The reference draws from one generator shared by all requests
(src/zedinfer/scheduler.cpp:576-601), so its draws depend on what else is in the batch; here the
uniform number of a draw is a function of (request seed, index of the generated token) alone.
"""
from __future__ import annotations

import os
from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import ops

_MASK = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def uniform_for(seed: int, index: int) -> float:
    """A number in [0, 1) with 24 random bits, from (seed, index)."""
    z = _splitmix64(_splitmix64(seed & _MASK) ^ ((index + 1) * 0xD1342543DE82EF95 & _MASK))
    return (z >> 40) / float(1 << 24)


def fresh_seed() -> int:
    return int.from_bytes(os.urandom(8), "little") | 1


class PendingTokens:
    """Tokens chosen on the device and on their way to the host; ``wait()`` returns them as a list."""

    def __init__(self, device_tokens: torch.Tensor, host: torch.Tensor, event: torch.cuda.Event,
                 rows: Optional[int] = None, chosen_with_step: bool = False):
        self.device_tokens, self._host, self._event = device_tokens, host, event
        self._rows = host.numel() - 1 if rows is None else rows
        self.chosen_with_step = chosen_with_step        # the step's own graph chose the tokens (EngineCore.step_greedy)
        self.drawn = False                              # ... by the rows' own sampling options, not all by argmax

    def wait(self) -> List[int]:
        """The tokens; raises if a kernel of the step reported that one of its bounded waits ran out (the last
        element of the copy is the kernels' status word)."""
        self._event.synchronize()
        values = self._host.tolist()
        if values[-1] != 0:
            ops.tcgen05_status(self.device_tokens.device)            # reads and clears the word
            raise ops.KernelError(f"a bounded wait ran out inside a kernel of this step (code {values[-1]}); its output is not valid")
        return values[:self._rows]


class Sampler:
    def __init__(self, device: torch.device, core=None):
        """``core``: an ``EngineCore`` that keeps a table of generated tokens per request (``count_generated``); the
        repetition penalty then works from that table on the device and the generated tokens never travel.  Without
        it the tokens generated so far are sent with every step that penalises them."""
        self.device = device
        self.core = core if core is not None and getattr(core, "generated_counts", None) is not None else None
        self._pinned: List[torch.Tensor] = []
        self._turn = 0

    # ---- the table of generated tokens ---------------------------------------------------------
    @staticmethod
    def _penalised(r) -> bool:
        return not r.config.use_argmax and r.config.repetition_penalty != 1.0

    def _count_slot(self, r, ahead: int) -> Optional[int]:
        """The slot of ``r``'s table of generated tokens, brought up to the ``len(r.output_ids) + ahead`` tokens that
        have been chosen for it; -1 if ``r`` needs none; None if that cannot be done here (no table is kept, or the
        table is behind while tokens are still on their way to the host)."""
        if not self._penalised(r):
            return -1
        if self.core is None:
            return None
        rc = self.core.cache.get(r.request_id)
        if rc is None or rc.slot < 0:
            return None
        if r.count_serial != rc.serial:                # a slot fresh from open(): zero
            r.count_serial, r.counted = rc.serial, 0
        expected = len(r.output_ids) + ahead
        if r.counted != expected:
            if ahead or r.counted > expected:
                return None
            missing = torch.tensor(r.output_ids[r.counted:], dtype=torch.int32).to(self.device, non_blocking=True)
            ops.count_token_list(self.core.generated_counts[rc.slot], missing)
            r.counted = expected
        return rc.slot

    def counted(self, requests: Sequence) -> None:
        """A step has chosen one more token for each of these requests and added it to their tables."""
        if self.core is not None:
            for r in requests:
                if self._penalised(r):
                    r.counted += 1

    def _host_buffer(self, rows: int) -> torch.Tensor:
        """One of a few pinned buffers, taken in turn (a copy is waited for before its buffer comes round again)."""
        if not self._pinned:
            self._pinned = [torch.empty(256, dtype=torch.int32).pin_memory() for _ in range(4)]
        self._turn = (self._turn + 1) % len(self._pinned)
        if self._pinned[self._turn].numel() < rows:
            self._pinned[self._turn] = torch.empty(rows, dtype=torch.int32).pin_memory()
        return self._pinned[self._turn][:rows]

    def from_step(self, tokens_and_status: torch.Tensor, rows: int) -> PendingTokens:
        """Tokens that the step's own graph chose (``EngineCore.step_greedy``): int32 on the device, the first
        ``rows`` entries the tokens, the last the kernels' status word.  Starts their copy to the host."""
        host = self._host_buffer(tokens_and_status.numel())
        host.copy_(tokens_and_status, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return PendingTokens(tokens_and_status[:rows], host, event, rows=rows, chosen_with_step=True)

    def params(self, requests: Sequence, ahead: int = 0):
        """The rows' options as arrays: float32 ``[4, rows]`` (temperature, 0 for greedy rows; top_p; the uniform
        number of this draw; repetition penalty) and int32 ``[2, rows]`` (top_k; the slot of the row's table of
        generated tokens, -1 where no penalty applies).  None if a row needs a repetition penalty and no table is
        kept (or it is not up to date): the penalty then works on the logits with the tokens from the host."""
        rows = len(requests)
        par = np.zeros((4, rows), dtype=np.float32)
        par[1, :] = 1.0
        par[3, :] = 1.0
        ints = np.zeros((2, rows), dtype=np.int32)
        ints[1, :] = -1
        for i, r in enumerate(requests):
            c = r.config
            if c.use_argmax:
                continue
            slot = self._count_slot(r, ahead)
            if slot is None:
                return None
            par[0, i], par[1, i], par[3, i] = c.temperature, c.top_p, c.repetition_penalty
            par[2, i] = uniform_for(r.sample_seed, len(r.output_ids) + ahead)
            ints[0, i], ints[1, i] = c.top_k, slot
        return par, ints

    def sample(self, logits: torch.Tensor, requests: Sequence) -> List[int]:
        """One token per row of ``logits`` (float32 ``[rows, vocab]``); ``requests[i]`` gives row i's options."""
        return self.launch(logits, requests).wait()

    def launch(self, logits: torch.Tensor, requests: Sequence, ahead: int = 0) -> PendingTokens:
        """Choose the tokens on the device and start their copy to the host without waiting for it.

        ``ahead``: how many tokens of each request are chosen but not yet appended to ``output_ids`` (1 when this
        step was launched before the host read the step before it); it moves the index of the random draw.
        """
        rows = logits.shape[0]
        if rows != len(requests):
            raise ValueError(f"{rows} rows of logits for {len(requests)} requests")
        out = torch.empty(rows, dtype=torch.int32, device=self.device)
        if all(r.config.use_argmax for r in requests):
            ops.argmax(logits, out)
        else:
            sampling = self.params(requests, ahead)
            if sampling is not None:
                par, ints = sampling
                fl = torch.from_numpy(par).to(self.device, non_blocking=True)
                it = torch.from_numpy(ints).to(self.device, non_blocking=True)
                if self.core is not None:
                    ops.penalty_rows(logits, self.core.generated_counts, it[1], fl[3])
                ops.sample(logits, out, fl[0], it[0], fl[1], fl[2])
                if self.core is not None:
                    ops.count_tokens(self.core.generated_counts, it[1], out)
                    self.counted(requests)
            else:
                # no table of generated tokens: they go up with the step
                par = np.zeros((3, rows), dtype=np.float32)      # temperature, top_p, uniform
                par[1, :] = 1.0
                top_k = np.zeros(rows, dtype=np.int32)
                for i, r in enumerate(requests):
                    c = r.config
                    if c.use_argmax:
                        continue
                    par[0, i], par[1, i] = c.temperature, c.top_p
                    par[2, i] = uniform_for(r.sample_seed, len(r.output_ids) + ahead)
                    top_k[i] = c.top_k
                    if c.repetition_penalty != 1.0 and r.output_ids:
                        if ahead:
                            raise ValueError("a repetition penalty needs the tokens of the step before on the host")
                        recent = torch.tensor(r.output_ids, dtype=torch.int32).to(self.device, non_blocking=True)
                        ops.repetition_penalty(logits[i], recent, c.repetition_penalty)
                fl = torch.from_numpy(par).to(self.device, non_blocking=True)
                tk = torch.from_numpy(top_k).to(self.device, non_blocking=True)
                ops.sample(logits, out, fl[0], tk, fl[1], fl[2])
        host = self._host_buffer(rows + 1)
        host[:rows].copy_(out, non_blocking=True)
        host[rows:].copy_(ops.status_word(self.device), non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return PendingTokens(out, host, event)
