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
    def __init__(self, device: torch.device):
        self.device = device
        self._pinned: List[torch.Tensor] = []
        self._turn = 0

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

    @staticmethod
    def params(requests: Sequence, ahead: int = 0):
        """The rows' options as arrays: float32 ``[3, rows]`` (temperature, 0 for greedy rows; top_p; the uniform
        number of this draw) and int32 ``[rows]`` (top_k); None if a row needs a repetition penalty, which works on
        the logits with the tokens generated so far and is not part of these."""
        rows = len(requests)
        par = np.zeros((3, rows), dtype=np.float32)
        par[1, :] = 1.0
        top_k = np.zeros(rows, dtype=np.int32)
        for i, r in enumerate(requests):
            c = r.config
            if c.use_argmax:
                continue
            if c.repetition_penalty != 1.0:
                return None
            par[0, i], par[1, i] = c.temperature, c.top_p
            par[2, i] = uniform_for(r.sample_seed, len(r.output_ids) + ahead)
            top_k[i] = c.top_k
        return par, top_k

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
            par = np.zeros((4, rows), dtype=np.float32)      # temperature, top_p, uniform, top_k (as int bits)
            top_k = np.zeros(rows, dtype=np.int32)
            for i, r in enumerate(requests):
                c = r.config
                if c.use_argmax:
                    par[0, i], par[1, i] = 0.0, 1.0
                    continue
                par[0, i], par[1, i] = c.temperature, c.top_p
                par[2, i] = uniform_for(r.sample_seed, len(r.output_ids) + ahead)
                top_k[i] = c.top_k
                if c.repetition_penalty != 1.0 and r.output_ids:
                    if ahead:
                        raise ValueError("a repetition penalty needs the tokens of the step before on the host")
                    recent = torch.tensor(r.output_ids, dtype=torch.int32).to(self.device, non_blocking=True)
                    ops.repetition_penalty(logits[i], recent, c.repetition_penalty)
            fl = torch.from_numpy(par[:3].copy()).to(self.device, non_blocking=True)
            tk = torch.from_numpy(top_k).to(self.device, non_blocking=True)
            ops.sample(logits, out, fl[0], tk, fl[1], fl[2])
        host = self._host_buffer(rows + 1)
        host[:rows].copy_(out, non_blocking=True)
        host[rows:].copy_(ops.status_word(self.device), non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return PendingTokens(out, host, event)
