"""A generation request and its result (include/zedinfer/request.hpp:47-243, generation_types.hpp:97-126)."""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass
from typing import Callable, List, Optional

from ..config.engine_config import GenerationConfig


class RequestPhase(enum.Enum):
    WAITING = "waiting"
    PREFILL = "prefill"
    DECODE = "decode"
    COMPLETE = "complete"


@dataclass
class GenerationStats:
    prompt_tokens: int = 0
    generated_tokens: int = 0
    queue_time_ms: float = 0.0
    prefill_time_ms: float = 0.0        # until the first generated token
    decode_time_ms: float = 0.0
    total_time_ms: float = 0.0
    preemptions: int = 0

    def prefill_tokens_per_second(self) -> float:
        return self.prompt_tokens * 1000.0 / self.prefill_time_ms if self.prefill_time_ms > 0 else 0.0

    def decode_tokens_per_second(self) -> float:
        return self.generated_tokens * 1000.0 / self.decode_time_ms if self.decode_time_ms > 0 else 0.0


@dataclass
class GenerationResult:
    request_id: int
    output_ids: List[int]
    finish_reason: str                  # "stop", "length", "error" or "cancelled"
    error: Optional[str]
    stats: GenerationStats


class InferenceRequest:
    _next_id = 0

    def __init__(self, input_ids: List[int], config: Optional[GenerationConfig] = None,
                 stream_callback: Optional[Callable[[int], None]] = None, request_id: Optional[int] = None):
        if request_id is None:
            request_id = InferenceRequest._next_id
            InferenceRequest._next_id += 1
        self.request_id = request_id
        self.input_ids: List[int] = list(input_ids)
        self.config = config or GenerationConfig()
        self.stream_callback = stream_callback
        self.output_ids: List[int] = []
        self.phase = RequestPhase.WAITING
        self.prefill_progress = 0            # tokens of `sequence()` that are in the cache
        # the sampler's record of the request's table of generated tokens on the device: which cache slot it was
        # (the slot's serial) and how many tokens have been added to it
        self.count_serial, self.counted = -1, 0
        self.finish_reason: Optional[str] = None
        self.error: Optional[str] = None
        self.cancelled = False
        self.cache = None                    # RequestCache while the request holds pages
        self.sample_seed = 0
        self.max_new_tokens = 0              # resolved at submit
        self.stats = GenerationStats(prompt_tokens=len(self.input_ids))
        self.arrival_time = time.perf_counter()
        self.first_scheduled_time: Optional[float] = None
        self.first_token_time: Optional[float] = None
        self.admission_warned = False

    def sequence(self) -> List[int]:
        """Everything that has to be in the cache before the next token: prompt, then what was generated."""
        return self.input_ids + self.output_ids

    @property
    def generated_count(self) -> int:
        return len(self.output_ids)

    def result(self) -> GenerationResult:
        return GenerationResult(self.request_id, list(self.output_ids), self.finish_reason or "error", self.error,
                                self.stats)
