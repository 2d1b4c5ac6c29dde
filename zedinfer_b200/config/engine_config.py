"""Engine-side options, with the reference's names, defaults and meanings.

``SchedulerConfig`` follows include/zedinfer/scheduler.hpp:42-60 and
``GenerationConfig`` include/zedinfer/generation_types.hpp:20-90 (the text-side
fields of the latter — chat mode, thinking, stop strings — belong to the
tokenizer front-end and are not here).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class SchedulerConfig:
    max_batch_tokens: int = 2048        # tokens one step may hold (decode + prefill portions)
    max_batch_requests: int = 64        # requests that may be live at once
    max_prefill_tokens: int = 2048      # prompt tokens one step may hold, shared by its prefills (the reference: 512;
    #                                     on this GPU a step below about 1,000 tokens is bound by the host's launches)
    max_queue_size: int = 256           # waiting requests; submit() raises "Queue full" above it
    gpu_memory_utilization: float = 0.9  # share of device memory the engine may use in total
    kv_block_size: int = 16             # tokens per page
    # Additions of this engine (the reference has none of them):
    num_kv_pages: Optional[int] = None  # explicit page count per cache group; None = from the budget
    max_seq_len: Optional[int] = None   # context limit; None = max_position_embeddings
    on_exhaust: str = "preempt"         # pages run out during decode: "preempt" the youngest, or "fail"
    generation_reserve: int = 0         # tokens beyond the prompt reserved at admission (reference: min(max_new, 256))
    cuda_graphs: bool = True            # capture decode-only steps
    run_ahead: bool = True              # launch the next decode step before the host has read this one's tokens

    def validate(self) -> None:
        if self.max_batch_tokens <= 0 or self.max_batch_requests <= 0 or self.max_prefill_tokens <= 0:
            raise ValueError("max_batch_tokens, max_batch_requests and max_prefill_tokens must be positive")
        if self.max_queue_size <= 0:
            raise ValueError("max_queue_size must be positive")
        if not 0.0 < self.gpu_memory_utilization <= 1.0:
            raise ValueError("gpu_memory_utilization must be in (0, 1]")
        if self.kv_block_size <= 0:
            raise ValueError("kv_block_size must be positive")
        if self.on_exhaust not in ("preempt", "fail"):
            raise ValueError("on_exhaust must be 'preempt' or 'fail'")
        if self.num_kv_pages is not None and self.num_kv_pages <= 0:
            raise ValueError("num_kv_pages must be positive")
        if self.generation_reserve < 0:
            raise ValueError("generation_reserve must not be negative")


@dataclass
class GenerationConfig:
    max_new_tokens: int = 0            # 0 = until the context is full
    use_argmax: bool = True            # greedy; the reference's engine default when do_sample is unset
    temperature: float = 1.0
    top_k: int = 0                     # 0 = off
    top_p: float = 1.0                 # 1 = off
    repetition_penalty: float = 1.0    # on generated tokens only
    seed: int = 0                      # 0 = a fresh seed per request
    ignore_eos: bool = False           # addition: run to max_new_tokens (benchmarks with random weights)

    def validate(self) -> None:
        # src/zedinfer/generation_types.cpp:13-25 and src/frontend/sampler/sampler.cpp:24-38
        if self.max_new_tokens < 0:
            raise ValueError("max_new_tokens must be non-negative (0 means unlimited)")
        if not self.use_argmax:
            if not self.temperature > 0.0:
                raise ValueError("temperature must be positive")
            if self.top_k < 0:
                raise ValueError("top_k must be non-negative")
            if not 0.0 < self.top_p <= 1.0:
                raise ValueError("top_p must be in (0, 1]")
            if not self.repetition_penalty > 0.0:
                raise ValueError("repetition_penalty must be positive")


def resolve_max_new_tokens(requested: int, used_context_tokens: int, max_seq_len: int) -> int:
    """0 or too large → what is left of the context (src/zedinfer/generation_types.cpp:39-61)."""
    if requested < 0:
        raise ValueError("max_new_tokens must be non-negative (0 means unlimited)")
    if used_context_tokens < 0:
        raise ValueError("used_context_tokens must be non-negative")
    if max_seq_len <= 0:
        raise ValueError("max_seq_len must be positive")
    remaining = max_seq_len - used_context_tokens
    if remaining <= 0:
        raise ValueError(f"prompt leaves no room for generation: context={used_context_tokens} tokens "
                         f"(max {max_seq_len})")
    if requested == 0 or requested > remaining:
        return remaining
    return requested
