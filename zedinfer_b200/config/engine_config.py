"""Engine-side options, with the reference's names, defaults and meanings.

``SchedulerConfig`` follows include/zedinfer/scheduler.hpp:42-60 and
``GenerationConfig`` include/zedinfer/generation_types.hpp:20-90 (the text-side
fields of the latter — chat mode, thinking, stop strings — belong to the
tokenizer front-end and are not here).
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Mapping, Optional


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
    """Per-request options (include/zedinfer/generation_types.hpp:20-90).  As in the reference, the sampling fields
    count only with ``has_sampling_override``; a request without it is sampled by the engine's default, which comes
    from the model folder's generation_config.json (:func:`sampling_defaults`; greedy when there is none).  Giving
    any sampling field another value than its default sets the flag; say ``has_sampling_override=True`` to insist on
    greedy against a folder that asks for sampling."""
    max_new_tokens: int = 0            # 0 = until the context is full
    use_argmax: bool = True            # greedy
    temperature: float = 1.0
    top_k: int = 0                     # 0 = off
    top_p: float = 1.0                 # 1 = off
    repetition_penalty: float = 1.0    # on generated tokens only
    seed: int = 0                      # 0 = a fresh seed per request
    ignore_eos: bool = False           # addition: run to max_new_tokens (benchmarks with random weights)
    has_sampling_override: bool = False

    def __post_init__(self) -> None:
        if (not self.use_argmax or self.temperature != 1.0 or self.top_k != 0 or self.top_p != 1.0
                or self.repetition_penalty != 1.0 or self.seed != 0):
            self.has_sampling_override = True

    def with_sampling_of(self, default: "GenerationConfig") -> "GenerationConfig":
        """This request's options with the engine's default sampling, unless the request brought its own."""
        if self.has_sampling_override:
            return self
        return replace(self, use_argmax=default.use_argmax, temperature=default.temperature, top_k=default.top_k,
                       top_p=default.top_p, repetition_penalty=default.repetition_penalty, seed=default.seed,
                       has_sampling_override=True)

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


def sampling_defaults(model_dir: Optional[str], environ: Optional[Mapping[str, str]] = None) -> GenerationConfig:
    """The engine's default sampling, as the reference derives it (src/zedinfer/engine.cpp:49-126):

    * ``ZEDINFER_FORCE_ARGMAX`` set to anything but "" or "0": greedy, whatever the folder says;
    * no generation_config.json in the folder, ``do_sample`` false or absent, a file that does not parse, or values
      that do not validate: greedy;
    * else ``temperature`` / ``top_k`` / ``top_p`` / ``repetition_penalty`` (1.0 if absent) / ``seed`` (0 if
      absent) from the file, with ``ZEDINFER_REPETITION_PENALTY`` overriding the penalty.
    """
    import json
    import os
    env = os.environ if environ is None else environ
    greedy = GenerationConfig(use_argmax=True, has_sampling_override=True)
    force = env.get("ZEDINFER_FORCE_ARGMAX", "")
    if force not in ("", "0"):
        return greedy
    path = os.path.join(model_dir, "generation_config.json") if model_dir and os.path.isdir(model_dir) else None
    if path is None or not os.path.isfile(path):
        return greedy
    try:
        with open(path, "r", encoding="utf-8") as f:
            j = json.load(f)
        if not isinstance(j, dict) or not j.get("do_sample", False):
            return greedy
        cfg = GenerationConfig(use_argmax=False, temperature=float(j.get("temperature", 1.0)), top_k=int(j.get("top_k", 0)),
                               top_p=float(j.get("top_p", 1.0)), repetition_penalty=float(j.get("repetition_penalty", 1.0)),
                               seed=int(j.get("seed", 0)), has_sampling_override=True)
        rp = env.get("ZEDINFER_REPETITION_PENALTY", "")
        if rp != "":
            try:
                cfg.repetition_penalty = float(rp)
            except ValueError:
                pass                            # the reference keeps the file's value when the variable does not parse
        cfg.validate()
        return cfg
    except (OSError, ValueError, TypeError):
        return greedy
