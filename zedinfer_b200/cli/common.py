"""Options shared by the command-line programs; names and defaults follow the reference's
examples (examples/ping.cpp:31-79, examples/bench.cpp:23-60, examples/serve.cpp:44-46)."""
from __future__ import annotations

import argparse
import logging
import os
import sys

from ..config.engine_config import SchedulerConfig


def add_engine_arguments(p: argparse.ArgumentParser) -> None:
    p.add_argument("model_path", help="Path to the model directory (config.json + *.safetensors)")
    p.add_argument("--random-weights", type=int, default=None, metavar="SEED",
                   help="model_path may be a config.json alone: draw the weights on the device from this seed "
                        "instead of reading *.safetensors (shapes too large to write out as a folder)")
    p.add_argument("--nvidia", action="store_true",
                   help="Use NVIDIA GPU backend (accepted for parity; this engine has no other backend)")
    p.add_argument("--gpu-memory-utilization", type=float, default=0.9,
                   help="Fraction of GPU memory the engine may use (0.0-1.0)")
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16",
                   help="bfloat16: serving kernels; float32: the true 32-bit path")
    p.add_argument("--max-batch-tokens", type=int, default=2048)
    p.add_argument("--max-batch-requests", type=int, default=64)
    p.add_argument("--max-prefill-tokens", type=int, default=2048,
                   help="Prompt tokens one step may hold (the reference defaults to 512; steps of fewer than about "
                        "1,000 tokens are bound by the host here)")
    p.add_argument("--kv-block-size", type=int, default=int(os.environ.get("ZEDINFER_KV_BLOCK_SIZE", "16")),
                   help="Tokens per cache page (the reference reads ZEDINFER_KV_BLOCK_SIZE)")
    p.add_argument("--kv-pages", type=int, default=None, help="Pages per cache group instead of a memory budget")
    p.add_argument("--max-seq-len", type=int, default=None, help="Context limit (default: max_position_embeddings)")
    p.add_argument("--on-exhaust", choices=["preempt", "fail"], default="preempt",
                   help="When pages run out during decode: preempt the youngest request, or fail it as the reference does")
    p.add_argument("--no-cuda-graphs", action="store_true", help="Launch decode steps kernel by kernel")
    add_logging_arguments(p)


_LEVELS = {"none": logging.CRITICAL + 10, "fatal": logging.CRITICAL, "error": logging.ERROR, "warning": logging.WARNING,
           "info": logging.INFO, "debug": logging.DEBUG, "verbose": logging.DEBUG - 5}
log = logging.getLogger("zedinfer_b200")


def add_logging_arguments(p: argparse.ArgumentParser, default_log_file: str = "", default_level: str = "info") -> None:
    """The reference's logging options (include/utils/logging_cli.hpp:11-38); an empty --log-file writes no file."""
    p.add_argument("--log-level", choices=sorted(_LEVELS, key=_LEVELS.get), default=default_level,
                   help="Log level: none, fatal, error, warning, info, debug, verbose")
    p.add_argument("--log-file", default=default_log_file, help="Path to the log file")
    p.add_argument("--log-to-console", dest="log_to_console", action="store_true", default=True,
                   help="Mirror logs to stderr (default)")
    p.add_argument("--no-log-to-console", dest="log_to_console", action="store_false",
                   help="Disable stderr log mirroring")
    p.add_argument("--log-append", action="store_true", help="Append to --log-file instead of replacing it")
    p.add_argument("--log-overwrite", action="store_true", help="Replace --log-file on startup (default)")


def setup_logging(args) -> logging.Logger:
    log.handlers.clear()
    log.propagate = False
    log.setLevel(_LEVELS[getattr(args, "log_level", "info")])
    fmt = logging.Formatter("%(message)s")
    if getattr(args, "log_to_console", True):
        h = logging.StreamHandler(sys.stderr)
        h.setFormatter(fmt)
        log.addHandler(h)
    path = getattr(args, "log_file", "")
    if path:
        h = logging.FileHandler(path, mode="a" if getattr(args, "log_append", False) and not getattr(args, "log_overwrite", False) else "w")
        h.setFormatter(logging.Formatter("%(asctime)s %(levelname)s %(message)s"))
        log.addHandler(h)
    if not log.handlers:
        log.addHandler(logging.NullHandler())
    return log


def scheduler_config_from(args) -> SchedulerConfig:
    return SchedulerConfig(max_batch_tokens=args.max_batch_tokens, max_batch_requests=args.max_batch_requests,
                           max_prefill_tokens=args.max_prefill_tokens,
                           gpu_memory_utilization=args.gpu_memory_utilization, kv_block_size=args.kv_block_size,
                           num_kv_pages=args.kv_pages, max_seq_len=args.max_seq_len, on_exhaust=args.on_exhaust,
                           cuda_graphs=not args.no_cuda_graphs)


def create_engine(args):
    from ..engine import InferenceEngine
    setup_logging(args)
    engine = InferenceEngine.create(args.model_path, scheduler_config_from(args), dtype=args.dtype,
                                    random_seed=args.random_weights)
    st = engine.cache_stats()
    log.info(f"[engine] cache: pages of {st['page_size']} tokens, per group of layers {st['pages_per_group']} "
             f"({st['pool_tokens']} tokens, {st['pool_bytes'] / 2**30:.2f} GiB)")
    d = engine.default_generation
    log.info("[engine] default sampling: " + ("greedy" if d.use_argmax else
             f"temperature={d.temperature} top_k={d.top_k} top_p={d.top_p} repetition_penalty={d.repetition_penalty}"))
    return engine


def parse_ids(text: str):
    return [int(t) for t in text.replace(",", " ").split()]
