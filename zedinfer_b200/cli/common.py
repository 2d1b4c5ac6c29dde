"""Options shared by the command-line programs; names and defaults follow the reference's
examples (examples/ping.cpp:31-79, examples/bench.cpp:23-60, examples/serve.cpp:44-46)."""
from __future__ import annotations

import argparse
import os

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


def scheduler_config_from(args) -> SchedulerConfig:
    return SchedulerConfig(max_batch_tokens=args.max_batch_tokens, max_batch_requests=args.max_batch_requests,
                           max_prefill_tokens=args.max_prefill_tokens,
                           gpu_memory_utilization=args.gpu_memory_utilization, kv_block_size=args.kv_block_size,
                           num_kv_pages=args.kv_pages, max_seq_len=args.max_seq_len, on_exhaust=args.on_exhaust,
                           cuda_graphs=not args.no_cuda_graphs)


def create_engine(args):
    import sys
    from ..engine import InferenceEngine
    engine = InferenceEngine.create(args.model_path, scheduler_config_from(args), dtype=args.dtype,
                                    random_seed=args.random_weights)
    st = engine.cache_stats()
    print(f"[engine] cache: {st['pages_per_group']} pages of {st['page_size']} tokens ({st['pages_per_group'] * st['page_size']} "
          f"tokens, {st['pool_bytes'] / 2**30:.2f} GiB)", file=sys.stderr)
    return engine


def parse_ids(text: str):
    return [int(t) for t in text.replace(",", " ").split()]
