"""N requests of random token ids through submit_async + run_loop, in the manner of the reference's
``batch_bench`` (examples/batch_bench.cpp:100-183): ids uniform in [100, 30000], seed 12345."""
from __future__ import annotations

import argparse
import random
import sys
import time

from .common import add_engine_arguments, scheduler_config_from


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="zedinfer-batch-bench", description=__doc__.split("\n")[0])
    add_engine_arguments(p)
    p.add_argument("-b", "--batch-size", type=int, default=4, help="Number of concurrent requests")
    p.add_argument("-p", "--prefill-len", type=int, default=128, help="Prompt length per request (tokens)")
    p.add_argument("-d", "--decode-len", "--max-tokens", dest="decode_len", type=int, default=128,
                   help="Max tokens to generate per request")
    p.add_argument("-r", "--rounds", type=int, default=1, help="Number of benchmark rounds")
    args = p.parse_args(argv)
    from .. import GenerationConfig
    from ..engine import InferenceEngine, InferenceRequest
    engine = InferenceEngine.create(args.model_path, scheduler_config_from(args), dtype=args.dtype)
    vocab = engine.core.spec.vocab_size
    lo, hi = (100, min(30000, vocab - 1)) if vocab > 200 else (0, vocab - 1)
    rng = random.Random(12345)
    gc = GenerationConfig(max_new_tokens=args.decode_len, ignore_eos=True)
    # warm-up: the same workload twice, untimed (kernels are compiled and loaded at the first step, recurring steps
    # are captured in CUDA graphs at their second appearance)
    for _ in range(2):
        engine.generate_batch([[rng.randint(lo, hi) for _ in range(args.prefill_len)] for _ in range(args.batch_size)], gc)
    print("\n============ Batch Benchmark ============")
    print(f"Config: batch_size={args.batch_size}, prefill={args.prefill_len}, decode={args.decode_len}, rounds={args.rounds}")
    total_ms, total_tokens = 0.0, 0
    for r in range(args.rounds):
        import torch
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        futs = [engine.submit_async(InferenceRequest([rng.randint(lo, hi) for _ in range(args.prefill_len)], gc))
                for _ in range(args.batch_size)]
        engine.run_loop()
        ms = (time.perf_counter() - t0) * 1000.0
        tokens = sum(len(f.result().output_ids) for f in futs)
        total_ms, total_tokens = total_ms + ms, total_tokens + tokens
        print(f"Round {r + 1}: {args.batch_size} requests, {tokens} tokens generated, {ms:.2f} ms")
    avg_ms, avg_tokens = total_ms / args.rounds, total_tokens / args.rounds
    print("\n============ Batch Performance Report ============")
    print(f"Batch size     : {args.batch_size} requests")
    print(f"Avg total time : {avg_ms:8.2f} ms")
    print(f"Avg tokens/batch: {avg_tokens:8.0f}")
    print(f"Throughput     : {avg_tokens / avg_ms * 1000.0:8.2f} tok/s  (total, all requests)")
    print(f"Per-request    : {avg_ms / args.batch_size:8.2f} ms  (avg wall time per request)")
    print("===================================================")
    return 0


if __name__ == "__main__":
    sys.exit(main())
