"""N requests of random token ids through submit_async + run_loop, in the manner of the reference's
``batch_bench`` (examples/batch_bench.cpp:100-183): ids uniform in [100, 30000], seed 12345.

Beyond the reference's options, ``--prefill-len-max`` draws each prompt's length uniformly from
[--prefill-len, --prefill-len-max] (continuous batching of unequal requests), and the report adds the share of
prompt tokens, the time to the first token, the steps taken and how often a request was taken off the GPU when
pages ran out, and the context (prompt + generated tokens) that the requests reached."""
from __future__ import annotations

import argparse
import random
import sys
import time

from .common import add_engine_arguments, create_engine


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="zedinfer-batch-bench", description=__doc__.split("\n")[0])
    add_engine_arguments(p)
    p.add_argument("-b", "--batch-size", type=int, default=4, help="Number of concurrent requests")
    p.add_argument("-p", "--prefill-len", type=int, default=128, help="Prompt length per request (tokens)")
    p.add_argument("--prefill-len-max", type=int, default=None,
                   help="Draw each prompt's length uniformly from [--prefill-len, this]")
    p.add_argument("-d", "--decode-len", "--max-tokens", dest="decode_len", type=int, default=128,
                   help="Max tokens to generate per request")
    p.add_argument("-r", "--rounds", type=int, default=1, help="Number of benchmark rounds")
    p.add_argument("--warmup-rounds", type=int, default=2,
                   help="Untimed rounds of the same workload before the timed ones (kernels are compiled and loaded at "
                        "the first step; a recurring step is captured in a CUDA graph at its second appearance)")
    args = p.parse_args(argv)
    hi_len = args.prefill_len if args.prefill_len_max is None else args.prefill_len_max
    if args.prefill_len <= 0 or hi_len < args.prefill_len:
        print("--prefill-len must be positive and --prefill-len-max not below it", file=sys.stderr)
        return 1
    import torch
    from .. import GenerationConfig
    from ..engine import InferenceRequest
    engine = create_engine(args)
    vocab = engine.core.spec.vocab_size
    lo, hi = (100, min(30000, vocab - 1)) if vocab > 200 else (0, vocab - 1)
    rng = random.Random(12345)
    gc = GenerationConfig(max_new_tokens=args.decode_len, ignore_eos=True)

    def prompts():
        return [[rng.randint(lo, hi) for _ in range(rng.randint(args.prefill_len, hi_len))]
                for _ in range(args.batch_size)]

    for _ in range(max(0, args.warmup_rounds)):
        engine.generate_batch(prompts(), gc)
    print("\n============ Batch Benchmark ============")
    lens = f"{args.prefill_len}" if hi_len == args.prefill_len else f"{args.prefill_len}..{hi_len}"
    print(f"Config: batch_size={args.batch_size}, prefill={lens}, decode={args.decode_len}, rounds={args.rounds}")
    total_ms, total_tokens, total_prompt, total_steps, total_pre = 0.0, 0, 0, 0, 0
    ttft, failed, reached = [], 0, []
    for r in range(args.rounds):
        work = prompts()
        steps0, pre0 = engine.steps_run, engine.scheduler.num_preemptions
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        futs = [engine.submit_async(InferenceRequest(ids, gc)) for ids in work]
        engine.run_loop()
        ms = (time.perf_counter() - t0) * 1000.0
        results = [f.result() for f in futs]
        tokens = sum(len(x.output_ids) for x in results)
        failed += sum(1 for x in results if x.error)
        reached += [len(ids) + len(x.output_ids) for ids, x in zip(work, results)]
        ttft += [x.stats.queue_time_ms + x.stats.prefill_time_ms for x in results if not x.error]
        total_ms, total_tokens = total_ms + ms, total_tokens + tokens
        total_prompt += sum(len(ids) for ids in work)
        total_steps += engine.steps_run - steps0
        total_pre += engine.scheduler.num_preemptions - pre0
        print(f"Round {r + 1}: {args.batch_size} requests, {tokens} tokens generated, {ms:.2f} ms")
    n = max(1, args.rounds)
    avg_ms, avg_tokens = total_ms / n, total_tokens / n
    print("\n============ Batch Performance Report ============")
    print(f"Batch size     : {args.batch_size} requests")
    print(f"Avg total time : {avg_ms:8.2f} ms")
    print(f"Avg tokens/batch: {avg_tokens:8.0f}")
    print(f"Throughput     : {avg_tokens / avg_ms * 1000.0:8.2f} tok/s  (total, all requests)")
    print(f"Per-request    : {avg_ms / args.batch_size:8.2f} ms  (avg wall time per request)")
    print(f"Prompt tokens  : {total_prompt / n:8.0f} per batch | {(total_prompt + total_tokens) / total_ms * 1000.0:8.2f} tok/s "
          "(prompt + generated)")
    if ttft:
        ttft.sort()
        print(f"First token    : {sum(ttft) / len(ttft):8.2f} ms mean | {ttft[len(ttft) // 2]:8.2f} ms median | "
              f"{ttft[-1]:8.2f} ms max  (from submission)")
    print(f"Steps          : {total_steps / n:8.0f} per batch | {avg_ms / max(1.0, total_steps / n):8.3f} ms per step")
    reached.sort()
    print(f"Context reached: {reached[0]:8d} min | {reached[len(reached) // 2]:8d} median | {reached[-1]:8d} max  "
          "(prompt + generated tokens per request)")
    st = engine.cache_stats()
    print(f"Cache pool     : {st['pool_tokens']:8d} tokens ({st['pool_bytes'] / 2**30:.1f} GiB)")
    print(f"Preemptions    : {total_pre:8d} | failed requests: {failed}")
    print("===================================================")
    return 0


if __name__ == "__main__":
    sys.exit(main())
