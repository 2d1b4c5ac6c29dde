"""Prefill / decode timing of one request of random token ids, in the manner of the reference's
``bench`` (examples/bench.cpp, src/zedinfer/profiler.cpp:119-162)."""
from __future__ import annotations

import argparse
import sys

from .common import add_engine_arguments, create_engine


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="zedinfer-bench", description=__doc__.split("\n")[0])
    add_engine_arguments(p)
    p.add_argument("-p", "--prefill-len", type=int, default=128, help="Sequence length for prefill phase")
    p.add_argument("-d", "--decode-len", "--max-tokens", dest="decode_len", type=int, default=128,
                   help="Number of tokens to decode")
    p.add_argument("-r", "--rounds", type=int, default=3, help="Number of benchmark rounds")
    args = p.parse_args(argv)
    if args.decode_len <= 0:
        print("--decode-len/--max-tokens must be > 0 for benchmark runs", file=sys.stderr)
        return 1
    engine = create_engine(args)
    for _ in range(2):                                                     # warm-up with the same lengths, twice:
        engine.profile(args.prefill_len, args.decode_len)                  # a recurring step is captured at its second run
    total_p = total_d = 0.0
    for i in range(args.rounds):
        pm, dm = engine.profile(args.prefill_len, args.decode_len)
        total_p, total_d = total_p + pm, total_d + dm
        print(f"Round {i + 1}: prefill={pm:.2f}ms, decode={dm:.2f}ms", file=sys.stderr)
    avg_p, avg_d = total_p / args.rounds, total_d / args.rounds
    steps = max(args.decode_len - 1, 1)                                     # decode_len - 1 steps ran
    print("\n================ Performance Report ================")
    print(f"Config : prefill={args.prefill_len}, decode={args.decode_len}, rounds={args.rounds}")
    print(f"Prefill: {avg_p:8.2f} ms | {args.prefill_len / avg_p * 1000.0:8.2f} tok/s")
    print(f"Decode : {avg_d:8.2f} ms | {steps / avg_d * 1000.0 if avg_d > 0 else 0.0:8.2f} tok/s")
    print("====================================================")
    return 0


if __name__ == "__main__":
    sys.exit(main())
