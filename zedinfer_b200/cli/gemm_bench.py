"""Time the matrix-product kernels on the shapes of a step (device time, CUDA events, L2 flushed between
repetitions): cuBLAS through torch, the tcgen05 kernel in both orientations and the weight-streaming kernel."""
from __future__ import annotations

import argparse
import json
import sys


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="zedinfer-gemm-bench", description=__doc__)
    p.add_argument("--rows", type=int, nargs="+", default=[8, 64, 2048])
    p.add_argument("--hidden", type=int, default=1536)
    p.add_argument("--intermediate", type=int, default=8960)
    p.add_argument("--qkv", type=int, default=2048)
    p.add_argument("--vocab", type=int, default=151936)
    p.add_argument("--reps", type=int, default=20)
    p.add_argument("--shapes", nargs="+", default=None, help="only these products (qkv o gate_up down lm_head)")
    args = p.parse_args(argv)
    import torch
    from .. import ops
    dev = torch.device("cuda:0")
    shapes = [("qkv", args.qkv, args.hidden), ("o", args.hidden, args.hidden), ("gate_up", 2 * args.intermediate, args.hidden),
              ("down", args.hidden, args.intermediate), ("lm_head", args.vocab, args.hidden)]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn):
        for _ in range(3):
            fn()
        total = 0.0
        for _ in range(args.reps):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            total += a.elapsed_time(b)
        return total / args.reps * 1000.0          # microseconds

    for m in args.rows:
        for name, n, k in shapes:
            if (name == "lm_head" and m > 64) or (args.shapes and name not in args.shapes):
                continue
            x = (torch.randn(m, k, device=dev) * 0.5).to(torch.bfloat16)
            w = (torch.randn(n, k, device=dev) * 0.05).to(torch.bfloat16)
            out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
            row = {"rows": m, "shape": name, "n": n, "k": k, "weight_mb": round(n * k * 2 / 1e6, 1)}
            row["cublas_us"] = round(timed(lambda: torch.mm(x, w.t(), out=out)), 2)
            if m <= 256:
                row["tcgen05_swapped_us"] = round(timed(lambda: ops.gemm_tcgen05(x, w, None, out, swapped=True)), 2)
            if m >= 64:
                row["tcgen05_normal_us"] = round(timed(lambda: ops.gemm_tcgen05(x, w, None, out, swapped=False)), 2)
                row["tcgen05_tiles_us"] = round(timed(lambda: ops.gemm_tcgen05_tiles(x, w, None, out, pairs=False)), 2)
                row["tcgen05_pairs_us"] = round(timed(lambda: ops.gemm_tcgen05_tiles(x, w, None, out, pairs=True)), 2)
                if name == "gate_up":
                    act = torch.empty(m, n // 2, dtype=torch.bfloat16, device=dev)
                    row["cublas_plus_silu_mul_us"] = round(timed(lambda: (torch.mm(x, w.t(), out=out), ops.silu_mul(out, act))), 2)
                    row["tcgen05_tiles_silu_mul_us"] = round(timed(lambda: ops.gemm_tcgen05_tiles(x, w, None, act, silu_mul=True, pairs=False)), 2)
                    row["tcgen05_pairs_silu_mul_us"] = round(timed(lambda: ops.gemm_tcgen05_tiles(x, w, None, act, silu_mul=True, pairs=True)), 2)
            if m <= 16:
                row["smallm_us"] = round(timed(lambda: ops.gemm_smallm(x, w, None, out)), 2)
            best = min(v for kk, v in row.items() if kk.endswith("_us"))
            row["best_gbs"] = round(n * k * 2 / best / 1e3, 1)
            row["best_tflops"] = round(2.0 * m * n * k / best / 1e6, 1)
            print(json.dumps(row), flush=True)
    if ops.tcgen05_status(dev):
        print("a bounded wait ran out in the tcgen05 kernel", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
