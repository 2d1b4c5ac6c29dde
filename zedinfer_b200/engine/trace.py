"""Trace replay: feed given token ids through a model step by step and write logits.

It samples nothing and has no forward pass, cache or loader of its own: every step goes
through :meth:`EngineCore.step`, the function generation uses.

Input, one JSON object per line on standard input::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, ``<out>/<step>.f32`` receives the logits at the
wanted places, in the order of the entries and of ``want``, as little-endian float32
``[wanted, vocab]``.  After every step the line ``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List, Optional

PAGE_SIZE = 16
MAX_LIVE = 8


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", required=True, choices=["bfloat16", "float32"],
                   help="bfloat16: the kernels and precisions that serving uses; float32: everything in true 32-bit")
    p.add_argument("--out", required=True, help="folder for <step>.f32 files")
    p.add_argument("--max-tokens", type=int, required=True,
                   help="the most tokens live requests hold at any time (each rounded up to a multiple of 64); "
                        "the cache pool is made for this many")
    return p


def main(argv: Optional[List[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    if args.max_tokens <= 0:
        print("trace_run: --max-tokens must be positive", file=sys.stderr)
        return 2
    os.makedirs(args.out, exist_ok=True)

    import torch  # noqa: F401

    from ..csrc import build
    from .core import EngineCore, StepEntry

    print("[trace_run] preparing kernels (compiled at the first call) ...", file=sys.stderr, flush=True)
    build.compile_all(EngineCore.kernel_libraries(args.dtype))
    print(f"[trace_run] loading {args.model} as {args.dtype} ...", file=sys.stderr, flush=True)
    core = EngineCore(args.model, args.dtype, page_size=PAGE_SIZE, max_tokens=args.max_tokens,
                      max_requests=MAX_LIVE, max_seq_len=args.max_tokens)
    print("[trace_run] ready", file=sys.stderr, flush=True)

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        obj = json.loads(line)
        step = obj["step"]
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", [])) for e in obj.get("entries", [])]
        logits = core.step(entries) if entries else None
        if logits is not None:
            arr = logits.to("cpu").numpy().astype("<f4", copy=False)
            core.check_kernels()
            tmp = os.path.join(args.out, f".{step}.f32.tmp")
            arr.tofile(tmp)
            os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
        else:
            core.check_kernels()
            torch.cuda.synchronize()
        for rid in obj.get("end", []):
            core.end(rid)
        sys.stdout.write(f"done {step}\n")
        sys.stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
