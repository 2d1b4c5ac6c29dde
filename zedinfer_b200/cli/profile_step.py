"""Run a few decode, prefill or mixed steps of a random-weight Qwen2-shaped model between cudaProfilerStart/Stop,
for ``ncu --profile-from-start off``.  Steps are launched kernel by kernel (no CUDA graph), so every
kernel shows up as a launch of its own.  Prints the mean time of a step measured with CUDA events."""
from __future__ import annotations

import argparse
import json
import sys


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="zedinfer-profile-step", description=__doc__)
    p.add_argument("--mode", choices=["decode", "prefill", "mixed", "sample"], default="decode",
                   help="mixed: --batch decoding requests beside a prompt portion of --tokens; sample: the sampling "
                        "kernel alone on --batch rows of --vocab logits with a few likely tokens and a long tail")
    p.add_argument("--temperature", type=float, default=0.7, help="sample: the rows' temperature")
    p.add_argument("--top-k", type=int, default=20, help="sample: the rows' top-k (0: none)")
    p.add_argument("--top-p", type=float, default=0.8, help="sample: the rows' top-p (1: none)")
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--context", type=int, default=3072, help="decode: tokens already cached per request")
    p.add_argument("--tokens", type=int, default=2048, help="prefill: tokens of the portion")
    p.add_argument("--layers", type=int, default=28)
    p.add_argument("--steps", type=int, default=2)
    p.add_argument("--hidden", type=int, default=1536)
    p.add_argument("--heads", type=int, default=12)
    p.add_argument("--kv-heads", type=int, default=2)
    p.add_argument("--head-dim", type=int, default=128)
    p.add_argument("--intermediate", type=int, default=8960)
    p.add_argument("--vocab", type=int, default=151936)
    p.add_argument("--graphs", action="store_true", help="decode through the captured step instead")
    p.add_argument("--tcgen05-plain-products", action="store_true",
                   help="plain products of 1,024 rows or more on the tcgen05 kernel instead of the library")
    args = p.parse_args(argv)
    import torch
    from .. import ops
    from ..engine.core import EngineCore, StepEntry
    if args.mode == "sample":
        return profile_sampling(args)
    ops.TC_PLAIN_PRODUCTS = bool(args.tcgen05_plain_products)
    cfg = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": args.layers,
           "hidden_size": args.hidden, "num_attention_heads": args.heads, "num_key_value_heads": args.kv_heads,
           "head_dim": args.head_dim, "intermediate_size": args.intermediate, "vocab_size": args.vocab,
           "max_position_embeddings": 8192}
    span = args.tokens if args.mode == "prefill" else max(args.context + args.steps + 8, args.tokens)
    core = EngineCore(None, "bfloat16", config=cfg, random_seed=3, page_size=16,
                      max_tokens=(args.batch + 1) * (span + 64), max_requests=args.batch + 1, max_seq_len=span + 64,
                      cuda_graphs=args.graphs)
    g = torch.Generator().manual_seed(0)
    rand = lambda n: torch.randint(0, args.vocab, (n,), generator=g).tolist()      # noqa: E731
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    counter = [0]
    if args.mode in ("decode", "mixed"):
        for r in range(args.batch):
            left = args.context
            while left > 0:
                n = min(left, 2048)
                core.step([StepEntry(r, rand(n), [])])
                left -= n
    if args.mode == "decode":
        step = lambda: core.step([StepEntry(r, rand(1), [0]) for r in range(args.batch)])   # noqa: E731
    elif args.mode == "mixed":
        def step():
            rid = ("p", counter[0])
            counter[0] += 1
            core.step([StepEntry(r, rand(1), [0]) for r in range(args.batch)] + [StepEntry(rid, rand(args.tokens), [])])
            core.end(rid)
    else:
        def step():
            rid = ("p", counter[0])
            counter[0] += 1
            core.step([StepEntry(rid, rand(args.tokens), [args.tokens - 1])])
            core.end(rid)
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    a.record()
    for _ in range(args.steps):
        step()
    b.record()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    print(json.dumps({"mode": args.mode, "batch": args.batch, "layers": args.layers,
                      "ms_per_step": round(a.elapsed_time(b) / args.steps, 4)}))
    return 0


def profile_sampling(args) -> int:
    """The sampling kernel alone: probability ~ rank^-1.5 with the ranks dealt at random over the vocabulary, the
    largest logit 20."""
    import torch
    from .. import ops
    dev = torch.device("cuda:0")
    rows, vocab = args.batch, args.vocab
    g = torch.Generator().manual_seed(0)
    rank = torch.stack([torch.randperm(vocab, generator=g) for _ in range(rows)]).float() + 1.0
    logits = (20.0 - 1.5 * torch.log(rank)).to(dev)
    out = torch.empty(rows, dtype=torch.int32, device=dev)
    temp = torch.full((rows,), args.temperature, device=dev)
    top_k = torch.full((rows,), args.top_k, dtype=torch.int32, device=dev)
    top_p = torch.full((rows,), args.top_p, device=dev)
    uni = torch.rand(rows, generator=g).to(dev)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(3):
        ops.sample(logits, out, temp, top_k, top_p, uni)
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    a.record()
    for _ in range(args.steps):
        ops.sample(logits, out, temp, top_k, top_p, uni)
    b.record()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    print(json.dumps({"mode": "sample", "rows": rows, "vocab": vocab, "temperature": args.temperature, "top_k": args.top_k,
                      "top_p": args.top_p, "us_per_call": round(a.elapsed_time(b) * 1000.0 / args.steps, 2)}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
