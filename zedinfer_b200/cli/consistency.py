"""Do the logits of a request depend on how its tokens were cut into steps, on what else was in the batch, or on
which pages it got?  Runs a few requests of random token ids through ``EngineCore.step`` in four ways and compares
every logit with the first:

  whole     each request alone, its whole prompt in one step (the reference of the comparison)
  tail      all but the last 32 tokens in one step, the last 32 one by one
  portions  in portions of changing size, down to two tokens
  mixed     up to four requests live at a time, portions of some beside single tokens of others, in a pool so small
            that the pages of finished requests are used again

float32 is expected to agree to the last bit; bfloat16 to rounding, and its distance from float32 is reported too.
One JSON line per mode.  In the manner of nothing in the reference, which has no such program.
"""
from __future__ import annotations

import argparse
import json
import random
import sys


def _portions(n: int, rng: random.Random):
    sizes, left = [], n
    menu = [5, 2, 11, 3, 2, 64, 7, 130, 2, 33, 16, 17, 1]
    while left > 0:
        k = min(left, rng.choice(menu))
        if left - k == 1:                   # never leave a single token for last: portions go down to two
            k = left
        sizes.append(k)
        left -= k
    return sizes


def _run_alone(core, StepEntry, ids, sizes, tag):
    """One request in steps of the given sizes; returns its logits at every position, float32 on the device."""
    import torch
    rows, t = [], 0
    for k in sizes:
        rows.append(core.step([StepEntry(tag, ids[t:t + k], list(range(k)))]).float().clone())
        t += k
    core.end(tag)
    return torch.cat(rows, 0)


def _run_mixed(core, StepEntry, requests, rng):
    """All requests, at most four live; each live request moves by a portion or, once its prompt part is in, by
    single tokens; a finished request's pages go back and are taken by the next one."""
    import torch
    waiting = list(requests.items())
    live, got = {}, {rid: [] for rid in requests}
    while waiting or live:
        while waiting and len(live) < 4:
            rid, ids = waiting.pop(0)
            live[rid] = [ids, 0, max(2, len(ids) - rng.randrange(8, 40))]      # ids, done, where single tokens start
        entries, meta = [], []
        for rid, (ids, done, single_from) in live.items():
            if rng.random() < 0.2 and len(live) > 1:
                continue                                                        # a request may sit a step out
            if done >= single_from:
                k = 1
            else:
                k = min(single_from - done, rng.choice([2, 3, 9, 40, 128]))
            entries.append(StepEntry(rid, ids[done:done + k], list(range(k))))
            meta.append((rid, k))
        if not entries:
            continue
        entries.sort(key=lambda e: len(e.tokens) != 1)                          # single tokens first, as the engine does
        meta.sort(key=lambda m: m[1] != 1)
        logits = core.step(entries).float()
        row = 0
        for rid, k in meta:
            got[rid].append(logits[row:row + k].clone())
            row += k
            live[rid][1] += k
        for rid in [r for r, (ids, done, _) in live.items() if done >= len(ids)]:
            core.end(rid)
            del live[rid]
    return {rid: torch.cat(parts, 0) for rid, parts in got.items()}


def _compare(ref, got):
    import torch
    worst, unequal, total = 0.0, 0, 0
    for rid in ref:
        d = (ref[rid] - got[rid]).abs()
        worst = max(worst, float(d.max()))
        unequal += int((ref[rid] != got[rid]).sum())
        total += ref[rid].numel()
    return {"worst_abs_diff": worst, "values_not_bit_equal": unequal, "values": total}


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="zedinfer-consistency", description=__doc__.split("\n\n")[0])
    p.add_argument("model_path", help="Model folder, or a config.json alone with --random-weights")
    p.add_argument("--random-weights", type=int, default=None, metavar="SEED")
    p.add_argument("--dtype", choices=["float32", "bfloat16", "both"], default="both")
    p.add_argument("--tokens", type=int, default=300, help="Length of the longest request")
    p.add_argument("--requests", type=int, default=6)
    p.add_argument("--kv-block-size", type=int, default=16)
    p.add_argument("--layers", type=int, default=None, help="Fewer layers than the configuration has (same sizes)")
    p.add_argument("--seed", type=int, default=0)
    args = p.parse_args(argv)
    import torch
    from ..config.registry import read_config_json
    from ..engine.core import EngineCore, StepEntry
    if args.tokens < 48:
        print("--tokens must be at least 48", file=sys.stderr)
        return 1
    raw = read_config_json(args.model_path)
    if args.layers is not None:
        raw = dict(raw, num_hidden_layers=args.layers)
    rng = random.Random(args.seed)
    vocab = raw["vocab_size"]
    lengths = [args.tokens] + [rng.randrange(40, args.tokens + 1) for _ in range(args.requests - 1)]
    requests = {f"r{i}": [rng.randrange(vocab) for _ in range(n)] for i, n in enumerate(lengths)}
    page = args.kv_block_size
    need = sorted((-(-n // page) for n in lengths), reverse=True)
    pages = sum(need[:4]) + 2                                   # room for the four longest at once, hardly more
    results, whole32 = [], None
    for dtype in (["float32", "bfloat16"] if args.dtype == "both" else [args.dtype]):
        kw = dict(page_size=page, num_pages=pages, max_requests=4, max_seq_len=args.tokens + 8)
        if args.random_weights is None and args.layers is None:
            core = EngineCore(args.model_path, dtype, **kw)
        elif args.random_weights is None:
            print("--layers needs --random-weights (a folder's tensors belong to its own layer count)", file=sys.stderr)
            return 1
        else:
            core = EngineCore(None, dtype, config=raw, random_seed=args.random_weights, **kw)
        whole = {rid: _run_alone(core, StepEntry, ids, [len(ids)], rid) for rid, ids in requests.items()}
        runs = {
            "tail": {rid: _run_alone(core, StepEntry, ids, [len(ids) - 32] + [1] * 32, rid) for rid, ids in requests.items()},
            "portions": {rid: _run_alone(core, StepEntry, ids, _portions(len(ids), random.Random(args.seed + 1)), rid)
                         for rid, ids in requests.items()},
            "mixed": _run_mixed(core, StepEntry, requests, random.Random(args.seed + 2)),
        }
        core.check_kernels()
        core.cache.check()
        for mode, got in runs.items():
            line = dict(dtype=dtype, mode=mode, against="whole", **_compare(whole, got))
            results.append(line)
            print(json.dumps(line), flush=True)
        if dtype == "float32":
            whole32 = whole
        elif whole32 is not None:
            scale = max(float(v.abs().max()) for v in whole32.values())
            line = dict(dtype=dtype, mode="whole", against="float32 whole", largest_logit=scale, **_compare(whole32, whole))
            results.append(line)
            print(json.dumps(line), flush=True)
        del core, whole, runs
        torch.cuda.empty_cache()
    bad = [r for r in results if r["dtype"] == "float32" and r["values_not_bit_equal"]]
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
