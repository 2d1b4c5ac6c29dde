"""One prompt through the engine, in the manner of the reference's ``ping`` (examples/ping.cpp).
The prompt is token ids: tokenizer and chat template are not part of this engine."""
from __future__ import annotations

import argparse
import sys
import time

from .common import add_engine_arguments, create_engine, log, parse_ids


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="zedinfer-ping", description=__doc__.split("\n")[0])
    add_engine_arguments(p)
    p.add_argument("--prompt", "--prompt-ids", dest="prompt", default="1 2 3 4 5 6 7 8",
                   help="Prompt as token ids, separated by spaces or commas")
    p.add_argument("--max-new-tokens", "--max-tokens", dest="max_new_tokens", type=int, default=0,
                   help="Maximum number of new tokens to generate (0 = unlimited)")
    p.add_argument("--stream", action="store_true", help="Print token ids as they are generated")
    p.add_argument("--temperature", type=float, default=None,
                   help="0 = greedy; not given (and no other sampling option): the engine's default, which follows the "
                        "folder's generation_config.json as in the reference (greedy without one)")
    p.add_argument("--top-k", type=int, default=0)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--repetition-penalty", type=float, default=1.0)
    p.add_argument("--seed", type=int, default=0, help="0 = a fresh seed")
    p.add_argument("--ignore-eos", action="store_true")
    args = p.parse_args(argv)
    if args.max_new_tokens < 0:
        print("--max-new-tokens/--max-tokens must be >= 0", file=sys.stderr)
        return 1
    from .. import GenerationConfig
    t0 = time.perf_counter()
    try:
        engine = create_engine(args)
    except Exception as e:
        print(f"[ping] engine init failed: {e}", file=sys.stderr)
        return 3
    log.info(f"[ping] engine initialized in {(time.perf_counter() - t0) * 1000:.0f} ms")
    own = (args.temperature is not None or args.top_k != 0 or args.top_p != 1.0 or args.repetition_penalty != 1.0
           or args.seed != 0)
    if not own:
        gc = GenerationConfig(max_new_tokens=args.max_new_tokens, ignore_eos=args.ignore_eos)
    else:
        # sampling options without a temperature sample at temperature 1; --temperature 0 is greedy
        greedy = args.temperature is not None and args.temperature <= 0.0
        gc = GenerationConfig(max_new_tokens=args.max_new_tokens, use_argmax=greedy,
                              temperature=args.temperature if args.temperature and not greedy else 1.0, top_k=args.top_k,
                              top_p=args.top_p, repetition_penalty=args.repetition_penalty, seed=args.seed,
                              ignore_eos=args.ignore_eos, has_sampling_override=True)
    cb = (lambda tok: print(tok, end=" ", flush=True)) if args.stream else None
    try:
        result = engine.generate_tokens(parse_ids(args.prompt), gc, stream_callback=cb)
    except Exception as e:
        print(f"[ping] generation failed: {e}", file=sys.stderr)
        return 2
    if args.stream:
        print()
    else:
        print(" ".join(str(t) for t in result.output_ids))
    s = result.stats
    log.info(f"[ping] finish={result.finish_reason} prompt={s.prompt_tokens} generated={s.generated_tokens} "
             f"prefill={s.prefill_time_ms:.2f} ms ({s.prefill_tokens_per_second():.1f} tok/s) "
             f"decode={s.decode_time_ms:.2f} ms ({s.decode_tokens_per_second():.1f} tok/s)")
    if result.error:
        print(f"[ping] error: {result.error}", file=sys.stderr)
        return 2
    return 0


if __name__ == "__main__":
    sys.exit(main())
