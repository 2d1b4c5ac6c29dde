"""Write a model folder (config.json, model.safetensors) with random weights from a configuration and a seed."""
from __future__ import annotations

import argparse
import json
import sys


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="zedinfer-random-model", description=__doc__)
    p.add_argument("config", help="a config.json of a supported architecture")
    p.add_argument("out", help="folder to write")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--dtype", choices=["bfloat16", "float32", "float16"], default="bfloat16")
    p.add_argument("--init-scale", type=float, default=1.0, help="multiplies the 0.02 standard deviation")
    args = p.parse_args(argv)
    from ..weights import write_random_model
    with open(args.config) as f:
        raw = json.load(f)
    write_random_model(raw, args.seed, args.out, dtype=args.dtype, init_scale=args.init_scale)
    print(args.out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
