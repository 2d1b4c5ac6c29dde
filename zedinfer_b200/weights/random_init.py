"""Random-weights mode: write a model folder (config.json, model.safetensors) from a
configuration and a seed.

Every tensor is drawn on its own from a generator seeded with (seed, tensor name), so the
values do not depend on the order of tensors or on which other tensors exist.  The rule
of each tensor comes from the part that declares it: projections, biases and embeddings
N(0, 0.02), norm weights 1 + N(0, 0.01).  Values are drawn in float32 and rounded once to
the stored dtype.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Dict, Mapping

import torch

from .loader import TensorSpec
from .safetensors_io import save_file

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & ((1 << 63) - 1)


def random_tensors(specs: Mapping[str, TensorSpec], seed: int, dtype: torch.dtype,
                   init_scale: float = 1.0) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    for name in sorted(specs):
        spec = specs[name]
        if spec.optional:
            continue
        gen = torch.Generator(device="cpu")
        gen.manual_seed(_tensor_seed(seed, name))
        if spec.kind == "int":
            out[name] = torch.zeros(spec.shape, dtype=torch.int32)
            continue
        rule, std = spec.init
        if rule == "normal":
            std = std * init_scale
        t = torch.randn(spec.shape, generator=gen, dtype=torch.float32) * std
        if rule == "one_plus_normal":
            t += 1.0
        elif rule != "normal":
            raise ValueError(f"tensor {name}: unknown init rule {rule!r}")
        out[name] = t.to(dtype)
    return out


def write_random_model(config: Mapping[str, Any], seed: int, out_dir: str, dtype: str = "bfloat16",
                       name_prefix: str = "model.", init_scale: float = 1.0) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a config.json dict) into ``out_dir``.

    ``init_scale`` multiplies the standard deviation of the N(0, 0.02) tensors; tiny test models
    use it so that attention scores and logits are far from uniform."""
    from ..config.registry import resolve_architecture
    from ..engine.model import Model

    if dtype not in _DTYPES:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}, got {dtype!r}")
    raw = dict(config)
    raw["torch_dtype"] = dtype
    arch = resolve_architecture(raw)
    spec = arch.build_spec(arch.parse(raw))
    spec.validate()
    model = Model(spec)
    tensors = random_tensors(model.tensor_specs(), seed, _DTYPES[dtype], init_scale)
    # Names as checkpoints of this family carry them: everything but the head sits under "model."
    stored = {(n if n == spec.head_name else name_prefix + n): t for n, t in tensors.items()}
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(raw, f, indent=2)
    save_file(stored, os.path.join(out_dir, "model.safetensors"),
              metadata={"format": "pt", "seed": str(seed)})
    return out_dir
