"""Random-weights mode: one counter-based rule for every place that draws weights.

A value depends on (seed, tensor name, element index) and on nothing else: not on the device,
the order of tensors, which other tensors exist, or how a tensor is cut into pieces while it
is drawn.  The engine draws on the GPU without a folder (``EngineCore(config=..,
random_seed=..)``), ``write_random_model`` draws on the CPU and writes config.json and
model.safetensors, and a third party can restate the rule in a few lines (the plain
implementation under ``tests/`` does) and get the same bits:

    key      = mix(fnv1a64(name) ^ mix(seed))                       64-bit integers, wrapping
    word_j   = mix(key + (3 * index + j) * 0x9E3779B97F4A7C15)      j = 0, 1, 2
    s        = sum of the twelve 16-bit fields of the three words
    x        = (2 * s - 12 * 65535) / 2^17                          exact in float32
    value    = x * std          ("normal")         or   1 + x * std   ("one_plus_normal")

``mix`` is the splitmix64 finaliser.  ``x`` is the sum of twelve uniform numbers, centred
(Irwin-Hall): mean 0, variance 1, bell-shaped to within what random test weights need, and made
of integer arithmetic alone, so that no library's logarithm or cosine can differ between
machines.  The products and the sum that follow are single float32 operations; the stored
dtype is one more rounding.  The rule of each tensor comes from the part that declares it:
projections, biases and embeddings N(0, 0.02), norm weights 1 + N(0, 0.01)
(the reference has no random weights; it only draws token ids, src/zedinfer/profiler.cpp:79-84).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Mapping

import torch

from .loader import TensorSpec
from .safetensors_io import save_file

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}

_M64 = (1 << 64) - 1
_GOLDEN = 0x9E3779B97F4A7C15
_C1 = 0xBF58476D1CE4E5B9
_C2 = 0x94D049BB133111EB
_CHUNK = {"cpu": 1 << 18, "cuda": 1 << 24}    # elements drawn at a time: cache-sized on the host, bounded temporaries on the device


def _signed(v: int) -> int:
    """The int64 with the same bits as the unsigned 64-bit ``v``."""
    v &= _M64
    return v - (1 << 64) if v >> 63 else v


def _mix_int(z: int) -> int:
    z &= _M64
    z = ((z ^ (z >> 30)) * _C1) & _M64
    z = ((z ^ (z >> 27)) * _C2) & _M64
    return z ^ (z >> 31)


def tensor_key(seed: int, name: str) -> int:
    h = 0xCBF29CE484222325
    for byte in name.encode("utf-8"):
        h = ((h ^ byte) * 0x100000001B3) & _M64
    return _mix_int(h ^ _mix_int(seed))


def _lsr(z: torch.Tensor, s: int) -> torch.Tensor:
    """Logical shift right of int64 bit patterns (torch shifts arithmetically)."""
    return (z >> s) & ((1 << (64 - s)) - 1)


def _mix(z: torch.Tensor) -> torch.Tensor:
    z = (z ^ _lsr(z, 30)) * _signed(_C1)
    z = (z ^ _lsr(z, 27)) * _signed(_C2)
    return z ^ _lsr(z, 31)


def _fields16_sum(z: torch.Tensor) -> torch.Tensor:
    m = 0x0000FFFF0000FFFF
    t = (z & m) + (_lsr(z, 16) & m)
    return (t & 0xFFFFFFFF) + _lsr(t, 32)


def unit_normal(seed: int, name: str, numel: int, device, first: int = 0) -> torch.Tensor:
    """Elements ``first .. first + numel`` of the unit-variance stream of (seed, name), float32."""
    key = tensor_key(seed, name)
    out = torch.empty(numel, dtype=torch.float32, device=device)
    chunk = _CHUNK.get(torch.device(device).type, 1 << 20)
    for lo in range(0, numel, chunk):
        n = min(chunk, numel - lo)
        idx = torch.arange(first + lo, first + lo + n, dtype=torch.int64, device=device) * 3
        s = None
        for j in range(3):
            w = _mix((idx + j) * _signed(_GOLDEN) + _signed(key))
            f = _fields16_sum(w)
            s = f if s is None else s + f
        out[lo: lo + n] = (2 * s - 12 * 65535).to(torch.float32) * (1.0 / 131072.0)
    return out


def draw_tensor(seed: int, name: str, spec: TensorSpec, dtype: torch.dtype, device,
                init_scale: float = 1.0) -> torch.Tensor:
    """The tensor ``name`` of a model drawn with ``seed``, by its spec's rule, in ``dtype`` on ``device``."""
    if spec.kind == "int":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    rule, std = spec.init
    numel = 1
    for d in spec.shape:
        numel *= int(d)
    x = unit_normal(seed, name, numel, device)
    if rule == "normal":
        x *= float(torch.tensor(std * init_scale, dtype=torch.float32))       # the factor is a float32 number
    elif rule == "one_plus_normal":
        x *= float(torch.tensor(std, dtype=torch.float32))
        x += 1.0
    else:
        raise ValueError(f"tensor {name}: unknown init rule {rule!r}")
    return x.view(tuple(spec.shape)).to(dtype)


def random_tensors(specs: Mapping[str, TensorSpec], seed: int, dtype: torch.dtype,
                   init_scale: float = 1.0, device="cpu") -> Dict[str, torch.Tensor]:
    """Every non-optional tensor of ``specs``, drawn on ``device``.  ``init_scale`` multiplies the standard
    deviation of the N(0, std) tensors (tiny test models use it so that scores and logits are far from uniform)."""
    return {name: draw_tensor(seed, name, specs[name], dtype, device, init_scale)
            for name in sorted(specs) if not specs[name].optional}


def write_random_model(config: Mapping[str, Any], seed: int, out_dir: str, dtype: str = "bfloat16",
                       name_prefix: str = "model.", init_scale: float = 1.0) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a config.json dict) into ``out_dir``.
    The values are those that ``EngineCore(None, config=config, random_seed=seed)`` draws on the device."""
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
