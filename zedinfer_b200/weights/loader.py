"""Bind the tensors of a model folder to the names a model expects.

The model (built from parts) says which tensors it needs, with shapes; this
module reads the folder, checks everything at once and raises a single
:class:`WeightsError` that lists what is missing, what is unexpected and what has
the wrong shape or kind.  The reference only finds a missing tensor at its first
use (include/frontend/models/base.hpp:143-149) and never checks shapes.

Storage rule.  With ``compute_dtype=bfloat16`` floating tensors are kept in
bfloat16, except that a tensor stored in 32-bit (or 64-bit) floating point stays
in float32; with ``compute_dtype=float32`` every floating tensor is widened to
float32, which is exact.  Integer tables become int32.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Mapping, Tuple

import torch

from .safetensors_io import SafetensorsFile, TensorEntry, open_model_files


@dataclass(frozen=True)
class TensorSpec:
    shape: Tuple[int, ...]
    kind: str = "float"          # "float" or "int"
    optional: bool = False
    init: Tuple[str, float] = ("normal", 0.02)   # random-weights mode: ("normal", std) or ("one_plus_normal", std)


class WeightsError(ValueError):
    def __init__(self, model_dir: str, missing: List[str], unexpected: List[str],
                 wrong: List[str], duplicate: List[str]):
        self.missing, self.unexpected, self.wrong, self.duplicate = missing, unexpected, wrong, duplicate
        lines = [f"weights in {model_dir} do not match the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shape or kind ({len(wrong)}): " + "; ".join(wrong))
        if duplicate:
            lines.append(f"  stored more than once ({len(duplicate)}): " + ", ".join(duplicate))
        super().__init__("\n".join(lines))


def canonical_name(raw: str) -> str:
    """Strip a leading ``model.`` and then ``language_model.`` (src/frontend/models/base.cpp:1386-1396)."""
    name = raw
    if len(name) > 6 and name.startswith("model."):
        name = name[6:]
    if len(name) > 15 and name.startswith("language_model."):
        name = name[15:]
    return name


_FLOAT = (torch.float16, torch.bfloat16, torch.float32, torch.float64)
_INT = (torch.int8, torch.uint8, torch.int16, torch.int32, torch.int64)


def storage_dtype(stored: torch.dtype, kind: str, compute_dtype: torch.dtype) -> torch.dtype:
    if kind == "int":
        return torch.int32
    if compute_dtype == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return compute_dtype


def load_weights(model_dir: str, expected: Mapping[str, TensorSpec], compute_dtype: torch.dtype,
                 device: torch.device | str) -> Dict[str, torch.Tensor]:
    files: List[SafetensorsFile] = open_model_files(model_dir)
    found: Dict[str, TensorEntry] = {}
    duplicate: List[str] = []
    for f in files:
        for raw, entry in f.entries.items():
            name = canonical_name(raw)
            if name in found:
                duplicate.append(name)
            found[name] = entry
    missing = sorted(n for n, s in expected.items() if n not in found and not s.optional)
    unexpected = sorted(n for n in found if n not in expected)
    wrong: List[str] = []
    for name, spec in expected.items():
        e = found.get(name)
        if e is None:
            continue
        if tuple(e.shape) != tuple(spec.shape):
            wrong.append(f"{name}: stored {list(e.shape)}, model needs {list(spec.shape)}")
        elif spec.kind == "float" and e.torch_dtype not in _FLOAT:
            wrong.append(f"{name}: stored as {e.dtype}, model needs a floating tensor")
        elif spec.kind == "int" and e.torch_dtype not in _INT:
            wrong.append(f"{name}: stored as {e.dtype}, model needs an integer tensor")
    if missing or unexpected or wrong or duplicate:
        raise WeightsError(model_dir, missing, unexpected, wrong, sorted(set(duplicate)))
    out: Dict[str, torch.Tensor] = {}
    for name, spec in expected.items():
        e = found.get(name)
        if e is None:
            continue
        host = e.load()
        target = storage_dtype(host.dtype, spec.kind, compute_dtype)
        if spec.kind == "int" and host.dtype == torch.int64 and host.numel():
            lo, hi = int(host.min()), int(host.max())
            if lo < -2**31 or hi >= 2**31:
                raise WeightsError(model_dir, [], [], [f"{name}: values [{lo}, {hi}] do not fit int32"], [])
        out[name] = host.to(device=device, dtype=target, copy=True).contiguous()
    for f in files:
        f.close()
    return out
