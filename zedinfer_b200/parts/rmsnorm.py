"""RMSNorm: ``y = (w * x) * rstd``, ``rstd = 1 / sqrt(mean(x^2) + eps)``, in float32
(src/backend/ops/rms_norm/cpu/rms_norm_cpu.cpp:24-28).  No ``+1`` on the weight."""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import Norm, ResidualStream, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    capture_safe = True

    def __init__(self, size: int, eps: float):
        if size <= 0:
            raise ValueError(f"rmsnorm: size={size} must be positive")
        if not eps > 0.0:
            raise ValueError(f"rmsnorm: eps={eps} must be positive")
        self.size, self.eps = int(size), float(eps)
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.size,), init=("one_plus_normal", 0.01))}

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].contiguous()

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> None:
        ops.rmsnorm(x, self.weight, self.eps, out)

    def forward_residual(self, stream: ResidualStream, out: torch.Tensor,
                         row_idx: Optional[torch.Tensor] = None) -> None:
        ops.add_rmsnorm(stream.h, stream.delta, self.weight, self.eps, out, row_idx=row_idx,
                        write_residual=row_idx is None)
        if row_idx is None:
            stream.delta = None
