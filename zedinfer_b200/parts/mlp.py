"""Gated feed-forward: ``down(up(x) * act(gate(x)))`` with SiLU, no biases unless asked
(src/frontend/models/transformer_forward.cpp:128-137, src/backend/ops/swiglu/cpu/swiglu_cpu.cpp:13-20).
Gate and up weights are stacked at load so one product makes both."""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import FeedForward, StepContext, register_feed_forward


def _stack(tensors):
    """Concatenate along dim 0; if storage dtypes differ, float32 wins."""
    dtype = torch.float32 if any(t.dtype == torch.float32 for t in tensors) else tensors[0].dtype
    return torch.cat([t.to(dtype) for t in tensors], dim=0).contiguous()


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    capture_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "silu", bias: bool = False):
        if activation != "silu":
            raise ValueError(f"gated_mlp: activation {activation!r} is not supported (only 'silu')")
        if hidden_size <= 0 or intermediate_size <= 0:
            raise ValueError("gated_mlp: sizes must be positive")
        self.hidden_size, self.intermediate_size, self.bias = int(hidden_size), int(intermediate_size), bool(bias)
        self.w_gate_up: Optional[torch.Tensor] = None
        self.b_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None
        self.b_down: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        h, i = self.hidden_size, self.intermediate_size
        specs = {"gate_proj.weight": TensorSpec((i, h)), "up_proj.weight": TensorSpec((i, h)),
                 "down_proj.weight": TensorSpec((h, i))}
        if self.bias:
            specs.update({"gate_proj.bias": TensorSpec((i,)), "up_proj.bias": TensorSpec((i,)),
                          "down_proj.bias": TensorSpec((h,))})
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.w_gate_up = _stack([tensors["gate_proj.weight"], tensors["up_proj.weight"]])
        self.w_down = tensors["down_proj.weight"].contiguous()
        if self.bias:
            self.b_gate_up = _stack([tensors["gate_proj.bias"], tensors["up_proj.bias"]])
            self.b_down = tensors["down_proj.bias"].contiguous()

    def _activation(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        act = ctx.empty(x.shape[0], self.intermediate_size)
        ops.linear_silu_mul(x, self.w_gate_up, self.b_gate_up, act)     # activation in the product's epilogue where it can be
        return act

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        out = ctx.empty(x.shape[0], self.hidden_size)
        ops.linear(self._activation(x, ctx), self.w_down, self.b_down, out)
        return out

    def forward_for_residual(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        return ops.linear_for_residual(self._activation(x, ctx), self.w_down, self.b_down)   # the product, or partial sums over K
