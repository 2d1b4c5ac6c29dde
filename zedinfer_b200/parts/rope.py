"""Rotate-half rotary position encoding over the whole head.

``inv_freq[k] = 1 / theta^(2k / head_dim)`` in float32, ``angle = float(position) * inv_freq[k]``,
``y[k] = a*cos - b*sin``, ``y[k + half] = b*cos + a*sin`` with ``a = x[k]``, ``b = x[k + half]``
(src/backend/ops/rope/cpu/rope_cpu.cpp:32-52 and :60-65).  Values are not rotated.  The kernel
that rotates also appends k and v to the cache pages of each token's request.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..cache.manager import CallCacheView
from .base import PositionEncoding, StepContext, register_position


@register_position("rope")
class RotaryPosition(PositionEncoding):
    capture_safe = True

    def __init__(self, head_dim: int, theta: float):
        if head_dim <= 0 or head_dim % 2:
            raise ValueError(f"rope: head_dim={head_dim} must be positive and even")
        if not theta > 0.0:
            raise ValueError(f"rope: theta={theta} must be positive")
        self.head_dim, self.theta = int(head_dim), float(theta)
        self._inv_freq: Optional[torch.Tensor] = None

    def inverse_frequencies(self) -> torch.Tensor:
        """float32 table on the CPU: 1 / powf(theta, float(2k) / float(head_dim))."""
        expo = torch.arange(0, self.head_dim, 2, dtype=torch.float32) / torch.tensor(float(self.head_dim),
                                                                                     dtype=torch.float32)
        return 1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float32), expo)

    def _table(self, device: torch.device) -> torch.Tensor:
        if self._inv_freq is None or self._inv_freq.device != device:
            self._inv_freq = self.inverse_frequencies().to(device)
        return self._inv_freq

    def rotate_append(self, qkv: torch.Tensor, q_out: torch.Tensor, cache: CallCacheView, ctx: StepContext,
                      n_heads: int, n_kv_heads: int, head_dim: int, write_kv: bool) -> None:
        if head_dim != self.head_dim:
            raise ValueError(f"rope was built for head_dim={self.head_dim}, the mixer has {head_dim}")
        # few tokens (a decode step beyond what the product's epilogue takes): the step's angles, made once
        cs = self._step_angles(ctx, qkv.device) if qkv.shape[0] <= ops.ROPE_TABLE_MAX_TOKENS else None
        ops.rope_append(qkv, q_out, cache.tensor, ctx.tables[cache.group], ctx.tok_seg, ctx.positions,
                        self._table(qkv.device), n_heads, n_kv_heads, head_dim, cache.page_size, cache.page_stride,
                        cache.kv_stride, write_kv=write_kv, cs=cs)

    def _step_angles(self, ctx: StepContext, device: torch.device) -> torch.Tensor:
        """cos | sin of every token's angles, float32 ``[tokens, head_dim]``: made by the first layer of a step that
        asks, shared by every layer with the same theta and head size."""
        key = ("rope_cs", self.theta, self.head_dim)
        cs = ctx.step_cache.get(key)
        if cs is None:
            cs = torch.empty((ctx.positions.numel(), self.head_dim), dtype=torch.float32, device=device)
            ops.rope_table(ctx.positions, self._table(device), cs)
            ctx.step_cache[key] = cs
        return cs

    def project_rotate_append(self, x: torch.Tensor, w_qkv: torch.Tensor, b_qkv: Optional[torch.Tensor],
                              q_out: torch.Tensor, cache: CallCacheView, ctx: StepContext, n_heads: int,
                              n_kv_heads: int, head_dim: int, write_kv: bool) -> bool:
        """Steps of at most 16 tokens in bfloat16 (decode): rotation and append run in the epilogue of the q/k/v
        product.  The step's cosines and sines are made once and shared by every layer with the same theta and
        head size."""
        if not (write_kv and head_dim == self.head_dim
                and ops.can_fuse_rope_product(x, w_qkv, b_qkv, cache.tensor)):
            return False
        cs = self._step_angles(ctx, x.device)
        ops.gemm_smallm_rope(x, w_qkv, b_qkv, cs, q_out, cache.tensor, ctx.tables[cache.group], ctx.tok_seg,
                             ctx.positions, n_heads, n_kv_heads, head_dim, cache.page_size, cache.page_stride,
                             cache.kv_stride)
        return True
