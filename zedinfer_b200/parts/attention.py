"""Causal self-attention with grouped key/value heads over the paged cache.

Per token (src/frontend/models/transformer_forward.cpp:71-112, and
src/backend/ops/self_attention/cpu/paged_attention_cpu.cpp:113-159 for the scores):

    q, k, v = x Wq^T + bq, x Wk^T + bk, x Wv^T + bv       (one stacked product)
    q, k rotated by position; k, v appended to the request's cache pages
    s_j = (q . k_j) * scale for the keys j the query may see; softmax in float32; out = sum p_j v_j
    y = out Wo^T (+ bo)

A query at position P sees keys ``max(0, P - window + 1) .. P`` (all keys from 0 without a
window).  Query head ``h`` reads key/value head ``h // (num_heads // num_kv_heads)``.
"""
from __future__ import annotations

import math
from typing import Dict, Mapping, Optional

import torch

from .. import ops
from ..cache.manager import CallCacheView, PagedKVNeed
from ..config.spec import PartSpec
from ..weights.loader import TensorSpec
from .base import Mixer, StepContext, build_part, register_mixer
from .mlp import _stack


@register_mixer("attention")
class AttentionMixer(Mixer):
    @property
    def capture_safe(self) -> bool:        # as safe as the position rule it was built with
        return bool(getattr(self.position, "capture_safe", False))

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position: PartSpec, qkv_bias: bool = True, out_bias: bool = False,
                 scale: Optional[float] = None, window: Optional[int] = None):
        if num_heads <= 0 or num_kv_heads <= 0 or num_heads % num_kv_heads:
            raise ValueError(f"attention: {num_heads} query heads cannot share {num_kv_heads} key/value heads")
        if head_dim <= 0 or head_dim % 16:
            raise ValueError(f"attention: head_dim={head_dim} is not supported; the kernels take head sizes "
                             f"in steps of 16 (16, 32, ..., 256)")
        if head_dim > 256:
            raise ValueError(f"attention: head_dim={head_dim} is not supported; the kernels take at most 256")
        if window is not None and window <= 0:
            raise ValueError(f"attention: window={window} must be positive (or None for all keys)")
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.head_dim, self.window = int(head_dim), (int(window) if window is not None else None)
        self.qkv_bias, self.out_bias = bool(qkv_bias), bool(out_bias)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(float(head_dim))
        self.position = build_part("position", position)
        self.q_dim, self.kv_dim = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = None

    def cache_need(self):
        return PagedKVNeed(self.num_kv_heads, self.head_dim, self.window)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        h = self.hidden_size
        specs = {"q_proj.weight": TensorSpec((self.q_dim, h)), "k_proj.weight": TensorSpec((self.kv_dim, h)),
                 "v_proj.weight": TensorSpec((self.kv_dim, h)), "o_proj.weight": TensorSpec((h, self.q_dim))}
        if self.qkv_bias:
            specs.update({"q_proj.bias": TensorSpec((self.q_dim,)), "k_proj.bias": TensorSpec((self.kv_dim,)),
                          "v_proj.bias": TensorSpec((self.kv_dim,))})
        if self.out_bias:
            specs["o_proj.bias"] = TensorSpec((h,))
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.w_qkv = _stack([tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]])
        if self.qkv_bias:
            self.b_qkv = _stack([tensors["q_proj.bias"], tensors["k_proj.bias"], tensors["v_proj.bias"]])
            if self.b_qkv.dtype != self.w_qkv.dtype:
                # one product, one operand type: float32 wins
                self.w_qkv, self.b_qkv = self.w_qkv.float(), self.b_qkv.float()
        self.w_o = tensors["o_proj.weight"].contiguous()
        if self.out_bias:
            self.b_o = tensors["o_proj.bias"].contiguous()

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CallCacheView, owns_cache: bool) -> torch.Tensor:
        out = ctx.empty(x.shape[0], self.hidden_size)
        ops.linear(self._attend(x, ctx, cache, owns_cache), self.w_o, self.b_o, out)
        return out

    def forward_for_residual(self, x: torch.Tensor, ctx: StepContext, cache: CallCacheView,
                             owns_cache: bool) -> torch.Tensor:
        return ops.linear_for_residual(self._attend(x, ctx, cache, owns_cache), self.w_o, self.b_o)

    def _attend(self, x: torch.Tensor, ctx: StepContext, cache: CallCacheView, owns_cache: bool) -> torch.Tensor:
        """Everything up to the output projection: ``[tokens, heads * head_dim]``."""
        if cache.kind != "paged":
            raise RuntimeError("attention needs a paged key/value cache")
        n = x.shape[0]
        q = ctx.empty(n, self.num_heads, self.head_dim)
        if not self.position.project_rotate_append(x, self.w_qkv, self.b_qkv, q, cache, ctx, self.num_heads,
                                                   self.num_kv_heads, self.head_dim, write_kv=owns_cache):
            qkv = ctx.empty(n, self.q_dim + 2 * self.kv_dim)
            ops.linear(x, self.w_qkv, self.b_qkv, qkv)
            self.position.rotate_append(qkv, q, cache, ctx, self.num_heads, self.num_kv_heads, self.head_dim,
                                        write_kv=owns_cache)
        attn = ctx.empty(n, self.q_dim)
        ops.attention(q, cache, attn, ctx, self.num_heads, self.num_kv_heads, self.head_dim, self.window, self.scale)
        return attn
