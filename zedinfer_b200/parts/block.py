"""Pre-norm residual arrangement (src/frontend/models/transformer_forward.cpp:63-149):

    h = h + mixer(norm1(h));  h = h + ffn(norm2(h))

The adds are fused into the norm that follows them: a branch output stays "pending" in the
stream until the next norm folds it into the float32 residual."""
from __future__ import annotations

import torch

from .. import ops
from ..cache.manager import CallCacheView
from .base import Block, ResidualStream, StepContext, register_block


@register_block("pre_norm")
class PreNormBlock(Block):
    def _fusable(self, stream: ResidualStream, ctx: StepContext) -> bool:
        """A step of few tokens in bfloat16 runs each half of the block as two fused kernels (norm folded into the
        product that reads it, residual add into the product that writes it) when every part offers that."""
        if ctx.dtype != torch.bfloat16 or ctx.n_tokens > ops.FUSED_DECODE_ROWS:
            return False
        if stream.delta is not None or stream.ssq is None:
            return False
        n1, n2 = self.norms["norm1"], self.norms["norm2"]
        return (getattr(self.mixer, "fused_ok", lambda: False)() and getattr(self.ffn, "fused_ok", lambda: False)()
                and getattr(n1, "fused_ok", lambda: False)() and getattr(n2, "fused_ok", lambda: False)())

    def forward(self, stream: ResidualStream, ctx: StepContext, cache: CallCacheView, owns_cache: bool) -> None:
        if self._fusable(stream, ctx):
            self.mixer.forward_fused(stream, self.norms["norm1"], ctx, cache, owns_cache)
            self.ffn.forward_fused(stream, self.norms["norm2"], ctx)
            return
        stream.ssq = None                     # the kernels below change h without keeping its sums of squares
        n, hidden = stream.h.shape
        normed = ctx.empty(n, hidden)
        self.norms["norm1"].forward_residual(stream, normed)
        stream.delta = self.mixer.forward(normed, ctx, cache, owns_cache)
        normed2 = ctx.empty(n, hidden)
        self.norms["norm2"].forward_residual(stream, normed2)
        stream.delta = self.ffn.forward(normed2, ctx)
