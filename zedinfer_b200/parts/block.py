"""Pre-norm residual arrangement (src/frontend/models/transformer_forward.cpp:63-149):

    h = h + mixer(norm1(h));  h = h + ffn(norm2(h))

The adds are fused into the norm that follows them: a branch output stays "pending" in the
stream until the next norm folds it into the float32 residual."""
from __future__ import annotations

from typing import Mapping

from ..cache.manager import CallCacheView
from .base import Block, ResidualStream, StepContext, register_block


@register_block("pre_norm")
class PreNormBlock(Block):
    capture_safe = True

    def __init__(self, parts):
        super().__init__(parts)
        missing = [role for role in ("mixer", "ffn", "norm1", "norm2") if role not in self.parts()]
        if missing:
            raise ValueError(f"the pre_norm arrangement needs the parts {missing} as well")

    def forward(self, stream: ResidualStream, ctx: StepContext, caches: Mapping[str, CallCacheView],
                owns_cache: bool) -> None:
        n, hidden = stream.h.shape
        normed = ctx.empty(n, hidden)
        self.norms["norm1"].forward_residual(stream, normed)
        stream.delta = self.mixer.forward_for_residual(normed, ctx, caches["mixer"], owns_cache)
        normed2 = ctx.empty(n, hidden)
        self.norms["norm2"].forward_residual(stream, normed2)
        stream.delta = self.ffn.forward_for_residual(normed2, ctx)
