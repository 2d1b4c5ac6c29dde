"""A model put together from a :class:`ModelSpec`: embedding, blocks in schedule order, final
norm, output head.  It knows no architecture: which parts a layer has, their sizes and the
order of the calls all come from the spec."""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional, Tuple

import torch

from ..cache.manager import CallCacheView
from ..config.spec import ModelSpec
from ..config.spec import PartSpec
from ..parts.base import Block, ResidualStream, StepContext, block_class, build_part
from ..weights.loader import TensorSpec


class Model:
    def __init__(self, spec: ModelSpec):
        spec.validate()
        self.spec = spec
        self.blocks: List[Block] = []
        for layer in spec.layers:
            cls = block_class(layer.block)
            self.blocks.append(cls({role: build_part(family, ps) for role, family, ps in layer.part_specs()}))
        # the caches of each call, by the role of the mixer they belong to: the key of the usual mixer's cache is
        # the index of the call that owns it, the key of any other mixer's cache is (that index, role)
        self._call_caches: List[Dict[str, object]] = []
        for pos, call in enumerate(spec.schedule):
            owner = pos if call.cache_of is None else call.cache_of
            self._call_caches.append({role: (owner if role == "mixer" else (owner, role))
                                      for role in self.blocks[call.layer].mixers()})
        self.embedding = build_part("embedding", spec.embedding or PartSpec("token_embedding", {
            "vocab_size": spec.vocab_size, "hidden_size": spec.hidden_size, "name": spec.embed_name}))
        self.final_norm = build_part("norm", spec.final_norm)
        self.head = build_part("head", spec.head or PartSpec("output_head", {
            "vocab_size": spec.vocab_size, "hidden_size": spec.hidden_size, "tied": spec.tie_word_embeddings,
            "name": spec.head_name}))
        self.dtype: Optional[torch.dtype] = None
        self.device: Optional[torch.device] = None
        self._views_of: Optional[Mapping[object, CallCacheView]] = None
        self._views_by_call: List[Dict[str, CallCacheView]] = []

    # ---- tensors ----------------------------------------------------------------------------
    def _part_prefixes(self):
        """(part, global name prefix) for every part that loads tensors."""
        for i, (layer, blk) in enumerate(zip(self.spec.layers, self.blocks)):
            base = self.spec.layer_prefix.format(i=i)
            for role, part in blk.parts().items():
                yield part, base + layer.prefixes.get(role, role + ".")
        yield self.final_norm, self.spec.final_norm_prefix
        yield self.embedding, ""
        yield self.head, ""

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        out: Dict[str, TensorSpec] = {}
        for part, prefix in self._part_prefixes():
            for local, ts in part.tensor_specs().items():
                out[prefix + local] = ts
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype, device) -> None:
        self.dtype, self.device = dtype, torch.device(device)
        for part, prefix in self._part_prefixes():
            local = {name: tensors[prefix + name] for name in part.tensor_specs() if prefix + name in tensors}
            if part is self.head:
                self.head.bind(local, embedding=self.embedding.tied_weight())
            else:
                part.bind(local)

    def capture_blockers(self) -> List[str]:
        """The parts and arrangements that keep this model's steps from being captured in CUDA graphs (see
        ``Part.capture_safe``), by name; empty when every step may be captured.  One such part switches graphs off
        for every step of the model: each step is then launched kernel by kernel, which costs the host a few
        milliseconds per step whatever the step's size."""
        out = []
        for part, prefix in self._part_prefixes():
            if not getattr(part, "capture_safe", False):
                out.append(f"{prefix or '(model) '}{type(part).__name__}")
        for i, blk in enumerate(self.blocks):
            if not getattr(blk, "capture_safe", False):
                out.append(f"{self.spec.layer_prefix.format(i=i)}{type(blk).__name__}")
        return out

    def capture_safe(self) -> bool:
        """Every part and arrangement of the model only launches kernels on the step's device tensors, so steps may
        be captured in CUDA graphs."""
        return not self.capture_blockers()

    # ---- cache ------------------------------------------------------------------------------
    def cache_needs(self) -> List[Tuple[object, object]]:
        """(cache key, need) for every cache of every call that owns its caches.  The key of a layer's usual mixer is
        the call's index in the schedule; a further mixer of the layer has (index, role)."""
        out = []
        for pos, call in enumerate(self.spec.schedule):
            if call.cache_of is None:
                for role, mixer in self.blocks[call.layer].mixers().items():
                    out.append((self._call_caches[pos][role], mixer.cache_need()))
        return out

    # ---- one step ---------------------------------------------------------------------------
    def forward(self, ctx: StepContext, cache_views: Mapping[object, CallCacheView],
                logit_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Run the step's tokens through every call; return float32 logits of ``logit_rows`` (or None)."""
        ctx.step_cache.clear()                 # what layers share (a step's rotation angles) belongs to one step
        h = torch.empty((ctx.n_tokens, self.spec.hidden_size), dtype=torch.float32, device=ctx.device)
        self.embedding.forward(ctx.token_ids, h)
        stream = ResidualStream(h)
        if self._views_of is not cache_views:          # the same mapping step after step: resolve the keys once
            self._views_by_call = [{role: cache_views[key] for role, key in keys.items()} for keys in self._call_caches]
            self._views_of = cache_views
        for pos, call in enumerate(self.spec.schedule):
            self.blocks[call.layer].forward(stream, ctx, self._views_by_call[pos], owns_cache=call.cache_of is None)
        if logit_rows is None or logit_rows.numel() == 0:
            return None
        rows = logit_rows.numel()
        normed = ctx.empty(rows, self.spec.hidden_size)
        self.final_norm.forward_residual(stream, normed, row_idx=logit_rows)
        logits = torch.empty((rows, self.spec.vocab_size), dtype=torch.float32, device=ctx.device)
        self.head.forward(normed, logits)
        return logits
