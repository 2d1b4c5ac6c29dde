"""Interfaces of the parts a layer is put together from, and the registries that name them.

A part knows its own sizes and constants (constructor keywords) and nothing about the model
it sits in.  The kinds are:

* **Norm** — ``forward(x, out)`` and ``forward_residual(stream, out, ...)``, which first folds
  the pending branch output into the float32 residual.
* **PositionEncoding** — owns the constants of a position rule and applies it to the freshly
  projected q and k of a step, appending k and v to the cache on the way.
* **Mixer** — mixes information between tokens.  It says what cache it needs per request
  (pages of keys and values, a fixed-size state, or nothing) and runs on the tokens of one
  step: ``forward(x, ctx, cache, owns_cache) -> y``.
* **FeedForward** — works on each token alone: ``forward(x, ctx) -> y``.
* **Block** — the arrangement of the above around the residual stream.
* **Embedding** and **Head** — the two ends of the model: token ids to the residual stream, and the normed
  hidden states of the wanted rows to logits.

Every part declares the tensors it loads (``tensor_specs``: local name → shape and init
rule) and receives them in ``bind``.  New kinds are added with the ``register_*`` functions
from anywhere, a test file included; nothing in the framework's own files has to change.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Mapping, Optional, Sequence

import torch

from ..cache.manager import CallCacheView
from ..weights.loader import TensorSpec


# ---- what a step hands to the parts ---------------------------------------------------------
@dataclass
class StepContext:
    """One batch of (request, its next tokens), flattened.  Device tensors are int32.

    Token ``n`` belongs to segment ``tok_seg[n]`` and sits at absolute position ``positions[n]``
    of its request.  Segment ``s`` covers tokens ``seg_start[s] .. seg_start[s] + seg_len[s]``,
    the first of them at position ``seg_pos0[s]``.  ``tables[g][s]`` is the block table of
    segment ``s`` in cache group ``g``; ``slots[s]`` its state slot (``-1`` without state).
    The ``*_host`` lists carry the same numbers for parts that loop on the host.
    """
    n_tokens: int
    n_segments: int
    dtype: torch.dtype
    device: torch.device
    token_ids: torch.Tensor
    positions: torch.Tensor
    tok_seg: torch.Tensor
    tables: List[torch.Tensor]
    slots: Optional[torch.Tensor]
    seg_start_host: Sequence[int]
    seg_len_host: Sequence[int]
    seg_pos0_host: Sequence[int]
    slots_host: Sequence[int]
    position_axes: Optional[torch.Tensor] = None   # int32 [position_width, n_tokens]; row 0 is ``positions``
    decode_only: bool = False
    max_kv_len: int = 0                       # longest context (after this step) among the segments
    extras: Dict[str, Any] = field(default_factory=dict)   # device tensors of special paths (decode kernels)
    step_cache: Dict[Any, Any] = field(default_factory=dict)   # what parts share across the layers of ONE step
    #                                           (cleared by Model.forward; e.g. the step's rotation angles)

    def empty(self, *shape: int, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)


@dataclass
class ResidualStream:
    """The float32 residual ``h`` and a branch output ``delta`` that is not added to it yet.  ``delta`` is
    ``[tokens, hidden]`` of the step's type, or float32 partial sums ``[parts, tokens, hidden]`` of it (a product whose
    K was cut, ``ops.linear_for_residual``), which the norm that folds it adds in order and rounds to the step's type."""
    h: torch.Tensor
    delta: Optional[torch.Tensor] = None


# ---- part interfaces ------------------------------------------------------------------------
class Part:
    # True: ``forward`` only launches kernels whose arguments are device tensors of the step, with shapes that
    # depend on the step's counts alone (tokens, segments, tiles, wanted rows), so the step may be captured in a
    # CUDA graph and replayed for other steps of the same counts.  A part that loops on the host over the step's
    # segments (``ctx.*_host``) must leave it False; the engine then runs every step of its model eagerly.
    capture_safe = False

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {}

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """Receive the loaded tensors (local names).  May fuse or re-lay them out."""


class Norm(Part):
    def forward(self, x: torch.Tensor, out: torch.Tensor) -> None:
        raise NotImplementedError

    def forward_residual(self, stream: ResidualStream, out: torch.Tensor,
                         row_idx: Optional[torch.Tensor] = None) -> None:
        """Fold ``stream.delta`` into ``stream.h`` (float32 add) and write ``norm(h)`` to ``out``.

        With ``row_idx`` only those rows are produced and the stream is left as it is.
        """
        raise NotImplementedError


class Embedding(Part):
    """Token ids to the float32 residual stream: ``forward(ids, out[N, hidden])``.  ``tied_weight()`` is what a head
    with tied weights may use as its own (None: nothing to share)."""

    def forward(self, ids: torch.Tensor, out: torch.Tensor) -> None:
        raise NotImplementedError

    def tied_weight(self) -> Optional[torch.Tensor]:
        return None


class Head(Part):
    """Normed hidden states of the wanted rows to float32 logits: ``forward(x[rows, hidden], out[rows, vocab])``.
    ``bind`` also receives the embedding's ``tied_weight()``."""

    def bind(self, tensors: Mapping[str, torch.Tensor], embedding: Optional[torch.Tensor] = None) -> None:
        raise NotImplementedError

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> None:
        raise NotImplementedError


class PositionEncoding(Part):
    def rotate_append(self, qkv: torch.Tensor, q_out: torch.Tensor, cache: CallCacheView, ctx: StepContext,
                      n_heads: int, n_kv_heads: int, head_dim: int, write_kv: bool) -> None:
        raise NotImplementedError

    def project_rotate_append(self, x: torch.Tensor, w_qkv: torch.Tensor, b_qkv: Optional[torch.Tensor],
                              q_out: torch.Tensor, cache: CallCacheView, ctx: StepContext, n_heads: int,
                              n_kv_heads: int, head_dim: int, write_kv: bool) -> bool:
        """Optional: the stacked q/k/v product, the position rule and the cache append in one kernel.  Returns
        False when this encoding (or this step) has no such kernel; the mixer then does the product itself and
        calls :meth:`rotate_append`."""
        return False


class Mixer(Part):
    def cache_need(self):
        """``PagedKVNeed``, ``StateNeed`` or ``None``."""
        return None

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CallCacheView, owns_cache: bool) -> torch.Tensor:
        """``y [tokens, hidden]`` of x's type."""
        raise NotImplementedError

    def forward_for_residual(self, x: torch.Tensor, ctx: StepContext, cache: CallCacheView,
                             owns_cache: bool) -> torch.Tensor:
        """Optional.  For an arrangement that puts the result straight into ``ResidualStream.delta``: the same as
        :meth:`forward`, or float32 partial sums ``[parts, tokens, hidden]`` of it where that is faster (see
        ``ops.linear_for_residual``); the norm that folds the branch adds them."""
        return self.forward(x, ctx, cache, owns_cache)


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        """``y [tokens, hidden]`` of x's type."""
        raise NotImplementedError

    def forward_for_residual(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        """Optional; as :meth:`Mixer.forward_for_residual`."""
        return self.forward(x, ctx)


class Block:
    """Arrangement of a layer's parts around the residual stream.  ``parts`` maps role names to built parts: the
    usual ``"mixer"``, ``"ffn"`` and norms, or whatever else the layer's spec names.  ``forward`` receives the
    caches of the call by the role of the mixer they belong to (``caches["mixer"]`` for the usual one)."""
    capture_safe = False                  # see Part.capture_safe; an arrangement says so for its own code

    def __init__(self, parts: Mapping[str, Part]):
        self._parts: Dict[str, Part] = dict(parts)
        self.mixer: Optional[Mixer] = self._parts.get("mixer")
        self.ffn: Optional[FeedForward] = self._parts.get("ffn")
        self.norms: Dict[str, Norm] = {role: part for role, part in self._parts.items() if isinstance(part, Norm)}

    def parts(self) -> Dict[str, Part]:
        return dict(self._parts)

    def mixers(self) -> Dict[str, Mixer]:
        """The layer's mixers by role: each gets a cache of its own in every call of the layer."""
        return {role: part for role, part in self._parts.items() if isinstance(part, Mixer)}

    def forward(self, stream: ResidualStream, ctx: StepContext, caches: Mapping[str, CallCacheView],
                owns_cache: bool) -> None:
        raise NotImplementedError


# ---- registries -----------------------------------------------------------------------------
_REGISTRIES: Dict[str, Dict[str, Callable[..., Any]]] = {
    "norm": {}, "position": {}, "mixer": {}, "ffn": {}, "block": {}, "embedding": {}, "head": {},
}


def _register(family: str, kind: str):
    def deco(cls):
        _REGISTRIES[family][kind] = cls
        return cls
    return deco


def register_norm(kind: str):
    return _register("norm", kind)


def register_position(kind: str):
    return _register("position", kind)


def register_mixer(kind: str):
    return _register("mixer", kind)


def register_feed_forward(kind: str):
    return _register("ffn", kind)


def register_block(kind: str):
    return _register("block", kind)


def register_embedding(kind: str):
    return _register("embedding", kind)


def register_head(kind: str):
    return _register("head", kind)


def unregister(family: str, kind: str) -> None:
    _REGISTRIES[family].pop(kind, None)


def build_part(family: str, spec) -> Any:
    """Construct a part from a :class:`~zedinfer_b200.config.spec.PartSpec`."""
    table = _REGISTRIES[family]
    if spec.kind not in table:
        raise KeyError(f"no {family} of kind {spec.kind!r} is registered (known: {', '.join(sorted(table)) or 'none'})")
    return table[spec.kind](**dict(spec.params))


def block_class(kind: str):
    table = _REGISTRIES["block"]
    if kind not in table:
        raise KeyError(f"no block arrangement {kind!r} is registered (known: {', '.join(sorted(table)) or 'none'})")
    return table[kind]
