"""Architecture-neutral description of a model: parts, layers, and the run order.

A model is data: a tuple of :class:`LayerSpec` (which mixer, feed-forward, norms
and arrangement a layer has, each with its own sizes and constants) and a
*schedule*, the list of :class:`LayerCall` that says in which order layers run.
The schedule may name a layer twice (its weights are then used twice, each call
with a cache of its own) or let a call read the cache that an earlier call
wrote.  Nothing in here knows about a particular architecture; the files under
``zedinfer_b200/models`` translate an architecture's ``config.json`` into these
objects.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: a registered ``kind`` plus its constructor keywords."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def with_params(self, **kw: Any) -> "PartSpec":
        merged = dict(self.params)
        merged.update(kw)
        return PartSpec(self.kind, merged)


@dataclass(frozen=True)
class LayerSpec:
    """A layer: the arrangement (``block``) of its parts, each under a role name.

    The usual layer has one mixer (role ``"mixer"``), one feed-forward (``"ffn"``) and norms (``"norm1"``,
    ``"norm2"``, ...).  A layer may also have none of one (``mixer=None`` or ``ffn=None``) or more parts than
    these: ``extra`` maps further role names to ``(family, spec)``, the family being one of the part registries
    (``"mixer"``, ``"ffn"``, ``"norm"``, ``"position"``), e.g. ``{"mixer2": ("mixer", PartSpec("toy_decay", ...))}``.
    Which roles an arrangement expects is the arrangement's business; every mixer of a layer, whatever its role,
    gets a cache of its own per call.

    ``prefixes`` maps each role to the tensor-name prefix below the layer's own prefix, e.g.
    ``{"mixer": "self_attn.", "norm1": "input_layernorm."}``; a role without an entry uses ``"<role>."``.
    """

    block: str
    mixer: Optional[PartSpec]
    ffn: Optional[PartSpec]
    norms: Mapping[str, PartSpec]
    prefixes: Mapping[str, str]
    extra: Mapping[str, Tuple[str, PartSpec]] = field(default_factory=dict)

    def part_specs(self) -> Tuple[Tuple[str, str, PartSpec], ...]:
        """(role, family, spec) of every part of the layer, in a fixed order."""
        out = []
        if self.mixer is not None:
            out.append(("mixer", "mixer", self.mixer))
        if self.ffn is not None:
            out.append(("ffn", "ffn", self.ffn))
        out.extend((role, "norm", ns) for role, ns in self.norms.items())
        for role, (family, ps) in self.extra.items():
            if role in ("mixer", "ffn") or role in self.norms:
                raise ValueError(f"extra part {role!r} repeats a role the layer already has")
            out.append((role, family, ps))
        return tuple(out)


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    ``layer`` indexes :attr:`ModelSpec.layers`.  ``cache_of`` is ``None`` when the
    call owns a cache of its own, else the index (into the schedule) of an earlier
    call whose cache this call reads without writing to it.
    """

    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[LayerCall, ...]
    final_norm: PartSpec
    tie_word_embeddings: bool
    max_position_embeddings: int
    layer_prefix: str = "layers.{i}."
    embed_name: str = "embed_tokens.weight"
    final_norm_prefix: str = "norm."
    head_name: str = "lm_head.weight"
    bos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()
    # The parts at the two ends of the model, registered like every other part.  None: the plain table look-up
    # ("token_embedding") and the bias-free product with the head weight, or the embedding table when tied
    # ("output_head"), built from vocab_size, hidden_size, embed_name, head_name and tie_word_embeddings.
    embedding: Optional[PartSpec] = None
    head: Optional[PartSpec] = None
    # How many position numbers a token carries (axes of a multi-axis position rule).  The step's descriptor, the
    # captured decode step and the on-device hand-over between decode steps all carry this many per token; every
    # axis of a text token holds its index in the request.  Parts read ``StepContext.position_axes`` ([width, tokens]);
    # ``StepContext.positions`` is axis 0.
    position_width: int = 1

    def validate(self) -> None:
        if self.vocab_size <= 0 or self.hidden_size <= 0:
            raise ValueError("vocab_size and hidden_size must be positive")
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        if self.position_width < 1:
            raise ValueError(f"position_width={self.position_width} must be at least 1")
        for pos, call in enumerate(self.schedule):
            if not 0 <= call.layer < len(self.layers):
                raise ValueError(f"schedule[{pos}] names layer {call.layer}, "
                                 f"but the model has {len(self.layers)} layers")
            if call.cache_of is not None:
                if not 0 <= call.cache_of < pos:
                    raise ValueError(f"schedule[{pos}].cache_of={call.cache_of} must name an earlier call")
                if self.schedule[call.cache_of].cache_of is not None:
                    raise ValueError(f"schedule[{pos}].cache_of names a call that itself borrows a cache")
