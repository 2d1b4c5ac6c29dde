"""Token embedding and output head.

``hidden[n, :] = table[ids[n], :]`` (src/frontend/models/transformer_forward.cpp:58-59);
``logits = norm(hidden) @ head^T`` without bias (:152-156), computed only for the rows that
are asked for and returned in float32.  With tied embeddings the head is the embedding table
(src/frontend/models/base.cpp:411-416)."""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import Embedding, Head, register_embedding, register_head


@register_embedding("token_embedding")
class TokenEmbedding(Embedding):
    capture_safe = True

    def __init__(self, vocab_size: int, hidden_size: int, name: str = "embed_tokens.weight"):
        self.vocab_size, self.hidden_size, self.name = int(vocab_size), int(hidden_size), name
        self.table: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.name: TensorSpec((self.vocab_size, self.hidden_size))}

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.table = tensors[self.name].contiguous()

    def forward(self, ids: torch.Tensor, out: torch.Tensor) -> None:
        ops.embedding(self.table, ids, out)

    def tied_weight(self) -> Optional[torch.Tensor]:
        return self.table


@register_head("output_head")
class OutputHead(Head):
    capture_safe = True

    def __init__(self, vocab_size: int, hidden_size: int, tied: bool, name: str = "lm_head.weight"):
        self.vocab_size, self.hidden_size, self.tied, self.name = int(vocab_size), int(hidden_size), bool(tied), name
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.name: TensorSpec((self.vocab_size, self.hidden_size), optional=self.tied)}

    def bind(self, tensors: Mapping[str, torch.Tensor], embedding: Optional[torch.Tensor] = None) -> None:
        if self.name in tensors:
            self.weight = tensors[self.name].contiguous()
        elif self.tied and embedding is not None:
            self.weight = embedding
        else:
            raise KeyError(self.name)

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> None:
        ops.linear(x, self.weight, None, out)
