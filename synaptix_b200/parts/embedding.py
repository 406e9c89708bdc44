"""Token embedding and the output head.

``h0[t] = E[id_t]`` with no scale (crates/synaptix-ops/src/embed/token_embed.rs:4-15);
logits ``= norm(h)[rows] W^T`` with ``W = E`` when tied
(crates/synaptix-models/llm/common/src/model.rs:757-772,1068-1094), computed only for
the rows asked for and returned in float32.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import Part, Runtime, to_device_matrix
from .linear import Linear


class Embedding(Part):
    """``scale``: the gathered rows are multiplied by it (in 32-bit, on their way into the stream)."""

    def __init__(self, weight_name: str, vocab: int, width: int, scale: float = 1.0):
        self.weight_name, self.vocab, self.width = weight_name, vocab, width
        self.scale = float(scale)
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.weight_name: TensorSpec((self.vocab, self.width), "embedding")}

    def bind(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        self.weight = to_device_matrix(tensors[self.weight_name], rt)

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        """float32 residual stream ``[T, width]``."""
        return ops.embed_gather(self.weight, token_ids, scale=self.scale)


class BigramEmbedding(Embedding):
    """The token's row plus a row of a second table chosen by the pair (token before, token):
    ``E[id_t] + B[(id_(t-1) * mul_prev + id_t * mul_cur) mod buckets]`` with ``B [buckets + 1, width]``, whose last row
    stands for a sequence's first token.  The token before is part of a sequence's state: the model gives this part a
    cache entry (``cache_request``: one int32 per sequence) and calls ``forward_step(ctx, state)``."""

    def __init__(self, weight_name: str, bigram_name: str, vocab: int, width: int, buckets: int, mul_prev: int, mul_cur: int):
        super().__init__(weight_name, vocab, width)
        if buckets <= 0 or mul_prev < 0 or mul_cur < 0:
            raise ValueError("buckets > 0 and multipliers >= 0")
        self.bigram_name, self.buckets, self.mul_prev, self.mul_cur = bigram_name, int(buckets), int(mul_prev), int(mul_cur)
        self.bigram: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.weight_name: TensorSpec((self.vocab, self.width), "embedding"),
                self.bigram_name: TensorSpec((self.buckets + 1, self.width), "embedding")}

    def bind(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        super().bind(tensors, rt)
        self.bigram = to_device_matrix(tensors[self.bigram_name], rt)

    def cache_request(self):
        from ..cache.store import StateRequest
        return StateRequest((), torch.int32)

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        raise TypeError("an embedding with a state is called with the step: forward_step(ctx, state)")

    def forward_step(self, ctx, state: torch.Tensor) -> torch.Tensor:
        """float32 residual stream ``[T, width]``; ``state`` int32 ``[slots]`` (each sequence's last token) is moved on."""
        return ops.embed_bigram(self.weight, self.bigram, ctx, state, self.mul_prev, self.mul_cur)


class OutputHead(Part):
    """``tied`` is True, False, or None (= tied iff the weights hold no matrix of that name).  ``scale``: the logits
    are multiplied by it (in 32-bit)."""

    def __init__(self, weight_name: str, vocab: int, width: int, tied: Optional[bool], embedding: Embedding,
                 scale: float = 1.0):
        self.weight_name, self.vocab, self.width = weight_name, vocab, width
        self.scale = float(scale)
        self.tied = tied
        self.embedding = embedding
        self.linear = Linear(weight_name, width, vocab)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        # a tied checkpoint may still carry a copy of the matrix; it is then ignored
        return {self.weight_name: TensorSpec((self.vocab, self.width), "matrix", optional=self.tied is not False)}

    def bind(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        tied = self.tied if self.tied is not None else (self.weight_name not in tensors)
        if tied:
            self.linear.share(self.embedding.weight)
        else:
            self.linear.bind(tensors, rt)
        self.is_tied = tied

    def forward(self, x) -> torch.Tensor:
        """``x``: the normalised rows, or a ``PendingNorm`` of them."""
        logits = self.linear.forward(x, out_dtype=torch.float32)
        if self.scale != 1.0:
            ops.scale_rows(logits, self.scale)
        return logits
