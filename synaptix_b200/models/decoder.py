"""A decoder model as data: parts, and the order in which layers run.

``layers`` are blocks; ``schedule`` lists the runs of a step in order.  An embedding that carries a state per
sequence (``cache_request`` / ``forward_step``) gets a cache entry of its own behind the layers' entries.  A run
names a layer and the cache entry it works on, so a schedule may run a layer
twice (two runs, each with a cache entry of its own) or let a layer read the
cache another layer wrote (``write_cache=False`` and that layer's entry).  The
default schedule runs every layer once on its own entry.  Between two runs a
schedule may hold an ``Inject``: vectors added into the residual stream there
(the embedding output once more, a row of the model's table of stream vectors),
which is what a model needs that runs a stretch of layers several times and
marks each pass.

Step (crates/synaptix-models/llm/common/src/model.rs:1057-1117,1160-1262):
embedding -> runs -> final norm on the rows whose logits are wanted -> output
head.  The reference normalises all rows and then narrows (model.rs:1068-1074);
here only the wanted rows are normalised and projected.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Sequence

import torch

from ..cache.store import CacheRequest
from .. import ops
from ..parts.base import Norm, Part, PendingLinear, Runtime, StepContext, plain, to_device_f32
from ..parts.embedding import Embedding, OutputHead
from ..weights.loader import TensorSpec, WeightSource, bind_tensors


@dataclasses.dataclass(frozen=True)
class LayerRun:
    layer: int
    cache_entry: int
    write_cache: bool = True


@dataclasses.dataclass(frozen=True)
class Inject:
    """Between two runs: ``h += embedding output`` (the stream as the embedding left it) if ``embedding``, and
    ``h += stream_vectors[row]`` if ``row`` is not ``None``."""
    embedding: bool = False
    row: Optional[int] = None


class StreamVectors(Part):
    """A table ``[rows, width]`` of vectors that a schedule adds into the residual stream (``Inject.row``)."""

    def __init__(self, name: str, rows: int, width: int):
        self.name, self.rows, self.width = name, rows, width
        self.table: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.name: TensorSpec((self.rows, self.width), "embedding")}

    def bind(self, tensors, rt: Runtime) -> None:
        self.table = to_device_f32(tensors[self.name], rt)


class DecoderModel(Part):
    def __init__(self, config, embedding: Embedding, layers: Sequence[Part], final_norm: Norm,
                 head: OutputHead, schedule: Optional[Sequence] = None,
                 stop_token_ids: Sequence[int] = (), stream_vectors: Optional[StreamVectors] = None):
        self.config = config
        self.embedding = embedding
        self.layers = list(layers)
        self.final_norm = final_norm
        self.head = head
        self.steps = list(schedule) if schedule is not None else [
            LayerRun(i, i) for i in range(len(self.layers))]
        self.schedule = [r for r in self.steps if isinstance(r, LayerRun)]
        self.stream_vectors = stream_vectors
        for r in self.steps:
            if isinstance(r, Inject) and r.row is not None and (
                    stream_vectors is None or not (0 <= r.row < stream_vectors.rows)):
                raise ValueError(f"the schedule adds stream vector {r.row}, which the model does not have")
        self._keeps_embedding = any(isinstance(r, Inject) and r.embedding for r in self.steps)
        self.stop_token_ids = tuple(stop_token_ids)
        self.runtime: Optional[Runtime] = None
        n_entries = 1 + max((r.cache_entry for r in self.schedule), default=-1)
        owners: List[Optional[int]] = [None] * n_entries
        for r in self.schedule:
            if not (0 <= r.layer < len(self.layers)):
                raise ValueError(f"schedule names layer {r.layer}, the model has {len(self.layers)}")
            if r.write_cache:
                if owners[r.cache_entry] is not None:
                    raise ValueError(f"cache entry {r.cache_entry} is written by two runs")
                owners[r.cache_entry] = r.layer
        for r in self.schedule:
            if owners[r.cache_entry] is None:
                raise ValueError(f"cache entry {r.cache_entry} is read but never written")
        self._entry_owner = owners
        # an embedding with a state of its own (the token before) gets the cache entry behind the layers' entries
        self._embedding_entry = n_entries if getattr(embedding, "cache_request", None) is not None else None
        if self._embedding_entry is not None and self._keeps_embedding:
            raise ValueError("a schedule that adds the embedding again needs an embedding without a state")

    @property
    def vocab_size(self) -> int:
        return self.head.vocab

    def children(self) -> List[Part]:
        extra = [self.stream_vectors] if self.stream_vectors is not None else []
        return [self.embedding] + extra + self.layers + [self.final_norm, self.head]

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {}

    def cache_requests(self) -> List[CacheRequest]:
        """One request per cache entry, asked of the layer that writes it."""
        requests = [self.layers[o].cache_request() for o in self._entry_owner]
        if self._embedding_entry is not None:
            requests.append(self.embedding.cache_request())
        return requests

    # -- weights -----------------------------------------------------------
    def load(self, source: WeightSource, rt: Runtime, where: str = "weights") -> "DecoderModel":
        tensors = bind_tensors(self.all_tensor_specs(), source, where=where)
        self.bind_all(tensors, rt)
        self.runtime = rt
        return self

    # -- one step ------------------------------------------------------------
    def forward(self, ctx: StepContext, cache) -> torch.Tensor:
        """Logits float32 ``[n_want, vocab]`` for ``ctx.want_rows``."""
        if self._embedding_entry is not None:
            h = self.embedding.forward_step(ctx, cache.view(self._embedding_entry))
        else:
            h = self.embedding.forward(ctx.token_ids)
        h0 = self.embedding.forward(ctx.token_ids) if self._keeps_embedding else None     # h is summed into in place
        pending = None
        observe = getattr(ctx, "observe", None)
        n_run = 0
        for run in self.steps:
            if isinstance(run, Inject):
                ops.stream_add(h, plain(pending), h0 if run.embedding else None,
                               self.stream_vectors.table[run.row] if run.row is not None else None)
                pending = None
                continue
            if isinstance(pending, PendingLinear) and not getattr(self.layers[run.layer], "takes_pending_product", False):
                pending = pending.materialize()
            h, pending = self.layers[run.layer].forward(h, pending, ctx, cache.view(run.cache_entry), run.write_cache)
            if observe is not None:              # the stream after this run: h with the branch not yet added
                observe(n_run, h, plain(pending))
            n_run += 1
        if isinstance(pending, PendingLinear) and not self.final_norm.takes_pending_product:
            pending = pending.materialize()
        if getattr(ctx, "want_all", False):        # every row, in order: no gather, and the norm may fuse
            x = self.final_norm.add_forward(h, pending, lazy=True)
        else:
            x = self.final_norm.add_forward(h, pending, rows=ctx.want_rows)
        return self.head.forward(x)
