"""Grouped-query attention whose queries and keys pass a short convolution over time and a norm over the whole
projection, and whose values are the keys.

``q, k = conv(Wq x), conv(Wk x)`` with ``conv(u)_t = sum_j w[:, j] * u_(t - taps + 1 + j)`` per channel (zeros before
the sequence's start; the last ``taps - 1`` projected rows of a sequence are part of its state).  The values are the
keys as they leave the convolution: there is no value projection.  Then ``q`` and ``k`` are RMS-normed over ALL their
channels at once (before they are split into heads) with gains of that size.  No rotation: positions enter only
through the mask.  Scores ``(q . k) * scale`` over the visible keys (causal; with ``chunk``, only keys of the query's
own chunk of that many positions, counted from position 0), ordinary softmax, query head ``h`` reading kv head
``h // (heads / kv_heads)``.  With ``gated`` the concatenated heads are multiplied element by element with
``sigmoid(Wg x)`` before the output projection.

Cache: the library's paged keys and values (``KVRequest(kv_heads, dim, chunk=)``: pages behind the chunk a sequence has
reached are given back) bundled with the convolutions' history (``StateRequest((taps - 1, Cq + Ck))``, 32-bit).

The part runs alone (it owns its projections) or ``shared`` beside other mixers under one owner that stacks the
projections of all of them (``input_parts``, ``output_part``, ``mix``).
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional

import torch

from .. import ops
from ..cache.store import BundleRequest, KVRequest, StateRequest
from ..weights.loader import TensorSpec
from .base import Mixer, Part, Runtime, StepContext, to_device_f32
from .linear import Linear


class ConvNormAttention(Mixer):
    accepts_lazy_input = False
    can_defer_output = False

    NAMES = {"q": "q", "k": "k", "g": "g", "o": "o", "q_conv": "q.conv", "k_conv": "k.conv", "q_norm": "q.norm", "k_norm": "k.norm"}

    def __init__(self, prefix: str, width: int, heads: int, kv_heads: int, dim: int, *, taps: int, scale: float, norm_eps: float,
                 chunk: Optional[int] = None, window: Optional[int] = None, gated: bool = True,
                 names: Optional[Mapping[str, str]] = None, shared: bool = False):
        if heads % kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        if taps < 1:
            raise ValueError("a convolution has at least one tap")
        if chunk is not None and chunk <= 0:
            raise ValueError("chunk must be > 0")
        self.prefix, self.width = prefix, width
        self.heads, self.kv_heads, self.dim, self.taps = heads, kv_heads, dim, taps
        self.scale, self.norm_eps = float(scale), float(norm_eps)
        self.chunk, self.window, self.gated = chunk, window, bool(gated)
        self.names = dict(self.NAMES, **(names or {}))
        self.shared = bool(shared)
        self.cq, self.ck = heads * dim, kv_heads * dim
        self.proj = self.o = None
        if not shared:
            names_in, outs = zip(*self.input_parts())
            self.proj = Linear(list(names_in), width, list(outs))
            self.o = Linear(self.output_part()[0], self.output_part()[1], width)
        self.taps_q = self.taps_k = self.gain_q = self.gain_k = None

    def input_parts(self):
        """``(tensor name, outputs)`` of the projections, in the order of their columns: q, k[, g]."""
        p, n = self.prefix, self.names
        parts = [(p + n["q"], self.cq), (p + n["k"], self.ck)]
        if self.gated:
            parts.append((p + n["g"], self.cq))
        return parts

    def output_part(self):
        return self.prefix + self.names["o"], self.cq

    def children(self) -> List[Part]:
        return [] if self.shared else [self.proj, self.o]

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        p, n = self.prefix, self.names
        return {p + n["q_conv"]: TensorSpec((self.cq, self.taps), "bias"), p + n["k_conv"]: TensorSpec((self.ck, self.taps), "bias"),
                p + n["q_norm"]: TensorSpec((self.cq,), "gain"), p + n["k_norm"]: TensorSpec((self.ck,), "gain")}

    def bind(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        p, n = self.prefix, self.names
        # taps-major on the device ([taps, channels]): neighbouring channels' weights of one tap lie together
        self.taps_q = to_device_f32(tensors[p + n["q_conv"]].t(), rt)
        self.taps_k = to_device_f32(tensors[p + n["k_conv"]].t(), rt)
        self.gain_q = to_device_f32(tensors[p + n["q_norm"]], rt)
        self.gain_k = to_device_f32(tensors[p + n["k_norm"]], rt)

    def cache_request(self):
        return BundleRequest((KVRequest(self.kv_heads, self.dim, self.window, None, self.chunk),
                              StateRequest((self.taps - 1, self.cq + self.ck), torch.float32)))

    def mix(self, proj: torch.Tensor, col: int, ctx: StepContext, views, write_cache: bool = True, **_) -> torch.Tensor:
        """From a projection whose columns from ``col`` on are this part's q, k (and gate): what the output projection
        reads, ``[T, heads * dim]``."""
        kv, hist = views
        bt = ctx.block_tables[kv.group]
        q = ops.convqk_prepare(proj, col, col + self.cq, self.heads, self.kv_heads, self.dim, self.taps_q, self.taps_k,
                               self.gain_q, self.gain_k, self.norm_eps, hist, ctx, bt, kv.k if write_cache else None,
                               kv.v if write_cache else None)
        y = ops.attention(q, kv.k, kv.v, ctx, bt, self.heads, self.kv_heads, self.dim, self.scale, self.window, chunk=self.chunk)
        if self.gated:
            ops.sigmoid_gate(y, proj, col + self.cq + self.ck)
        return y

    def forward(self, x: torch.Tensor, ctx: StepContext, views, write_cache: bool = True) -> torch.Tensor:
        return self.o.forward(self.mix(self.proj.forward(x), 0, ctx, views, write_cache))
