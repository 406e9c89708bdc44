"""Grouped-query attention over the paged cache whose weights need not be a plain softmax of each head's own scores.

``q, k, v = Wq x (+ bq), Wk x (+ bk), Wv x (+ bv)``; per-head RMS norm of q and k with one gain shared by all heads
(optional); rotation of neighbouring pairs of the first elements of a head (optional, any ``PositionEncoding`` that
says ``pairs``); then, for the query at position ``i`` and the key at ``j`` (visible iff ``0 <= i - j < window``):

* ``talk``: the heads' scaled scores are mixed, ``s'_h = sum_g T[h, g] s_g`` with a learned ``[H, H]``;
* ``head_bias``: a learned number per head is added; ``distance_bias=(rows, far)``: a learned table ``[rows, H]`` gives
  a number per head and distance bucket, ``bucket(n) = n`` below ``rows / 2`` and logarithmic up to ``far`` beyond
  (``rows`` None: as many as the tensor has);
* ``weights="softmax"`` over the visible keys, or ``"sigmoid"``: every visible key weighs ``sigmoid(s')``, unnormalised;
* ``value_mix``: ``"source"`` keeps this layer's values for the step under ``value_key``; ``"blend"`` replaces its own by
  ``(1 - lam) v + lam v_source`` with a learned scalar before they are cached;
* ``head_gate``: head ``h``'s result is multiplied by ``sigmoid(Wg x)_h``.

All projections of the input run as one product whose result stays 32-bit; biases, norm, rotation, blend and gate are
one kernel behind it.  ``names`` maps q, k, v, o, g, q_norm, k_norm, talk, head_bias, distance, lam to tensor names.
"""
from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional, Tuple

import numpy as np
import torch

from .. import ops
from ..cache.store import KVRequest, KVView
from ..weights.loader import TensorSpec
from .base import Mixer, Part, PositionEncoding, Runtime, StepContext, to_device_f32
from .linear import Linear


def distance_bucket(n: int, rows: int, far: float) -> int:
    """``n`` below ``rows / 2``; beyond, ``rows / 2`` more buckets spread evenly over ``ln n`` up to ``far``."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def distance_columns(rows: int, far: float, window: Optional[int]) -> np.ndarray:
    """The bucket of every distance ``0 .. n - 1`` where all distances from ``n - 1`` on share a bucket (or lie beyond
    the window)."""
    n = 1
    while distance_bucket(n - 1, rows, far) < rows - 1 and (window is None or n < window):
        n += 1
    return np.asarray([distance_bucket(d, rows, far) for d in range(n)], dtype=np.int64)


class ScoredAttention(Mixer):
    NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "g": "g", "q_norm": "q.norm", "k_norm": "k.norm", "talk": "talk",
             "head_bias": "pb", "distance": "rel", "lam": "vmix", "bias_suffix": ".b"}

    def __init__(self, prefix: str, width: int, n_heads: int, n_kv_heads: int, head_dim: int, v_head_dim: int, *,
                 scale: float, position: Optional[PositionEncoding] = None, window: Optional[int] = None,
                 biases: bool = False, qk_norm_eps: Optional[float] = None, talk: bool = False, head_bias: bool = False,
                 distance_bias: Optional[Tuple[int, float]] = None, weights: str = "softmax",
                 value_mix: Optional[str] = None, value_key: str = "values", head_gate: bool = False,
                 names: Optional[Mapping[str, str]] = None):
        if n_heads % n_kv_heads:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        if weights not in ("softmax", "sigmoid"):
            raise ValueError("weights are 'softmax' or 'sigmoid'")
        if value_mix not in (None, "source", "blend"):
            raise ValueError("value_mix is None, 'source' or 'blend'")
        if position is not None and getattr(position, "rotary_dim", 0) and not getattr(position, "pairs", False):
            raise ValueError("this attention rotates neighbouring pairs")
        self.prefix, self.width = prefix, width
        self.nh, self.nkv, self.hd, self.vd = n_heads, n_kv_heads, head_dim, v_head_dim
        self.scale, self.window = float(scale), window
        self.position = position
        self.biases, self.qk_norm_eps = bool(biases), qk_norm_eps
        self.talk, self.head_bias, self.distance_bias = bool(talk), bool(head_bias), distance_bias
        self.softmax = weights == "softmax"
        self.value_mix, self.value_key, self.head_gate = value_mix, value_key, bool(head_gate)
        self.names = n = dict(self.NAMES, **(names or {}))
        parts = [(prefix + n["q"], n_heads * head_dim), (prefix + n["k"], n_kv_heads * head_dim),
                 (prefix + n["v"], n_kv_heads * v_head_dim)]
        if head_gate:
            parts.append((prefix + n["g"], n_heads))
        self.proj = Linear([p[0] for p in parts], width, [p[1] for p in parts])
        self._bias_names = [p[0] + n["bias_suffix"] for p in parts[:3]] if biases else []
        self._bias_sizes = [p[1] for p in parts]
        self.o = Linear(prefix + n["o"], n_heads * v_head_dim, width)
        self.proj_bias = self.output_bias = self.q_gain = self.k_gain = None
        self.talk_matrix = self.head_bias_vector = self.distance_table = self.lam = None

    def children(self) -> List[Part]:
        return [self.proj, self.o] + ([self.position] if self.position is not None else [])

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        n, p = self.names, self.prefix
        specs = {}
        for name, size in zip(self._bias_names, self._bias_sizes):
            specs[name] = TensorSpec((size,), "bias")
        if self.biases:
            specs[p + n["o"] + n["bias_suffix"]] = TensorSpec((self.width,), "bias")
        if self.qk_norm_eps is not None:
            specs[p + n["q_norm"]] = TensorSpec((self.hd,), "gain")
            specs[p + n["k_norm"]] = TensorSpec((self.hd,), "gain")
        if self.talk:
            specs[p + n["talk"]] = TensorSpec((self.nh, self.nh), "matrix")
        if self.head_bias:
            specs[p + n["head_bias"]] = TensorSpec((self.nh,), "bias")
        if self.distance_bias is not None:
            rows = self.distance_bias[0]            # None: as many rows as the tensor has
            specs[p + n["distance"]] = TensorSpec((-1 if rows is None else rows, self.nh), "bias")
        if self.value_mix is not None:
            specs[p + n["lam"]] = TensorSpec((), "bias")
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        n, p = self.names, self.prefix
        if self.biases:
            cols = [tensors[b].to(torch.float32) for b in self._bias_names]
            if self.head_gate:
                cols.append(torch.zeros(self.nh, dtype=torch.float32, device=cols[0].device))       # the gate's projection has no bias
            self.proj_bias = to_device_f32(torch.cat(cols), rt)
            self.output_bias = to_device_f32(tensors[p + n["o"] + n["bias_suffix"]], rt)
        if self.qk_norm_eps is not None:
            self.q_gain = to_device_f32(tensors[p + n["q_norm"]], rt)
            self.k_gain = to_device_f32(tensors[p + n["k_norm"]], rt)
        if self.talk:
            self.talk_matrix = to_device_f32(tensors[p + n["talk"]], rt)
        if self.head_bias:
            self.head_bias_vector = to_device_f32(tensors[p + n["head_bias"]], rt)
        if self.distance_bias is not None:
            # the table as the kernel reads it: [H, distances], the bucket of every distance looked up once
            table = tensors[p + n["distance"]].to(torch.float32)
            cols = distance_columns(table.shape[0], self.distance_bias[1], self.window)
            table = table[torch.from_numpy(cols).to(table.device)]                                               # [distances, H]
            self.distance_table = to_device_f32(table.t(), rt)
        if self.value_mix == "blend":
            self.lam = to_device_f32(tensors[p + n["lam"]].reshape(1), rt)

    def cache_request(self):
        return KVRequest(self.nkv, self.hd, self.window, None if self.vd == self.hd else self.vd)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache_view: KVView, write_cache: bool = True) -> torch.Tensor:
        T = x.shape[0]
        proj = self.proj.forward(x, out_dtype=torch.float32)
        rot = self.position.rotation() if self.position is not None else None
        inv_freq, rot_dims = rot if rot is not None else (None, 0)
        bt = ctx.block_tables[cache_view.group]
        q = torch.empty((T, self.nh * self.hd), dtype=x.dtype, device=x.device)
        gate = torch.empty((T, self.nh), dtype=torch.float32, device=x.device) if self.head_gate else None
        v_in = v_out = None
        if self.value_mix == "source":
            v_out = ctx.scratch[("value_mix", self.value_key)] = torch.empty((T, self.nkv * self.vd), dtype=torch.float32,
                                                                              device=x.device)
        elif self.value_mix == "blend":
            v_in = ctx.scratch[("value_mix", self.value_key)]
        ops.heads_prepare(proj, self.proj_bias, q, cache_view.k if write_cache else None,
                          cache_view.v if write_cache else None, ctx.positions, ctx.seq_of_token, bt, self.nh, self.nkv,
                          self.hd, self.vd, q_gain=self.q_gain, k_gain=self.k_gain,
                          eps=self.qk_norm_eps if self.qk_norm_eps is not None else 0.0, inv_freq=inv_freq,
                          rot_dims=rot_dims, magnitude=getattr(self.position, "magnitude", 1.0), v_first_in=v_in,
                          v_first_out=v_out, lam=self.lam, gate_out=gate)
        a = ops.attn_scored(q, cache_view.k, cache_view.v, ctx, bt, self.nh, self.nkv, self.hd, self.vd, self.scale,
                            self.window, talk=self.talk_matrix, head_bias=self.head_bias_vector,
                            dist_bias=self.distance_table, softmax=self.softmax, gate=gate)
        return self.o.forward(a)
