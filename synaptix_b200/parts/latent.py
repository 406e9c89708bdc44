"""Attention over a cached latent: keys and values of all heads are made from one small vector per token.

Per token the layer keeps ``c = rmsnorm(Wdkv x)[:kv_rank] * gain`` and one rotated key part of ``rot_dim`` elements
that all heads share (the last rows of ``Wdkv``, not normed).  Head ``h`` has the key ``[Wuk_h c | k_rot]`` and the
value ``Wuv_h c``; its query ``[q_h | q_rot_h]`` comes through a latent of its own,
``Wuq (rmsnorm(Wdq x) * gain)``, or, with ``q_rank=None``, straight from the input (``Wq x``, tensor ``q``).  Scores are ``(q_h . Wuk_h c + q_rot_h . k_rot) * scale`` over the visible keys
(causal, optionally a sliding window of ``window`` positions, the query's own included), ordinary softmax; head
``h``'s result is multiplied by ``sigmoid(Wg x)_h`` and the heads go through ``Wo``.

The per-head keys and values are never formed.  ``q_h . Wuk_h c = (Wuk_h^T q_h) . c``, so the query is taken into the
latent's space once (``q' = [Wuk_h^T q_h | q_rot_h]``, ``kv_rank + rot_dim`` elements), attention runs with ONE key
row ``[c | k_rot]`` per token for all heads, its weights are applied to ``c`` itself, and ``Wuv_h`` is applied to the
weighted latent afterwards.  The cache therefore holds keys only (``KVRequest(keys_only=True)``), one head of
``kv_rank + rot_dim`` elements; the values are its first ``kv_rank`` elements.  Queries in the latent's space and the
weighted latents stay 32-bit.

Whole prompts in bfloat16 whose head sizes a tensor-core attention kernel takes (``dim + rot_dim == vdim`` of 32, 64 or
128) run the other form instead: the step's latents are read back from the cache, ONE product with ``[Wuk; Wuv]`` makes
all heads' keys and values, which go into pages of the step's own with the rotated part behind each head's key, and the
library's attention over paged keys and values runs on them (``ops.attention``); nothing of it outlasts the step.

A layer built with ``own_kv=False`` has no ``Wdkv``: the schedule gives it the cache entry of the layer whose latent
it reads (``LayerRun(..., write_cache=False)``); its ``Wuk``, ``Wuv``, queries, window and gate are its own.
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional

import torch

from .. import ops
from ..cache.store import KVRequest, KVView
from ..weights.loader import TensorSpec
from .base import Mixer, Part, PositionEncoding, Runtime, StepContext, to_device_f32, to_device_matrix
from .linear import Linear


class LatentAttention(Mixer):
    accepts_lazy_input = False
    can_defer_output = False

    NAMES = {"q": "q", "dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv",
             "g": "g", "o": "o"}

    def __init__(self, prefix: str, width: int, heads: int, dim: int, rot_dim: int, vdim: int, q_rank: Optional[int],
                 kv_rank: int, *,
                 scale: float, position: PositionEncoding, norm_eps: float, window: Optional[int] = None,
                 keep_window="own", own_kv: bool = True, gated: bool = True,
                 names: Optional[Mapping[str, str]] = None):
        """``keep_window``: how many latest keys the cache entry must keep (the largest window of the layers that read
        it, ``None`` for all); ``"own"``: this layer's ``window``."""
        self.prefix, self.width = prefix, width
        self.heads, self.dim, self.rot_dim, self.vdim = heads, dim, rot_dim, vdim
        self.q_rank, self.kv_rank = (q_rank or 0), kv_rank
        self.scale = float(scale)
        self.position = position
        self.norm_eps = float(norm_eps)
        self.window = window
        self.keep_window = window if keep_window == "own" else keep_window
        self.own_kv, self.gated = bool(own_kv), bool(gated)
        self.names = n = dict(self.NAMES, **(names or {}))
        p = prefix
        # the first columns of the stacked projection: the query latent, or the queries themselves
        parts = [(p + n["dq"], q_rank)] if self.q_rank else [(p + n["q"], heads * (dim + rot_dim))]
        self.col_dkv = self.col_g = -1
        if own_kv:
            self.col_dkv = parts[0][1]
            parts.append((p + n["dkv"], kv_rank + rot_dim))
        if gated:
            self.col_g = sum(o for _, o in parts)
            parts.append((p + n["g"], heads))
        self.proj = Linear([x for x, _ in parts], width, [o for _, o in parts])
        self.uq = Linear(p + n["uq"], q_rank, heads * (dim + rot_dim)) if self.q_rank else None
        self.o = Linear(p + n["o"], heads * vdim, width)
        self.dq_gain = self.dkv_gain = self.uk = self.uv = None

    def children(self) -> List[Part]:
        return [x for x in (self.proj, self.uq, self.o, self.position) if x is not None]

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        p, n = self.prefix, self.names
        specs = {p + n["uk"]: TensorSpec((self.heads * self.dim, self.kv_rank), "matrix"),
                 p + n["uv"]: TensorSpec((self.heads * self.vdim, self.kv_rank), "matrix")}
        if self.q_rank:
            specs[p + n["dq_norm"]] = TensorSpec((self.q_rank,), "gain")
        if self.own_kv:
            specs[p + n["dkv_norm"]] = TensorSpec((self.kv_rank,), "gain")
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        p, n = self.prefix, self.names
        if self.q_rank:
            self.dq_gain = to_device_f32(tensors[p + n["dq_norm"]], rt)
        if self.own_kv:
            self.dkv_gain = to_device_f32(tensors[p + n["dkv_norm"]], rt)
        self.uk = to_device_matrix(tensors[p + n["uk"]], rt)          # [heads * dim, kv_rank]
        self.uv = to_device_matrix(tensors[p + n["uv"]], rt)          # [heads * vdim, kv_rank]
        self.ukv = torch.cat([self.uk, self.uv], dim=0).contiguous() if self._per_head_form_fits(rt.dtype) else None

    # prompts of fewer tokens run the latent form: its kernels cost less than the per-head form's products and launches
    PER_HEAD_MIN_TOKENS = 256

    def _per_head_form_fits(self, dtype) -> bool:
        return (dtype == torch.bfloat16 and self.dim + self.rot_dim == self.vdim and self.vdim in (32, 64, 128)
                and self.heads <= 65535 and self.kv_rank % 8 == 0)

    def _whole_prompts(self, ctx: StepContext) -> bool:
        return (self.ukv is not None and ctx.host is not None and not ctx.all_single
                and ctx.n_tokens >= self.PER_HEAD_MIN_TOKENS and all(p == 0 for p in ctx.host["seq_past"]))

    def _step_pages(self, ctx: StepContext, device):
        """Pages of the step's own for per-head keys and values: a table ``[S, pages]`` (made once a step) that gives
        every sequence consecutive pages from 1 on (page 0 stands where a sequence has none), and how many there are."""
        made = ctx.scratch.get("latent_step_pages")
        if made is None:
            import numpy as np
            lens = ctx.host["seq_lens"]
            maxp = max((n + 63) // 64 for n in lens)
            table = np.zeros((len(lens), maxp), dtype=np.int32)
            nxt = 1
            for i, n in enumerate(lens):
                k = (n + 63) // 64
                table[i, :k] = np.arange(nxt, nxt + k)
                nxt += k
            made = ctx.scratch["latent_step_pages"] = (torch.from_numpy(table).to(device, non_blocking=True), nxt)
        return made

    def _forward_per_head(self, x, p, q, ctx: StepContext, cache_view: KVView, bt, inv_freq, rot_dims, pairs, mag):
        H, D, Dr, Dv = self.heads, self.dim, self.rot_dim, self.vdim
        c, kr = ops.latent_gather(cache_view.k, ctx, bt, self.kv_rank, Dr)
        kv = ops.linear(c, self.ukv)
        table, n_pages = self._step_pages(ctx, x.device)
        # zeros: the rows behind a sequence's end are masked, but a tensor-core product still multiplies them
        kp = torch.zeros((n_pages, H, 64, D + Dr), dtype=x.dtype, device=x.device)
        vp = torch.zeros((n_pages, H, 64, Dv), dtype=x.dtype, device=x.device)
        ops.latent_expand(kv, kr, ctx, table, H, D, Dr, Dv, kp, vp)
        q = ops.latent_rotate_q(q, H, D, Dr, inv_freq, rot_dims, pairs, ctx, mag)
        y = ops.attention(q, kp, vp, ctx, table, H, H, D + Dr, self.scale, self.window)
        if self.gated:
            ops.head_gate(y, p, self.col_g, H, Dv)
        return self.o.forward(y)

    def cache_request(self):
        if not self.own_kv:
            return None
        return KVRequest(1, self.kv_rank + self.rot_dim, self.keep_window, keys_only=True)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache_view: KVView, write_cache: bool = True):
        if write_cache != self.own_kv:
            raise ValueError("a latent attention layer writes the cache exactly when it has a key/value latent of its own")
        rot = self.position.rotation()
        inv_freq, rot_dims = rot if rot is not None else (None, 0)
        pairs = bool(getattr(self.position, "pairs", False))
        mag = float(getattr(self.position, "magnitude", 1.0))
        bt = ctx.block_tables[cache_view.group]
        p = self.proj.forward(x)
        cq = ops.latent_prepare(p, self.q_rank, self.col_dkv, self.kv_rank, self.rot_dim, self.dq_gain, self.dkv_gain,
                                self.norm_eps, inv_freq, rot_dims, pairs, ctx, bt, cache_view.k if write_cache else None, mag)
        q = self.uq.forward(cq) if self.q_rank else p          # the queries are the projection's first columns
        if self._whole_prompts(ctx):
            return self._forward_per_head(x, p, q, ctx, cache_view, bt, inv_freq, rot_dims, pairs, mag)
        qa = ops.latent_query(q, self.uk, self.heads, self.dim, self.rot_dim, self.kv_rank, inv_freq, rot_dims, pairs, ctx, mag)
        ol = ops.latent_attention(qa, cache_view.k, ctx, bt, self.heads, self.kv_rank, self.rot_dim, self.scale, self.window)
        y = ops.latent_output(ol, self.uv, self.heads, self.vdim, self.kv_rank, p, self.col_g, x.dtype)
        return self.o.forward(y)
