"""Python faces of the kernels in ``csrc/normed.cu``: a branch that is RMS-normed on its way into the residual stream
(optionally the mean of two normed mixers), and the embedding with a hashed table of token pairs."""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from ._lib import KernelError, c_float, c_int, check, dt_code, fn, ptr, require_cuda, stream


class WeightedRows:
    """A branch that is a weighted sum of rows not formed yet: ``out[t] = sum_k weights[t, k] * rows[place[t * top + k]]``
    (``rows`` float32 ``[T * top, width]``, ``place`` int32 ``[T * top]``, ``weights`` float32 ``[T, top]``): what a mixture
    of experts holds before its last kernel.  ``add_normed`` takes it as its raw term and forms the sum on its way;
    ``materialize()`` runs the mixture's own kernel (``moe_combine``) and gives the tensor in ``dtype``."""
    __slots__ = ("rows", "place", "weights", "dtype", "_sum")

    def __init__(self, rows, place, weights, dtype):
        self.rows, self.place, self.weights, self.dtype = rows, place, weights, dtype
        self._sum = None

    @property
    def shape(self):
        return (self.weights.shape[0], self.rows.shape[1])

    def materialize(self) -> torch.Tensor:
        if self._sum is None:
            from .moe import moe_combine_rows
            self._sum = moe_combine_rows(self.rows, self.place, self.weights, self.dtype)
        return self._sum


def add_normed(h: Optional[torch.Tensor], terms: Sequence, post_gain: Optional[torch.Tensor], eps: float,
               out_dtype: Optional[torch.dtype], *, factor: float = 1.0, out_gain: Optional[torch.Tensor] = None,
               rows: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """One pass per row over a branch on its way into the residual stream ``h`` (float32 ``[T, width]``, summed into in
    place unless ``rows`` is given; ``None``: there is no stream and the result is the branch alone).

    ``terms``: none (nothing is added), one ``(x, None)`` (the branch is ``x``; ``x`` may be a ``WeightedRows``, the
    weighted sum of rows that a mixture of experts hands on), or one or two ``(x_i, gain_i)``: the
    branch is ``factor * sum_i rms_norm(x_i) * gain_i`` (mixers side by side, each with a norm of its own).  With
    ``post_gain`` the branch is normed once more, ``rms_norm(branch) * post_gain``, before it is added.  Returned: the
    rows after the sum in ``out_dtype`` (what the next sublayer reads), or ``rms_norm`` of them times ``out_gain``; all
    rows or ``rows`` (int32) only; ``out_dtype=None``: nothing is returned.  Norms and sums are 32-bit."""
    terms = list(terms)
    if len(terms) > 2 or (len(terms) == 2 and any(g is None for _, g in terms)):
        raise KernelError("add_normed: one raw term, or one or two terms with gains")
    (a, ga), (b, gb) = (terms + [(None, None), (None, None)])[:2]
    place = wts = None
    top = 0
    if isinstance(a, WeightedRows):
        if ga is not None or b is not None:
            raise KernelError("add_normed: a weighted sum of rows is a raw term and stands alone")
        place, wts, top, a_shape = a.place, a.weights, a.weights.shape[1], a.shape
        a = a.rows
        if a.dtype != torch.float32:
            raise KernelError("add_normed: the rows of a weighted sum are float32")
    else:
        a_shape = None if a is None else tuple(a.shape)
    require_cuda(h, a, ga, b, gb, post_gain, out_gain, rows, place, wts)
    if h is None and a is None:
        raise KernelError("add_normed: neither a stream nor a branch")
    T, H = h.shape if h is not None else a_shape
    if a_shape is not None and tuple(a_shape) != (T, H):
        raise KernelError("add_normed: a branch must have the stream's shape")
    ref = h if h is not None else a
    if b is not None and tuple(b.shape) != (T, H):
        raise KernelError("add_normed: a branch must have the stream's shape")
    for g in (ga, gb, post_gain, out_gain):
        if g is not None and (g.dtype != torch.float32 or g.numel() != H):
            raise KernelError("add_normed: gains are float32 vectors over the width")
    if h is not None and h.dtype != torch.float32:
        raise KernelError("add_normed: the residual stream is float32")
    R = T if rows is None else rows.numel()
    y = torch.empty((R, H), dtype=out_dtype, device=ref.device) if out_dtype is not None else None
    check(fn("normed", "sx_add_normed")(
        ptr(h), ptr(a), c_int(dt_code(a.dtype) if a is not None else 0), ptr(ga), ptr(b),
        c_int(dt_code(b.dtype) if b is not None else 0), ptr(gb), c_float(factor), ptr(post_gain), ptr(out_gain), c_float(eps),
        ptr(y), c_int(dt_code(out_dtype) if out_dtype is not None else 0), ptr(rows), c_int(R), c_int(H),
        c_int(1 if (rows is None and h is not None) else 0), ptr(place), ptr(wts), c_int(top), stream()), "add_normed")
    return y


def embed_bigram(table: torch.Tensor, bigram: torch.Tensor, ctx, last_token: torch.Tensor, mul_prev: int, mul_cur: int) -> torch.Tensor:
    """``out[t] = table[id_t] + bigram[(prev_t * mul_prev + id_t * mul_cur) mod buckets]`` as float32 ``[T, width]``, with
    ``bigram [buckets + 1, width]`` and its last row for a sequence's first token.  ``prev_t`` is the token before in the
    step or, for a portion's first token, ``last_token[slot]`` (int32 ``[slots]``), which is moved on to the portion's
    last token."""
    require_cuda(table, bigram, last_token)
    V, H = table.shape
    if bigram.dtype != table.dtype or bigram.shape[1] != H or bigram.shape[0] < 2 or last_token.dtype != torch.int32:
        raise KernelError("embed_bigram: the tables or the state do not fit")
    T = ctx.token_ids.numel()
    out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    check(fn("normed", "sx_embed_bigram")(ptr(table), ptr(bigram), c_int(dt_code(table.dtype)), ptr(ctx.token_ids),
                                          ptr(ctx.positions), ptr(ctx.seq_of_token), ptr(ctx.cu_seqlens), ptr(ctx.seq_slots),
                                          ptr(last_token), ptr(out), c_int(T), c_int(H), c_int(V), c_int(bigram.shape[0] - 1),
                                          c_int(mul_prev), c_int(mul_cur), stream()), "embed_bigram")
    return out
