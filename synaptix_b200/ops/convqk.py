"""Python faces of the kernels in ``csrc/convqk.cu``: head preparation with a short convolution over time on queries
and keys, a norm over the whole projection and values that are the convolved keys; an output gate per element."""
from __future__ import annotations

from typing import Optional

import torch

from ._lib import KernelError, c_float, c_int, check, dt_code, fn, ptr, require_cuda, stream


def convqk_prepare(proj: torch.Tensor, col_q: int, col_k: int, heads: int, kv_heads: int, dim: int, taps_q: torch.Tensor,
                   taps_k: torch.Tensor, gain_q: torch.Tensor, gain_k: torch.Tensor, eps: float, hist: torch.Tensor, ctx,
                   block_table: torch.Tensor, k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor]) -> torch.Tensor:
    """From ``proj [T, row]`` (q in ``heads * dim`` columns from ``col_q``, k in ``kv_heads * dim`` from ``col_k``):
    both convolved over each sequence's own positions with ``taps_*`` (float32, taps-major: ``[n, channels]``, the
    transpose of the stored ``[channels, n]``; ``hist`` float32
    ``[slots, n - 1, Cq + Ck]`` holds every sequence's last ``n - 1`` projected rows and is moved on); the convolved
    keys are the values; queries and keys are RMS-normed over ALL their channels times ``gain_*``.  Returns the
    queries ``[T, heads * dim]``; keys and values go into the cache pages (``None``: nothing is cached)."""
    require_cuda(proj, taps_q, taps_k, gain_q, gain_k, hist, block_table, k_pages, v_pages)
    T, row = proj.shape
    Cq, Ck = heads * dim, kv_heads * dim
    taps = taps_q.shape[0]
    for t in (taps_q, taps_k, gain_q, gain_k, hist):
        if t.dtype != torch.float32:
            raise KernelError("convqk_prepare: taps, gains and the history are float32")
    if (tuple(taps_q.shape) != (taps, Cq) or tuple(taps_k.shape) != (taps, Ck) or gain_q.numel() != Cq or gain_k.numel() != Ck
            or tuple(hist.shape[1:]) != (taps - 1, Cq + Ck)):
        raise KernelError("convqk_prepare: the taps, gains or history do not fit the heads")
    if k_pages is not None and (v_pages is None or k_pages.dtype != proj.dtype or tuple(k_pages.shape[1:]) != (kv_heads, 64, dim)
                                or k_pages.shape != v_pages.shape):
        raise KernelError("convqk_prepare: cache pages must be [n_pages, kv_heads, 64, dim] of the compute dtype")
    q = torch.empty((T, Cq), dtype=proj.dtype, device=proj.device)
    single = bool(ctx.all_single and ctx.n_seqs == T)
    check(fn("convqk", "sx_convqk_prepare")(
        ptr(proj), c_int(row), c_int(col_q), c_int(col_k), c_int(Cq), c_int(Ck), c_int(taps), ptr(taps_q), ptr(taps_k),
        ptr(gain_q), ptr(gain_k), c_float(eps), ptr(hist), ptr(ctx.positions), ptr(ctx.seq_of_token), ptr(ctx.cu_seqlens),
        ptr(ctx.seq_past), ptr(ctx.seq_slots), ptr(block_table), c_int(block_table.shape[1]), ptr(q), ptr(k_pages), ptr(v_pages),
        c_int(kv_heads), c_int(dim), c_int(T), c_int(ctx.n_seqs), c_int(1 if single else 0), c_int(dt_code(proj.dtype)),
        stream()), "convqk_prepare", launches=1 if (single or taps == 1) else 2)
    return q


def sigmoid_gate(y: torch.Tensor, proj: torch.Tensor, col: int) -> None:
    """``y[t, c] *= sigmoid(proj[t, col + c])`` in place."""
    require_cuda(y, proj)
    if y.dtype != proj.dtype or y.shape[0] != proj.shape[0] or col + y.shape[1] > proj.shape[1]:
        raise KernelError("sigmoid_gate: sizes or dtypes do not fit")
    check(fn("convqk", "sx_sigmoid_gate")(ptr(y), ptr(proj), c_int(proj.shape[1]), c_int(col), c_int(y.shape[1]), c_int(y.shape[0]),
                                          c_int(dt_code(y.dtype)), stream()), "sigmoid_gate")
