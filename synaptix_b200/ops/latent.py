"""Python faces of the kernels in ``csrc/latent.cu``: attention over a cached latent.  A token's cache row is
``[c | k_rot]`` (``kv_rank`` + ``rot_dim`` elements, one head); queries in the latent's space and weighted latents are
float32."""
from __future__ import annotations

from typing import Optional

import torch

from ._lib import KernelError, c_float, c_int, check, dt_code, fn, ptr, require_cuda, stream


def latent_prepare(proj: torch.Tensor, q_rank: int, col_kv: int, kv_rank: int, rot_dim: int, gain_q: Optional[torch.Tensor],
                   gain_kv: Optional[torch.Tensor], eps: float, inv_freq: Optional[torch.Tensor], rot_dims: int, pairs: bool,
                   ctx, block_table: torch.Tensor, k_pages: Optional[torch.Tensor], magnitude: float = 1.0) -> Optional[torch.Tensor]:
    """From the stacked input projection ``proj [T, row]``: the normed query latent ``rmsnorm(proj[:, :q_rank]) * gain_q``
    (returned, ``proj``'s dtype; ``q_rank = 0``: there is none and ``None`` is returned) and, if ``k_pages`` is given,
    the token's cache row: ``rmsnorm(proj[:, col_kv : col_kv + kv_rank]) * gain_kv`` and behind it the next ``rot_dim``
    columns with their first ``rot_dims`` elements rotated (``pairs``: neighbouring elements paired, else element ``i``
    with ``i + rot_dims / 2``; cos and sin times ``magnitude``)."""
    require_cuda(proj, gain_q, gain_kv, inv_freq, block_table, k_pages)
    T, row = proj.shape
    if k_pages is not None:
        if col_kv < 0 or col_kv + kv_rank + rot_dim > row or gain_kv is None:
            raise KernelError("latent_prepare: the key/value latent's columns do not fit")
        if k_pages.dtype != proj.dtype or k_pages.dim() != 4 or tuple(k_pages.shape[1:]) != (1, 64, kv_rank + rot_dim):
            raise KernelError("latent_prepare: cache pages must be [n_pages, 1, 64, kv_rank + rot_dim] of the compute dtype")
    if q_rank > row or (q_rank > 0 and (gain_q is None or gain_q.numel() != q_rank)):
        raise KernelError("latent_prepare: the query latent does not fit")
    if q_rank == 0 and k_pages is None:
        return None
    cq = torch.empty((T, q_rank), dtype=proj.dtype, device=proj.device) if q_rank > 0 else None
    check(fn("latent", "sx_latent_prepare")(
        ptr(proj), c_int(row), c_int(q_rank), c_int(col_kv if k_pages is not None else -1), c_int(kv_rank), c_int(rot_dim),
        ptr(gain_q), ptr(gain_kv), c_float(eps), ptr(inv_freq), c_int(rot_dims if inv_freq is not None else 0),
        c_int(1 if pairs else 0), c_float(magnitude), ptr(ctx.positions), ptr(ctx.seq_of_token), ptr(block_table),
        c_int(block_table.shape[1]), ptr(k_pages), ptr(cq), c_int(T), c_int(dt_code(proj.dtype)), stream()), "latent_prepare")
    return cq


def latent_query(q: torch.Tensor, wuk: torch.Tensor, heads: int, dim: int, rot_dim: int, kv_rank: int,
                 inv_freq: Optional[torch.Tensor], rot_dims: int, pairs: bool, ctx, magnitude: float = 1.0) -> torch.Tensor:
    """Queries (the first ``heads * (dim + rot_dim)`` columns of ``q``, which may be a wider stacked projection) taken into
    the latent's space: per head ``[Wuk_h^T q_h | rotate(q_rot_h)]`` with ``wuk [heads * dim, kv_rank]``; float32
    ``[T, heads, kv_rank + rot_dim]``."""
    require_cuda(q, wuk, inv_freq)
    T = q.shape[0]
    if q.shape[1] < heads * (dim + rot_dim) or tuple(wuk.shape) != (heads * dim, kv_rank) or wuk.dtype != q.dtype:
        raise KernelError("latent_query: sizes do not fit")
    qa = torch.empty((T, heads, kv_rank + rot_dim), dtype=torch.float32, device=q.device)
    check(fn("latent", "sx_latent_query")(ptr(q), c_int(q.shape[1]), ptr(wuk), c_int(heads), c_int(dim), c_int(rot_dim), c_int(kv_rank),
                                          ptr(inv_freq), c_int(rot_dims if inv_freq is not None else 0),
                                          c_int(1 if pairs else 0), c_float(magnitude), ptr(ctx.positions), ptr(qa), c_int(T),
                                          c_int(dt_code(q.dtype)), stream()), "latent_query")
    return qa


class WeightedLatents:
    """What ``latent_attention`` leaves: per (token, head) and part of the window the weighted sum of ``c`` without its
    division, ``parts`` float32 ``[T, heads, splits, kv_rank]``, and each part's maximum and sum of weights, ``ml``
    float32 ``[T, heads, splits, 2]``; ``latent_output`` merges them."""
    __slots__ = ("parts", "ml", "splits")

    def __init__(self, parts, ml, splits):
        self.parts, self.ml, self.splits = parts, ml, splits

    def merged(self) -> torch.Tensor:
        """float32 ``[T, heads, kv_rank]`` (for tests: torch arithmetic)."""
        m, l = self.ml[..., 0], self.ml[..., 1]
        w = torch.exp(m - m.max(dim=-1, keepdim=True).values)
        return (self.parts * w[..., None]).sum(2) / (l * w).sum(-1, keepdim=True)


_SMS = {}


def _pick_latent_splits(ctx, heads: int, window: Optional[int], device) -> int:
    """Parts of the window for single-token steps, so that the blocks fill the SMs about twice; prompts take one."""
    if not ctx.all_single:
        return 1
    keys = ctx.max_len if window is None else min(ctx.max_len, int(window))
    tiles = (keys + 31) // 32
    idx = device.index or 0
    if idx not in _SMS:
        _SMS[idx] = torch.cuda.get_device_properties(device).multi_processor_count
    blocks = ctx.n_tokens * ((heads + 7) // 8)
    want = (2 * _SMS[idx] + blocks - 1) // blocks
    return max(1, min(want, tiles // 2, 16))


def latent_attention(qa: torch.Tensor, k_pages: torch.Tensor, ctx, block_table: torch.Tensor, heads: int, kv_rank: int,
                     rot_dim: int, scale: float, window: Optional[int], splits: Optional[int] = None) -> WeightedLatents:
    """Causal (optionally windowed) softmax attention of ``qa`` float32 ``[T, heads, kv_rank + rot_dim]`` over the cache
    rows ``[c | k_rot]``; the weights are applied to ``c`` (see ``WeightedLatents``)."""
    require_cuda(qa, k_pages, block_table)
    T = qa.shape[0]
    if qa.dtype != torch.float32 or tuple(qa.shape[1:]) != (heads, kv_rank + rot_dim):
        raise KernelError("latent_attention: queries are float32 [T, heads, kv_rank + rot_dim]")
    if k_pages.dim() != 4 or tuple(k_pages.shape[1:]) != (1, 64, kv_rank + rot_dim):
        raise KernelError("latent_attention: cache pages must be [n_pages, 1, 64, kv_rank + rot_dim]")
    if splits is None:
        splits = _pick_latent_splits(ctx, heads, window, qa.device)
    out = torch.empty((T, heads, splits, kv_rank), dtype=torch.float32, device=qa.device)
    ml = torch.empty((T, heads, splits, 2), dtype=torch.float32, device=qa.device)
    check(fn("latent", "sx_latent_attention")(ptr(qa), ptr(k_pages), ptr(ctx.positions), ptr(ctx.seq_of_token), ptr(block_table),
                                              c_int(block_table.shape[1]), c_int(heads), c_int(kv_rank), c_int(rot_dim),
                                              c_float(scale), c_int(0 if window is None else int(window)), ptr(out), ptr(ml),
                                              c_int(splits), c_int(T), c_int(dt_code(k_pages.dtype)), stream()), "latent_attention")
    return WeightedLatents(out, ml, splits)


def latent_output(ol: WeightedLatents, wuv: torch.Tensor, heads: int, vdim: int, kv_rank: int, proj: torch.Tensor, col_gate: int,
                  out_dtype: torch.dtype) -> torch.Tensor:
    """``y[t, h * vdim + j] = sigmoid(proj[t, col_gate + h]) * sum_r wuv[h * vdim + j, r] * o[t, h, r]`` with ``o`` the
    merged, divided weighted latents (no gate if ``col_gate < 0``); ``[T, heads * vdim]`` in ``out_dtype``."""
    require_cuda(ol.parts, ol.ml, wuv, proj)
    T = ol.parts.shape[0]
    if tuple(ol.parts.shape[1:]) != (heads, ol.splits, kv_rank) or tuple(wuv.shape) != (heads * vdim, kv_rank):
        raise KernelError("latent_output: sizes do not fit")
    if wuv.dtype != out_dtype or proj.dtype != out_dtype or (col_gate >= 0 and col_gate + heads > proj.shape[1]):
        raise KernelError("latent_output: dtypes or the gate's columns do not fit")
    y = torch.empty((T, heads * vdim), dtype=out_dtype, device=wuv.device)
    check(fn("latent", "sx_latent_output")(ptr(ol.parts), ptr(ol.ml), c_int(ol.splits), ptr(wuv), c_int(heads), c_int(vdim),
                                           c_int(kv_rank), ptr(proj), c_int(proj.shape[1]), c_int(col_gate), ptr(y), c_int(T),
                                           c_int(dt_code(out_dtype)), stream()), "latent_output")
    return y


def latent_gather(k_pages: torch.Tensor, ctx, block_table: torch.Tensor, kv_rank: int, rot_dim: int):
    """The cache rows of the step's own tokens: ``c [T, kv_rank]`` and ``k_rot [T, rot_dim]`` in the cache's dtype."""
    require_cuda(k_pages, block_table)
    T = ctx.n_tokens
    c = torch.empty((T, kv_rank), dtype=k_pages.dtype, device=k_pages.device)
    kr = torch.empty((T, rot_dim), dtype=k_pages.dtype, device=k_pages.device)
    check(fn("latent", "sx_latent_gather")(ptr(k_pages), ptr(ctx.positions), ptr(ctx.seq_of_token), ptr(block_table),
                                           c_int(block_table.shape[1]), c_int(kv_rank), c_int(rot_dim), ptr(c), ptr(kr), c_int(T),
                                           c_int(dt_code(k_pages.dtype)), stream()), "latent_gather")
    return c, kr


def latent_expand(kv: torch.Tensor, kr: torch.Tensor, ctx, table: torch.Tensor, heads: int, dim: int, rot_dim: int, vdim: int,
                  k_out: torch.Tensor, v_out: torch.Tensor) -> None:
    """Per-head keys ``[k_h | k_rot]`` and values of the step's tokens into pages ``k_out [P, heads, 64, dim + rot_dim]``,
    ``v_out [P, heads, 64, vdim]`` by the page table ``table [S, pages]``; ``kv [T, heads * dim + heads * vdim]`` holds
    every head's unrotated key, then every head's value."""
    require_cuda(kv, kr, table, k_out, v_out)
    T = kv.shape[0]
    if (kv.shape[1] != heads * (dim + vdim) or tuple(k_out.shape[1:]) != (heads, 64, dim + rot_dim)
            or tuple(v_out.shape[1:]) != (heads, 64, vdim) or tuple(kr.shape) != (T, rot_dim)):
        raise KernelError("latent_expand: sizes do not fit")
    check(fn("latent", "sx_latent_expand")(ptr(kv), ptr(kr), ptr(ctx.positions), ptr(ctx.seq_of_token), ptr(table),
                                           c_int(table.shape[1]), c_int(heads), c_int(dim), c_int(rot_dim), c_int(vdim),
                                           ptr(k_out), ptr(v_out), c_int(T), c_int(dt_code(kv.dtype)), stream()), "latent_expand")


def latent_rotate_q(q: torch.Tensor, heads: int, dim: int, rot_dim: int, inv_freq: Optional[torch.Tensor], rot_dims: int,
                    pairs: bool, ctx, magnitude: float = 1.0) -> torch.Tensor:
    """The queries ``[T, heads * (dim + rot_dim)]`` with every head's rotated part rotated: in place when ``q`` has exactly
    those columns, else (``q`` a wider stacked projection that begins with them) into a new tensor."""
    require_cuda(q, inv_freq)
    n = heads * (dim + rot_dim)
    if q.shape[1] < n:
        raise KernelError("latent_rotate_q: the queries do not fit")
    no_rotation = inv_freq is None or rot_dims == 0
    if q.shape[1] == n and no_rotation:
        return q
    out = q if q.shape[1] == n else torch.empty((q.shape[0], n), dtype=q.dtype, device=q.device)
    check(fn("latent", "sx_latent_rotate_q")(ptr(q), c_int(q.shape[1]), ptr(out), ptr(ctx.positions), ptr(inv_freq),
                                             c_int(0 if no_rotation else rot_dims), c_int(1 if pairs else 0), c_float(magnitude),
                                             c_int(heads), c_int(dim), c_int(rot_dim), c_int(q.shape[0]), c_int(dt_code(q.dtype)),
                                             stream()), "latent_rotate_q")
    return out


def head_gate(y: torch.Tensor, proj: torch.Tensor, col: int, heads: int, vdim: int) -> None:
    """``y[t, h, :] *= sigmoid(proj[t, col + h])`` in place (``y [T, heads * vdim]``)."""
    require_cuda(y, proj)
    if y.dtype != proj.dtype or y.shape[1] != heads * vdim or col + heads > proj.shape[1]:
        raise KernelError("head_gate: sizes or dtypes do not fit")
    check(fn("latent", "sx_head_gate")(ptr(y), ptr(proj), c_int(proj.shape[1]), c_int(col), c_int(heads), c_int(vdim),
                                       c_int(y.shape[0]), c_int(dt_code(y.dtype)), stream()), "head_gate")
