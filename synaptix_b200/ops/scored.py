"""Python faces of ``csrc/attn_scored.cu``: head preparation from a float32 projection (bias, shared-gain RMS norm,
rotation of neighbouring pairs, blend of the values with another layer's, cache write, head gates) and the attention
whose weights may be a mixture of all heads' scores (sigmoid or softmax weights, biases per head and per distance)."""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from ._lib import KernelError, c_float, c_int, check, dt_code, fn, ptr, require_cuda, stream
from .options import OPTIONS


def heads_prepare(proj: torch.Tensor, bias: Optional[torch.Tensor], q_out: torch.Tensor, k_pages: Optional[torch.Tensor],
                  v_pages: Optional[torch.Tensor], positions: torch.Tensor, seq_of_token: torch.Tensor,
                  block_table: torch.Tensor, H: int, G: int, dim: int, vdim: int, *, q_gain=None, k_gain=None,
                  eps: float = 0.0, inv_freq=None, rot_dims: int = 0, magnitude: float = 1.0, v_first_in=None,
                  v_first_out=None, lam=None, gate_out=None) -> None:
    """``proj`` float32 ``[T, >= (H + G) dim + G vdim + gates]``: q heads, k heads, v heads, then one gate column per
    entry of ``gate_out``'s row.  See the kernel's comment for what is done to each."""
    require_cuda(proj, bias, q_out, k_pages, v_pages, positions, seq_of_token, block_table, q_gain, k_gain, inv_freq,
                 v_first_in, v_first_out, lam, gate_out)
    if proj.dtype != torch.float32:
        raise KernelError("heads_prepare takes the projection in float32")
    T = proj.shape[0]
    n_gate = 0 if gate_out is None else gate_out.shape[1]
    n_pages = 0
    for pg, d in ((k_pages, dim), (v_pages, vdim)):
        if pg is None:
            continue
        if pg.dtype != q_out.dtype or pg.dim() != 4 or tuple(pg.shape[1:]) != (G, 64, d):
            raise KernelError("heads_prepare: cache pages must be [n_pages, kv heads, 64, head size] in the queries' dtype")
        n_pages = pg.shape[0]
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != (H + G) * dim + G * vdim + n_gate):
        raise KernelError("heads_prepare: the bias covers every column of the projection")
    for x in (v_first_in, v_first_out):
        if x is not None and (x.dtype != torch.float32 or tuple(x.shape) != (T, G * vdim)):
            raise KernelError("heads_prepare: shared values are float32 [T, kv heads * value size]")
    check(fn("attn_scored", "sx_heads_prepare")(
        ptr(proj), c_int(proj.shape[1]), ptr(bias), ptr(q_out), ptr(k_pages), ptr(v_pages), ptr(positions),
        ptr(seq_of_token), ptr(block_table), c_int(block_table.shape[1]), c_int(n_pages), c_int(T), c_int(H), c_int(G),
        c_int(dim), c_int(vdim), ptr(q_gain), ptr(k_gain), c_float(eps), ptr(inv_freq), c_int(rot_dims if inv_freq is not None else 0),
        c_float(magnitude), ptr(v_first_in), ptr(v_first_out), ptr(lam), ptr(gate_out), c_int(n_gate),
        c_int(dt_code(q_out.dtype)), stream()), "heads_prepare")


SCORED_TILE_ROWS = 4
TALK_TILE_ROWS = 8          # rows a block of the tensor-core kernel for sigmoid weights takes
TALK_MAX_SMEM = 220 * 1024

_TALK_SMEM = {}


def talk_prefill_applies(H: int, G: int, dim: int, vdim: int, dtype, softmax: bool, dist_bias) -> bool:
    """Whether prompt portions of this attention run on the tensor-core kernel: sigmoid weights, no distance table,
    bfloat16, a shape it is built for, and a block's shared memory within the SM's."""
    if softmax or dist_bias is not None or dtype != torch.bfloat16 or not OPTIONS.attn_scored_tc:
        return False
    key = (H, G, dim, vdim)
    need = _TALK_SMEM.get(key)
    if need is None:
        f = fn("attn_scored", "sx_attn_talk_prefill_smem")
        need = _TALK_SMEM[key] = int(f(c_int(H), c_int(G), c_int(dim), c_int(vdim)))
    return 0 <= need <= TALK_MAX_SMEM


def _tiles(ctx, rows: int, device):
    tiles = ctx.scratch.get(("scored_tiles", rows))
    if tiles is None:
        a, b = scored_tiles(ctx.host["cu_seqlens"], rows)
        both = torch.from_numpy(np.asarray([a, b], dtype=np.int32)).to(device, non_blocking=True)
        tiles = ctx.scratch[("scored_tiles", rows)] = (both[0], both[1])
    return tiles


def scored_tiles(cu_seqlens, rows: int = SCORED_TILE_ROWS):
    """Tiles of up to ``rows`` consecutive rows of one sequence: (first packed row, number of rows) per tile."""
    tok0, n = [], []
    for s in range(len(cu_seqlens) - 1):
        for t in range(cu_seqlens[s], cu_seqlens[s + 1], rows):
            tok0.append(t)
            n.append(min(rows, cu_seqlens[s + 1] - t))
    return tok0, n


def _chunks(n_tokens: int, max_len: int, window: Optional[int], device) -> int:
    """Into how many parts a single token's keys are cut so that a few sequences fill the GPU."""
    keys = max_len if not window else min(max_len, window)
    tiles = max(1, (keys + 31) // 32 + 1)
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    want = max(1, (2 * sms) // max(1, n_tokens))
    return max(1, min(want, tiles, 64))


def attn_scored(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, ctx, block_table: torch.Tensor, H: int,
                G: int, dim: int, vdim: int, scale: float, window: Optional[int], *, talk=None, head_bias=None,
                dist_bias=None, softmax: bool = False, gate=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """See ``csrc/attn_scored.cu``.  ``q`` ``[T, H * dim]``; ``talk`` float32 ``[H, H]``; ``head_bias`` float32 ``[H]``;
    ``dist_bias`` float32 ``[H, n]`` (distance ``d`` reads column ``min(d, n - 1)``); ``gate`` float32 ``[T, H]``."""
    require_cuda(q, k_pages, v_pages, block_table, talk, head_bias, dist_bias, gate, out)
    T = q.shape[0]
    if out is None:
        out = torch.empty((T, H * vdim), dtype=q.dtype, device=q.device)
    if k_pages.dtype != q.dtype or v_pages.dtype != q.dtype or out.dtype != q.dtype:
        raise KernelError("attn_scored: queries, cache and output share a dtype")
    for x, shape in ((talk, (H, H)), (head_bias, (H,)), (gate, (T, H))):
        if x is not None and (x.dtype != torch.float32 or tuple(x.shape) != shape):
            raise KernelError(f"attn_scored: expected float32 {shape}")
    if dist_bias is not None and (dist_bias.dtype != torch.float32 or dist_bias.dim() != 2 or dist_bias.shape[0] != H):
        raise KernelError("attn_scored: the distance bias is float32 [H, n]")
    tok0 = rows = part = part_ml = None
    n_tiles, tq, n_chunks = T, 1, 1
    if (ctx.all_single or ctx.host is None) and talk_prefill_applies(H, G, dim, vdim, q.dtype, softmax, dist_bias):
        # single tokens on the tensor-core kernel: a block a (token, part of its keys), 16 keys a turn
        keys = ctx.max_len if not window else min(ctx.max_len, window)
        sms = torch.cuda.get_device_properties(q.device).multi_processor_count
        n_chunks = max(1, min((2 * sms) // max(1, T), (keys + 15) // 16 + 1, 64))
        part = torch.empty((T, n_chunks, H, vdim), dtype=torch.float32, device=q.device) if n_chunks > 1 else None
        check(fn("attn_scored", "sx_attn_talk_prefill")(
            ptr(q), ptr(k_pages), ptr(v_pages), ptr(out), ptr(ctx.positions), ptr(ctx.seq_of_token), ptr(block_table),
            c_int(block_table.shape[1]), ptr(None), ptr(None), c_int(T), c_int(H), c_int(G), c_int(dim), c_int(vdim),
            c_float(scale), c_int(0 if not window else int(window)), ptr(talk), ptr(head_bias), ptr(gate),
            c_int(out.shape[1]), ptr(part), c_int(n_chunks), stream()), "attn_talk_prefill", launches=2 if n_chunks > 1 else 1)
        return out
    if ctx.all_single or ctx.host is None:
        n_chunks = _chunks(T, ctx.max_len, window, q.device)
        if n_chunks > 1:
            part = torch.empty((T, n_chunks, H, vdim), dtype=torch.float32, device=q.device)
            part_ml = torch.empty((T, n_chunks, H, 2), dtype=torch.float32, device=q.device) if softmax else None
    elif ctx.max_new >= TALK_TILE_ROWS and talk_prefill_applies(H, G, dim, vdim, q.dtype, softmax, dist_bias):
        tok0, rows = _tiles(ctx, TALK_TILE_ROWS, q.device)
        check(fn("attn_scored", "sx_attn_talk_prefill")(
            ptr(q), ptr(k_pages), ptr(v_pages), ptr(out), ptr(ctx.positions), ptr(ctx.seq_of_token), ptr(block_table),
            c_int(block_table.shape[1]), ptr(tok0), ptr(rows), c_int(tok0.numel()), c_int(H), c_int(G), c_int(dim),
            c_int(vdim), c_float(scale), c_int(0 if not window else int(window)), ptr(talk), ptr(head_bias), ptr(gate),
            c_int(out.shape[1]), ptr(None), c_int(1), stream()), "attn_talk_prefill")
        return out
    elif ctx.max_new >= SCORED_TILE_ROWS:
        tok0, rows = _tiles(ctx, SCORED_TILE_ROWS, q.device)
        n_tiles, tq = tok0.numel(), SCORED_TILE_ROWS
    check(fn("attn_scored", "sx_attn_scored")(
        ptr(q), ptr(k_pages), ptr(v_pages), ptr(out), ptr(part), ptr(part_ml), ptr(ctx.positions), ptr(ctx.seq_of_token),
        ptr(block_table), c_int(block_table.shape[1]), ptr(tok0), ptr(rows), c_int(n_tiles), c_int(tq), c_int(T), c_int(H),
        c_int(G), c_int(dim), c_int(vdim), c_float(scale), c_int(0 if not window else int(window)), ptr(talk),
        ptr(head_bias), ptr(dist_bias), c_int(0 if dist_bias is None else dist_bias.shape[1]), c_int(1 if softmax else 0),
        c_int(n_chunks), c_int(out.shape[1]), ptr(gate), c_int(dt_code(q.dtype)), stream()),
        "attn_scored", launches=2 if n_chunks > 1 else 1)
    return out
