"""Python faces of the kernels in ``csrc/sequence.cu``: the short convolution over time in front of a sublayer, the
minGRU recurrence, retention (linear attention with a fixed decay per head), the capped gated activation and sums
into the residual stream.  Float32 and bfloat16; states, norms, gates and sums are 32-bit in both."""
from __future__ import annotations

from typing import Optional

import torch

from ._lib import KernelError, c_float, c_int, check, dt_code, fn, ptr, require_cuda, stream


def _f32(*tensors) -> None:
    for t in tensors:
        if t is not None and t.dtype != torch.float32:
            raise KernelError("states, gains, biases and the residual stream are float32")


def add_rmsnorm_conv(h: torch.Tensor, delta: Optional[torch.Tensor], gain: torch.Tensor, eps: float,
                     conv_w: torch.Tensor, hist: torch.Tensor, ctx, out_dtype: torch.dtype) -> torch.Tensor:
    """``h += delta`` (in place), ``y = rmsnorm(h) * gain``, and the result ``y + conv(y)`` in ``out_dtype``, where
    ``conv(y)_t = sum_j conv_w[:, j] * y_(t - taps + 1 + j)`` runs over each sequence's own positions.

    ``conv_w`` float32 ``[width, taps]``; ``hist`` float32 ``[slots, taps - 1, width]`` holds each sequence's last
    ``taps - 1`` inputs ``y`` (oldest first, zero in a fresh slot) and is moved on.  Steps of one token a sequence run
    as one kernel; others as two (norm into a 32-bit buffer that also takes a copy of the history, then the
    convolution, which writes the new history)."""
    require_cuda(h, delta, gain, conv_w, hist)
    _f32(h, gain, conv_w, hist)
    T, H = h.shape
    taps = conv_w.shape[1]
    P = taps - 1
    if conv_w.shape[0] != H or gain.numel() != H or tuple(hist.shape[1:]) != (P, H):
        raise KernelError("add_rmsnorm_conv: sizes of the gain, the taps and the history do not fit the width")
    if delta is not None and delta.shape != h.shape:
        raise KernelError("add_rmsnorm_conv: delta must have the residual's shape")
    out = torch.empty((T, H), dtype=out_dtype, device=h.device)
    if ctx.all_single and ctx.n_seqs == T and (delta is None or delta.dtype == out_dtype) and H <= 8192:
        check(fn("sequence", "sx_norm_conv_step")(ptr(h), ptr(delta), ptr(gain), c_float(eps), ptr(conv_w), ptr(out),
                                                  ptr(hist), ptr(ctx.seq_slots), c_int(T), c_int(P), c_int(H),
                                                  c_int(dt_code(out_dtype)), stream()), "norm_conv_step")
        return out
    S = ctx.n_seqs
    y = torch.empty((T + S * P, H), dtype=torch.float32, device=h.device)
    check(fn("sequence", "sx_add_rmsnorm_hist")(ptr(h), ptr(delta), c_int(dt_code(delta.dtype) if delta is not None else 0),
                                                ptr(gain), c_float(eps), ptr(y), ptr(hist), ptr(ctx.seq_slots), c_int(T),
                                                c_int(S), c_int(P), c_int(H), stream()), "add_rmsnorm_hist")
    check(fn("sequence", "sx_token_conv")(ptr(y), ptr(conv_w), ptr(out), c_int(dt_code(out_dtype)), ptr(hist),
                                          ptr(ctx.positions), ptr(ctx.seq_of_token), ptr(ctx.cu_seqlens), ptr(ctx.seq_past),
                                          ptr(ctx.seq_lens), ptr(ctx.seq_slots), c_int(T), c_int(P), c_int(H), stream()),
          "token_conv")
    return out


_PIECE = [0]

# portions of at least this many tokens (the longest of a step) run retention in pieces
PIECES_MIN_TOKENS = 48


def mingru(proj: torch.Tensor, z_off: int, x_off: int, g_off: int, n: int, bias_z: Optional[torch.Tensor],
           bias_x: Optional[torch.Tensor], state: torch.Tensor, ctx) -> torch.Tensor:
    """The minGRU recurrence over the step's tokens.  ``proj [T, row]`` holds, for channel ``c < n``, the gate's
    pre-activation in column ``z_off + c``, the candidate's in ``x_off + c`` and the output gate's in ``g_off + c``;
    ``state`` float32 ``[slots, n]`` is moved on; returns ``S_t * silu(g_t)`` ``[T, n]`` in ``proj``'s dtype."""
    require_cuda(proj, bias_z, bias_x, state)
    _f32(bias_z, bias_x, state)
    T, row = proj.shape
    if state.shape[1] != n or max(z_off, x_off, g_off) + n > row:
        raise KernelError("mingru: the state or the columns do not fit")
    out = torch.empty((T, n), dtype=proj.dtype, device=proj.device)
    if _PIECE[0] == 0:
        _PIECE[0] = int(fn("sequence", "sx_mingru_piece_tokens")())
    scratch = None
    if ctx.max_new > 2 * _PIECE[0]:
        pieces = (ctx.max_new + _PIECE[0] - 1) // _PIECE[0]
        scratch = torch.empty((ctx.n_seqs, pieces, 2, n), dtype=torch.float32, device=proj.device)
    check(fn("sequence", "sx_mingru")(ptr(proj), c_int(row), c_int(z_off), c_int(x_off), c_int(g_off), ptr(bias_z), ptr(bias_x),
                                      ptr(state), ptr(out), ptr(scratch), ptr(ctx.cu_seqlens), ptr(ctx.seq_slots),
                                      c_int(ctx.n_seqs), c_int(n), c_int(ctx.max_new), c_int(dt_code(proj.dtype)), stream()),
          "mingru", launches=3 if scratch is not None else 1)
    return out


def retention(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, g_off: Optional[int], heads: int, dim: int, vdim: int,
              decay: torch.Tensor, k_scale: float, eps: float, unit_norm: bool, state: torch.Tensor, ctx,
              out: Optional[torch.Tensor] = None, out_col: int = 0, out_scale: float = 1.0) -> torch.Tensor:
    """Linear attention with a fixed decay per head over the step's tokens: ``S <- decay S + (k k_scale) v^T``,
    ``o = S^T q``; with ``unit_norm`` each head's ``o`` is divided by its root mean square; with ``g_off`` it is
    multiplied by ``silu`` of the gate's columns.  ``proj [T, row]`` holds q, k (``heads * dim`` columns each from
    ``q_off``, ``k_off``), v and the gate (``heads * vdim`` from ``v_off``, ``g_off``).  ``state`` float32
    ``[slots, heads, dim, vdim]`` is moved on.  The result, times ``out_scale``, goes to columns
    ``out_col .. out_col + heads * vdim`` of ``out`` (default: a new ``[T, heads * vdim]``)."""
    require_cuda(proj, decay, state)
    _f32(decay, state)
    T, row = proj.shape
    if tuple(state.shape[1:]) != (heads, dim, vdim) or decay.numel() != heads:
        raise KernelError("retention: the state or the decays do not fit the heads")
    if out is None:
        out = torch.empty((T, heads * vdim), dtype=proj.dtype, device=proj.device)
    if out.dtype != proj.dtype or out_col + heads * vdim > out.shape[1] or not out.is_contiguous():
        raise KernelError("retention: the output does not fit")
    o = out if out_col == 0 else out.view(-1)[out_col:]
    # single tokens: the state goes through registers; long portions: pieces of 64 tokens (three kernels); else a block
    # a (sequence, head) walks the tokens
    mode, scratch, launches = 0, None, 1
    if ctx.all_single and ctx.n_seqs == T and 2 * dim + max(256, 2 * vdim) <= 12 * 1024:
        mode = 1
    elif ctx.max_new >= PIECES_MIN_TOKENS and fn("sequence", "sx_retention_pieces_fit")(c_int(dim), c_int(vdim)):
        mode, launches = 2, 3
        pieces = (ctx.max_new + 63) // 64
        scratch = torch.empty((ctx.n_seqs, pieces, heads, dim * vdim), dtype=torch.float32, device=proj.device)
    check(fn("sequence", "sx_retention_any")(ptr(proj), c_int(row), c_int(q_off), c_int(k_off), c_int(v_off),
                                             c_int(-1 if g_off is None else g_off), ptr(decay), c_float(k_scale), c_float(eps),
                                             c_int(1 if unit_norm else 0), c_float(out_scale), ptr(state),
                                             ptr(o), c_int(out.shape[1]), ptr(scratch), ptr(ctx.cu_seqlens), ptr(ctx.seq_slots),
                                             c_int(ctx.n_seqs), c_int(heads), c_int(dim), c_int(vdim), c_int(ctx.max_new),
                                             c_int(mode), c_int(dt_code(proj.dtype)), stream()), "retention", launches=launches)
    return out


def capped_glu(gu: torch.Tensor, alpha: float, limit: float, form: int = 0) -> torch.Tensor:
    """``g sigmoid(alpha g) (u + 1)`` with ``g = min(gu[:, :I], limit)``, ``u = clamp(gu[:, I:], -limit, limit)``; with
    ``form = 1``: ``gelu_tanh(gu[:, :I]) * gu[:, I:]`` (the tanh form of GELU)."""
    require_cuda(gu)
    T, I2 = gu.shape
    out = torch.empty((T, I2 // 2), dtype=gu.dtype, device=gu.device)
    check(fn("sequence", "sx_capped_glu")(ptr(gu), ptr(out), c_int(T), c_int(I2 // 2), c_float(alpha), c_float(limit),
                                          c_int(form), c_int(dt_code(gu.dtype)), stream()), "capped_glu")
    return out


def stream_add(h: torch.Tensor, delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
               vec: Optional[torch.Tensor] = None) -> None:
    """``h += delta + rows + vec`` in place: ``h`` float32 ``[T, width]``; ``delta [T, width]`` in either dtype,
    ``rows`` float32 ``[T, width]``, ``vec`` float32 ``[width]``; each may be absent."""
    require_cuda(h, delta, rows, vec)
    _f32(h, rows, vec)
    T, H = h.shape
    for t in (delta, rows):
        if t is not None and t.shape != h.shape:
            raise KernelError("stream_add: shapes differ")
    if vec is not None and vec.numel() != H:
        raise KernelError("stream_add: the vector does not fit the width")
    check(fn("sequence", "sx_stream_add")(ptr(h), ptr(delta), c_int(dt_code(delta.dtype) if delta is not None else 0), ptr(rows),
                                          ptr(vec), c_int(T), c_int(H), stream()), "stream_add")
