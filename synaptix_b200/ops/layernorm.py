"""Python face of ``csrc/layernorm.cu``: the sum into the residual stream (optionally of a layer-normed branch, times
a factor), the layer norm of the result, and optionally a token shift of the normed rows, in one kernel."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ._lib import KernelError, c_float, c_int, check, dt_code, fn, ptr, require_cuda, stream


def add_layernorm(h: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, bias: torch.Tensor, eps: float,
                  out_dtype: torch.dtype, *, post: Optional[Tuple[torch.Tensor, torch.Tensor]] = None, mult: float = 1.0,
                  delta_bias: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
                  shift: Optional[torch.Tensor] = None, state: Optional[torch.Tensor] = None, ctx=None,
                  in_place: bool = True, write_back: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """``h' = h + mult * post(delta + delta_bias)`` (``post = (gain, bias)`` of a layer norm, ``None``: the identity;
    without ``delta`` nothing is added), ``y = layernorm(h') * weight + bias`` in ``out_dtype``.

    ``rows`` (int32): only those rows are computed and returned; nothing is written back.
    ``shift`` (float32 ``[width]``): the result is ``y_t + (y_(t-1) - y_t) * shift`` with ``y_(t-1)`` the row before in
    the token's sequence: the step's row before it or, for the first row a sequence brings, ``state[slot]``
    (``state`` float32 ``[slots, width]``), which then takes the sequence's last ``y``; ``ctx`` gives
    ``seq_of_token``, ``cu_seqlens`` and ``seq_slots``.  With a shift and ``in_place=False`` the sums go to a new
    tensor (needed whenever a sequence brings more than one row: a block reads its neighbour's row of ``h``).

    Returns ``(y, h')`` where ``h'`` is ``h`` itself when the sums were written in place."""
    require_cuda(h, delta, weight, bias, delta_bias, rows, shift, state)
    T, W = h.shape
    if h.dtype != torch.float32 or weight.dtype != torch.float32 or bias.dtype != torch.float32:
        raise KernelError("the residual stream, gains and biases of a norm are float32")
    if weight.numel() != W or bias.numel() != W:
        raise KernelError(f"a norm's gain and bias have one element per column ({W})")
    if delta is not None and delta.shape != h.shape:
        raise KernelError("delta must have the residual stream's shape")
    if post is not None:
        require_cuda(*post)
        if any(p.dtype != torch.float32 or p.numel() != W for p in post):
            raise KernelError("the branch's norm has float32 gain and bias over the width")
    if shift is not None:
        if rows is not None or state is None or ctx is None:
            raise KernelError("a token shift needs the state and the step's context, and takes all rows")
        if shift.dtype != torch.float32 or state.dtype != torch.float32 or state.shape[-1] != W:
            raise KernelError("shift and state are float32 over the width")
    R = T if rows is None else rows.numel()
    out = torch.empty((R, W), dtype=out_dtype, device=h.device)
    if rows is not None or not write_back:
        h_out = None
        h_after = h
    elif in_place:
        h_out = h_after = h
    else:
        h_out = h_after = torch.empty_like(h)
    check(fn("layernorm", "sx_add_layernorm")(
        ptr(h), ptr(h_out), ptr(delta), c_int(dt_code(delta.dtype) if delta is not None else 0), ptr(delta_bias),
        ptr(post[0] if post else None), ptr(post[1] if post else None), c_float(mult), ptr(weight), ptr(bias),
        c_float(eps), ptr(out), c_int(dt_code(out_dtype)), ptr(rows), c_int(R), c_int(W), ptr(shift), ptr(state),
        ptr(ctx.seq_of_token if shift is not None else None), ptr(ctx.cu_seqlens if shift is not None else None),
        ptr(ctx.seq_slots if shift is not None else None), stream()), "add_layernorm")
    return out, h_after
