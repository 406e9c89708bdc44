"""Python faces of the kernels in ``csrc/moe.cu``: router, sort by expert, grouped products, weighted sum."""
from __future__ import annotations

from typing import NamedTuple, Optional, Tuple

import torch

import ctypes

from ._lib import KernelError, c_float, c_int, check, dt_code, fn, ptr, require_cuda, stream, use_gate

# From this many (token, choice) rows on, bfloat16 products run the tcgen05 kernel (128-row tiles, rows gathered into
# sorted order first); fewer rows (single-token steps, short prompts) run the mma.sync kernel, which gathers as it loads.
TC_MIN_ROWS = 512


def _tc_fits(rows: int, K: int, dtype) -> bool:
    return dtype == torch.bfloat16 and rows >= TC_MIN_ROWS and K % 8 == 0


def moe_tc_status(reset: bool = False) -> int:
    """0, or which bounded wait of the tcgen05 grouped product ran out (1 producer, 2 MMA issuer, 3 epilogue)."""
    v = ctypes.c_int(0)
    check(fn("moe_tc", "sx_moe_tc_status")(ctypes.byref(v), c_int(1 if reset else 0)), "moe_tc_status", launches=0)
    return int(v.value)


class ExpertPlan(NamedTuple):
    """The step's (token, choice) pairs sorted by expert, all on the device: ``offsets [experts + 1]`` (first sorted place
    of each expert), ``order [pairs]`` (sorted place -> pair ``token * top + choice``), ``place [pairs]`` (the inverse)."""
    offsets: torch.Tensor
    order: torch.Tensor
    place: torch.Tensor
    experts: int


def moe_route(x: torch.Tensor, router: torch.Tensor, top: int, scale: float, sum_eps: float, *, scoring: str = "softmax",
              correction: Optional[torch.Tensor] = None, groups: Optional[Tuple[int, int]] = None, renormalize: bool = True):
    """Router logits ``x @ router.T`` in 32-bit (``router`` float32 ``[experts, width]``), scores = their softmax over all
    experts (``scoring="sigmoid"``: the sigmoid of each), the ``top`` largest chosen (of equal values the lower index):
    ``ids`` int32 ``[T, top]`` and ``weights`` float32 ``[T, top]`` = chosen score / (sum of the chosen + ``sum_eps``) *
    ``scale`` (``renormalize=False``: chosen score * ``scale``).

    ``correction`` float32 ``[experts]`` is added to the scores for the choice only.  ``groups = (count, keep)``: the
    experts form ``count`` equal groups of neighbours, a group's value is the sum of its two largest choice values, and
    only experts of the ``keep`` best groups can be chosen."""
    require_cuda(x, router, correction)
    T, W = x.shape
    E = router.shape[0]
    if router.dtype != torch.float32 or router.shape[1] != W:
        raise KernelError("moe_route: the router is float32 [experts, width]")
    if scoring not in ("softmax", "sigmoid"):
        raise KernelError("moe_route: scoring is softmax or sigmoid")
    if correction is not None and (correction.dtype != torch.float32 or correction.numel() != E):
        raise KernelError("moe_route: the correction is float32, one number per expert")
    count, keep = groups if groups is not None else (0, 0)
    ids = torch.empty((T, top), dtype=torch.int32, device=x.device)
    weights = torch.empty((T, top), dtype=torch.float32, device=x.device)
    check(fn("moe", "sx_moe_route")(ptr(x), ptr(router), c_int(T), c_int(W), c_int(E), c_int(top), c_float(scale),
                                    c_float(sum_eps), ptr(ids), ptr(weights), c_int(1 if scoring == "sigmoid" else 0),
                                    ptr(correction), c_int(count), c_int(keep), c_int(1 if renormalize else 0),
                                    c_int(dt_code(x.dtype)), stream()), "moe_route")
    return ids, weights


def moe_sort(ids: torch.Tensor, experts: int) -> ExpertPlan:
    require_cuda(ids)
    n = ids.numel()
    offsets = torch.empty(experts + 1, dtype=torch.int32, device=ids.device)
    order = torch.empty(n, dtype=torch.int32, device=ids.device)
    place = torch.empty(n, dtype=torch.int32, device=ids.device)
    check(fn("moe", "sx_moe_sort")(ptr(ids), c_int(n), c_int(experts), ptr(offsets), ptr(order), ptr(place), stream()), "moe_sort")
    return ExpertPlan(offsets, order, place, experts)


def moe_gate_up(x: torch.Tensor, gate_up: torch.Tensor, plan: ExpertPlan, top: int) -> torch.Tensor:
    """``silu(x_t Wg_e^T) * (x_t Wu_e^T)`` for every pair in sorted order (inside ``gate_activation(...)`` the gated
    activation in force there instead): ``gate_up [experts, 2 * ff, width]`` holds each expert's gate rows, then its up
    rows; returns ``[pairs, ff]`` in ``x``'s dtype."""
    require_cuda(x, gate_up)
    T, W = x.shape
    E, ff2, W2 = gate_up.shape
    if W2 != W or E != plan.experts or ff2 % 2 or gate_up.dtype != x.dtype:
        raise KernelError("moe_gate_up: sizes or dtypes do not fit")
    rows = plan.order.numel()
    z = torch.empty((rows, ff2 // 2), dtype=x.dtype, device=x.device)
    if _tc_fits(rows, W, x.dtype):
        xs = torch.empty((rows, W), dtype=x.dtype, device=x.device)
        use_gate("moe_tc")
        check(fn("moe_tc", "sx_moe_gather")(ptr(x), ptr(plan.order), ptr(xs), c_int(rows), c_int(W), c_int(top), stream()), "moe_gather")
        check(fn("moe_tc", "sx_moe_tc")(ptr(xs), ptr(gate_up), ptr(z), ptr(plan.offsets), c_int(rows), c_int(E), c_int(ff2 // 2),
                                        c_int(W), c_int(1), stream()), "moe_gate_up")
        return z
    use_gate("moe")
    check(fn("moe", "sx_moe_gemm")(ptr(x), ptr(gate_up), ptr(z), ptr(plan.offsets), ptr(plan.order), c_int(rows), c_int(E),
                                   c_int(ff2 // 2), c_int(W), c_int(top), c_int(1), c_int(dt_code(x.dtype)),
                                   c_int(dt_code(z.dtype)), stream()), "moe_gate_up")
    return z


def moe_down(z: torch.Tensor, down: torch.Tensor, plan: ExpertPlan) -> torch.Tensor:
    """``z_r Wd_e^T`` for every sorted row ``r`` with its expert's ``down [experts, width, ff]``: float32 ``[pairs, width]``."""
    require_cuda(z, down)
    rows, ff = z.shape
    E, W, ff2 = down.shape
    if ff2 != ff or E != plan.experts or down.dtype != z.dtype or rows != plan.order.numel():
        raise KernelError("moe_down: sizes or dtypes do not fit")
    y = torch.empty((rows, W), dtype=torch.float32, device=z.device)
    if _tc_fits(rows, ff, z.dtype):
        check(fn("moe_tc", "sx_moe_tc")(ptr(z), ptr(down), ptr(y), ptr(plan.offsets), c_int(rows), c_int(E), c_int(W), c_int(ff),
                                        c_int(0), stream()), "moe_down")
        return y
    check(fn("moe", "sx_moe_gemm")(ptr(z), ptr(down), ptr(y), ptr(plan.offsets), ptr(plan.order), c_int(rows), c_int(E),
                                   c_int(W), c_int(ff), c_int(1), c_int(0), c_int(dt_code(z.dtype)), c_int(dt_code(y.dtype)),
                                   stream()), "moe_down")
    return y


def moe_combine(y: torch.Tensor, plan: ExpertPlan, weights: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """``out[t] = sum_j weights[t, j] * y[place[t * top + j]]`` with the choices in their order; ``[T, width]``."""
    return moe_combine_rows(y, plan.place, weights, out_dtype)


def moe_combine_rows(y: torch.Tensor, place: torch.Tensor, weights: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    require_cuda(y, weights, place)
    T, top = weights.shape
    if y.shape[0] != T * top or weights.dtype != torch.float32:
        raise KernelError("moe_combine: sizes do not fit")
    out = torch.empty((T, y.shape[1]), dtype=out_dtype, device=y.device)
    check(fn("moe", "sx_moe_combine")(ptr(y), c_int(dt_code(y.dtype)), ptr(place), ptr(weights), ptr(out),
                                      c_int(dt_code(out_dtype)), c_int(T), c_int(y.shape[1]), c_int(top), stream()), "moe_combine")
    return out
