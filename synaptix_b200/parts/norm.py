"""RMSNorm with a plain gain (or a gain stored around zero: ``offset + w``), fused with the residual sum.

Formula (crates/synaptix-ops/src/norm/rms_norm.rs:17-26; CUDA
crates/synaptix-kernels-cuda/src/cu/reduction/rms_norm.cu:84-96):
``y = x * rsqrt(mean(x^2) + eps) * w`` in 32-bit, gain ``w`` (not ``1 + w``).
The residual stream itself is float32 here, so the sum ``h + delta`` is never
rounded to the compute dtype (the reference rounds it, rmsnorm_residual.cu:97-159).
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import Norm, NormedDelta, PendingLinear, PendingNorm, Runtime, ScaledRows, ScaledSum, plain, to_device_f32


class RMSNorm(Norm):
    """``offset``: the stored tensor ``w`` lies around zero and the gain is ``offset + w`` (formed once, in 32-bit,
    when the weights are bound); 0 is the plain gain."""

    def __init__(self, weight_name: str, width: int, eps: float, offset: float = 0.0):
        self.weight_name = weight_name
        self.width = width
        self.eps = float(eps)
        self.offset = float(offset)
        self.weight: Optional[torch.Tensor] = None
        self._dtype = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.weight_name: TensorSpec((self.width,), "gain" if self.offset == 0.0 else "gain0")}

    def bind(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        w = tensors[self.weight_name].to(torch.float32)
        self.weight = to_device_f32(w + self.offset if self.offset != 0.0 else w, rt)
        self._dtype = rt.dtype

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return ops.add_rmsnorm(h, None, self.weight, self.eps, self._dtype)

    takes_pending_product = True
    takes_scaled_sum = True
    takes_normed_delta = True      # of a branch behind an RMS norm (a layer norm's branch is made plain first)

    def add_forward(self, h, delta, rows=None, lazy=False):
        if isinstance(delta, NormedDelta) and delta.is_rms and delta.norm.eps == self.eps:
            # the branch's norm, the sum into the stream and this norm in one kernel
            terms, factor = delta.rms_terms()
            return ops.add_normed(h, terms, delta.norm.weight, self.eps, self._dtype, factor=factor, out_gain=self.weight,
                                  rows=rows)
        if isinstance(delta, NormedDelta):
            delta = delta.materialize()
        if isinstance(delta, ScaledSum):
            # the branches' sum, the sum into the stream and the norm in one kernel
            return ops.add_scaled_rmsnorm(h, delta.terms, [self.weight], self.eps, self._dtype, rows=rows)[0]
        if isinstance(delta, PendingLinear):
            N, K = delta.weight.shape
            if (lazy and rows is None and N == self.width and h.dtype == torch.float32 and h.is_contiguous()
                    and delta.weight.dtype == self._dtype and delta.x.dtype == self._dtype
                    and ops.residual_product_fusable(h.shape[0], N, K, self._dtype)):
                # the product adds itself into h and leaves the rows of this norm without their factor
                x, ssq = ops.linear_into_residual(delta.x, delta.weight, h, self.weight)
                return ScaledRows(x, ssq, self.eps, h, self.weight, self._dtype)
            delta = delta.materialize()
        if lazy and rows is None and ops.norm_fusable(h.shape[0], h.shape[1], self._dtype):
            return PendingNorm(h, delta, self.weight, self.eps, self._dtype)
        return ops.add_rmsnorm(h, delta, self.weight, self.eps, self._dtype, rows=rows)


class LayerNorm(Norm):
    """``(x - mean) / sqrt(var + eps) * w + b`` over the width, ``var`` the mean of the squared deviations, all in
    32-bit; ``bias_name`` defaults to the gain's name with ``.b`` added.  Fused with the sum into the residual stream,
    also of a branch that has a norm of its own (``NormedDelta``)."""
    takes_normed_delta = True

    def __init__(self, weight_name: str, width: int, eps: float, bias_name: Optional[str] = None):
        self.weight_name = weight_name
        self.bias_name = bias_name if bias_name is not None else weight_name + ".b"
        self.width = width
        self.eps = float(eps)
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None
        self._dtype = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.weight_name: TensorSpec((self.width,), "gain"), self.bias_name: TensorSpec((self.width,), "bias")}

    def bind(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        self.weight = to_device_f32(tensors[self.weight_name], rt)
        self.bias = to_device_f32(tensors[self.bias_name], rt)
        self._dtype = rt.dtype

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return ops.add_layernorm(h, None, self.weight, self.bias, self.eps, self._dtype)[0]

    def add_forward(self, h, delta, rows=None, lazy=False, shift=None, state=None, ctx=None, in_place=True):
        """``shift``, ``state``, ``ctx``: a token shift of the normed rows (see ``ops.add_layernorm``); the stream
        after the sum is then returned too: ``(y, h')``."""
        kw = {}
        if isinstance(delta, NormedDelta):
            kw = dict(post=(delta.norm.weight, delta.norm.bias), mult=delta.mult, delta_bias=delta.bias)
            if delta.norm.eps != self.eps:
                raise ValueError("a branch's norm and the norm behind the sum share their eps")
            delta = delta.x
        else:
            delta = plain(delta)
        y, h_after = ops.add_layernorm(h, delta, self.weight, self.bias, self.eps, self._dtype, rows=rows, shift=shift,
                                       state=state, ctx=ctx, in_place=in_place, **kw)
        return (y, h_after) if shift is not None else y
