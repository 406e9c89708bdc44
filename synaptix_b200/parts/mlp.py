"""Dense gated feed-forward (SwiGLU): ``down( silu(x Wg^T) * (x Wu^T) )``,
``silu(x) = x / (1 + exp(-x))`` (crates/synaptix-models/llm/common/src/model.rs:1670-1691;
crates/synaptix-kernels-cuda/src/cu/fused/mlp/silu_and_mul.cu:11-25).  Gate and up
run as one product; the activation is computed in 32-bit.

``CappedGLU``: ``down( g sigmoid(alpha g) (u + 1) )`` with ``g = min(x Wg^T, limit)`` and
``u = clamp(x Wu^T, -limit, limit)``; ``alpha`` and ``limit`` are parameters.

``MixtureOfExperts``: ``experts`` small gated feed-forwards without biases, of which every token uses ``top``:
router logits ``z = Wr x`` in 32-bit, scores = their softmax over ALL experts (``scoring="sigmoid"``: the sigmoid of
each), the ``top`` largest chosen, their scores divided by their sum (+ ``1e-20``; ``renormalize=False``: left as they
are) and multiplied by ``scale``; the result is the weighted sum of the chosen experts' outputs.  Options of the
choice: ``correction`` (a tensor of one number per expert, added to the scores for the choice only; the weights use
the scores without it) and ``groups=(count, keep)`` (the experts form ``count`` equal groups of neighbours, a group's
value is the sum of its two largest choice values, only experts of the ``keep`` best groups can be chosen).
``activation=(alpha, limit)`` makes the experts ``CappedGLU``s instead of SwiGLUs.
The tokens are sorted by expert on the device and each expert's rows run as one group of a grouped product.
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional, Tuple

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import FeedForward, Part, Runtime, StepContext, to_device_f32, to_device_matrix
from .linear import Linear


class SwiGLU(FeedForward):
    accepts_lazy_input = True      # x goes straight into the fused gate/up product
    can_defer_output = True        # the down projection may be handed on unrun

    NAMES = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}

    def __init__(self, prefix: str, width: int, intermediate: int, names: Optional[Mapping[str, str]] = None):
        self.width, self.intermediate = width, intermediate
        n = dict(self.NAMES, **(names or {}))
        self.gate_up = Linear([prefix + n["gate"], prefix + n["up"]], width, [intermediate, intermediate])
        self.down = Linear(prefix + n["down"], intermediate, width)

    def children(self) -> List[Part]:
        return [self.gate_up, self.down]

    def forward(self, x: torch.Tensor, ctx: StepContext, defer_output: bool = False) -> torch.Tensor:
        z = self.gate_up.forward(x, epilogue="silu_mul")
        return self.down.deferred(z) if defer_output else self.down.forward(z)


class CappedGLU(FeedForward):
    accepts_lazy_input = False
    can_defer_output = True

    NAMES = {"gate": "gate", "up": "up", "down": "down"}

    def __init__(self, prefix: str, width: int, intermediate: int, *, limit: float, alpha: float = 1.702,
                 names: Optional[Mapping[str, str]] = None):
        self.width, self.intermediate = width, intermediate
        self.limit, self.alpha = float(limit), float(alpha)
        n = dict(self.NAMES, **(names or {}))
        self.gate_up = Linear([prefix + n["gate"], prefix + n["up"]], width, [intermediate, intermediate])
        self.down = Linear(prefix + n["down"], intermediate, width)

    def children(self) -> List[Part]:
        return [self.gate_up, self.down]

    def forward(self, x: torch.Tensor, ctx: StepContext, defer_output: bool = False) -> torch.Tensor:
        with ops.gate_activation(self.alpha, self.limit):          # the gate/up product's epilogue applies it
            z = self.gate_up.forward(x, epilogue="silu_mul")
        return self.down.deferred(z) if defer_output else self.down.forward(z)


class GeluGLU(SwiGLU):
    """``down( gelu_tanh(x Wg^T) * (x Wu^T) )`` with the tanh form of GELU,
    ``gelu_tanh(z) = z/2 (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))``: SwiGLU's arrangement with another activation in the
    gate/up product's epilogue."""
    accepts_lazy_input = False

    def forward(self, x: torch.Tensor, ctx: StepContext, defer_output: bool = False) -> torch.Tensor:
        with ops.gate_activation(form="gelu_tanh"):
            z = self.gate_up.forward(x, epilogue="silu_mul")
        return self.down.deferred(z) if defer_output else self.down.forward(z)


class MixtureOfExperts(FeedForward):
    accepts_lazy_input = False
    can_defer_output = False

    NAMES = {"router": "router", "correction": "correction", "expert": "e{}.", "gate": "gate", "up": "up", "down": "down"}
    SUM_EPS = 1e-20                 # added to the sum of the chosen scores before the division

    def __init__(self, prefix: str, width: int, intermediate: int, experts: int, top: int, *, scale: float = 1.0,
                 scoring: str = "softmax", renormalize: bool = True, correction: bool = False,
                 groups: Optional[Tuple[int, int]] = None, activation: Optional[Tuple[float, float]] = None,
                 names: Optional[Mapping[str, str]] = None):
        if not 0 < top <= experts:
            raise ValueError("0 < top <= experts")
        if scoring not in ("softmax", "sigmoid"):
            raise ValueError("scoring is softmax or sigmoid")
        if groups is not None:
            count, keep = groups
            if count <= 0 or experts % count or not 0 < keep <= count or top > keep * (experts // count):
                raise ValueError("groups: equal groups, 0 < keep <= count, and top experts must fit the kept groups")
        self.prefix, self.width, self.intermediate = prefix, width, intermediate
        self.experts, self.top, self.scale = experts, top, float(scale)
        self.scoring, self.renormalize, self.has_correction = scoring, bool(renormalize), bool(correction)
        self.groups = None if groups is None else (int(groups[0]), int(groups[1]))
        self.activation = None if activation is None else (float(activation[0]), float(activation[1]))
        self.correction: Optional[torch.Tensor] = None  # float32 [experts]
        self.names = dict(self.NAMES, **(names or {}))
        self.router: Optional[torch.Tensor] = None      # float32 [experts, width]
        self.gate_up: Optional[torch.Tensor] = None     # [experts, 2 * intermediate, width]: gate rows, then up rows
        self.down: Optional[torch.Tensor] = None        # [experts, width, intermediate]

    def _name(self, e: int, which: str) -> str:
        return self.prefix + self.names["expert"].format(e) + self.names[which]

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs = {self.prefix + self.names["router"]: TensorSpec((self.experts, self.width), "matrix")}
        if self.has_correction:
            specs[self.prefix + self.names["correction"]] = TensorSpec((self.experts,), "bias")
        for e in range(self.experts):
            specs[self._name(e, "gate")] = TensorSpec((self.intermediate, self.width), "matrix")
            specs[self._name(e, "up")] = TensorSpec((self.intermediate, self.width), "matrix")
            specs[self._name(e, "down")] = TensorSpec((self.width, self.intermediate), "matrix")
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        self.router = to_device_f32(tensors[self.prefix + self.names["router"]], rt)
        if self.has_correction:
            self.correction = to_device_f32(tensors[self.prefix + self.names["correction"]], rt)
        gu = [torch.cat([tensors[self._name(e, "gate")], tensors[self._name(e, "up")]], dim=0) for e in range(self.experts)]
        self.gate_up = to_device_matrix(torch.stack(gu), rt)
        self.down = to_device_matrix(torch.stack([tensors[self._name(e, "down")] for e in range(self.experts)]), rt)

    can_defer_combine = True        # forward(..., defer_combine=True) may hand the weighted sum on unformed (WeightedRows)

    def forward(self, x: torch.Tensor, ctx: StepContext, defer_combine: bool = False) -> torch.Tensor:
        ids, weights = ops.moe_route(x, self.router, self.top, self.scale, self.SUM_EPS, scoring=self.scoring,
                                     correction=self.correction, groups=self.groups, renormalize=self.renormalize)
        plan = ops.moe_sort(ids, self.experts)
        if self.activation is not None:
            with ops.gate_activation(*self.activation):          # the grouped gate/up product's epilogue applies it
                z = ops.moe_gate_up(x, self.gate_up, plan, self.top)
        else:
            z = ops.moe_gate_up(x, self.gate_up, plan, self.top)
        y = ops.moe_down(z, self.down, plan)
        if defer_combine:           # a block that norms this branch on its way into the stream forms the sum there
            return ops.WeightedRows(y, plan.place, weights, x.dtype)
        return ops.moe_combine(y, plan, weights, x.dtype)
