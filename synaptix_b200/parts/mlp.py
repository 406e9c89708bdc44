"""Dense gated feed-forward (SwiGLU): ``down( silu(x Wg^T) * (x Wu^T) )``,
``silu(x) = x / (1 + exp(-x))`` (crates/synaptix-models/llm/common/src/model.rs:1670-1691;
crates/synaptix-kernels-cuda/src/cu/fused/mlp/silu_and_mul.cu:11-25).  Gate and up
run as one product; the activation is computed in 32-bit.

``CappedGLU``: ``down( g sigmoid(alpha g) (u + 1) )`` with ``g = min(x Wg^T, limit)`` and
``u = clamp(x Wu^T, -limit, limit)``; ``alpha`` and ``limit`` are parameters.

``MixtureOfExperts``: ``experts`` small SwiGLU feed-forwards without biases, of which every token uses ``top``:
router logits ``z = Wr x`` and their softmax over ALL experts in 32-bit, the ``top`` largest scores chosen, divided by
their sum (+ ``1e-20``) and multiplied by ``scale``; the result is the weighted sum of the chosen experts' outputs.
The tokens are sorted by expert on the device and each expert's rows run as one group of a grouped product.
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional

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


class MixtureOfExperts(FeedForward):
    accepts_lazy_input = False
    can_defer_output = False

    NAMES = {"router": "router", "expert": "e{}.", "gate": "gate", "up": "up", "down": "down"}
    SUM_EPS = 1e-20                 # added to the sum of the chosen scores before the division

    def __init__(self, prefix: str, width: int, intermediate: int, experts: int, top: int, *, scale: float = 1.0,
                 names: Optional[Mapping[str, str]] = None):
        if not 0 < top <= experts:
            raise ValueError("0 < top <= experts")
        self.prefix, self.width, self.intermediate = prefix, width, intermediate
        self.experts, self.top, self.scale = experts, top, float(scale)
        self.names = dict(self.NAMES, **(names or {}))
        self.router: Optional[torch.Tensor] = None      # float32 [experts, width]
        self.gate_up: Optional[torch.Tensor] = None     # [experts, 2 * intermediate, width]: gate rows, then up rows
        self.down: Optional[torch.Tensor] = None        # [experts, width, intermediate]

    def _name(self, e: int, which: str) -> str:
        return self.prefix + self.names["expert"].format(e) + self.names[which]

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs = {self.prefix + self.names["router"]: TensorSpec((self.experts, self.width), "matrix")}
        for e in range(self.experts):
            specs[self._name(e, "gate")] = TensorSpec((self.intermediate, self.width), "matrix")
            specs[self._name(e, "up")] = TensorSpec((self.intermediate, self.width), "matrix")
            specs[self._name(e, "down")] = TensorSpec((self.width, self.intermediate), "matrix")
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        self.router = to_device_f32(tensors[self.prefix + self.names["router"]], rt)
        gu = [torch.cat([tensors[self._name(e, "gate")], tensors[self._name(e, "up")]], dim=0) for e in range(self.experts)]
        self.gate_up = to_device_matrix(torch.stack(gu), rt)
        self.down = to_device_matrix(torch.stack([tensors[self._name(e, "down")] for e in range(self.experts)]), rt)

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        ids, weights = ops.moe_route(x, self.router, self.top, self.scale, self.SUM_EPS)
        plan = ops.moe_sort(ids, self.experts)
        z = ops.moe_gate_up(x, self.gate_up, plan, self.top)
        y = ops.moe_down(z, self.down, plan)
        return ops.moe_combine(y, plan, weights, x.dtype)
