"""Mixers that carry a state of fixed size from token to token instead of keys and values.

``MinGRU``: a gated recurrence per channel whose gates read only the current token.  With ``a_z, a_x, a_g`` the three
projections of the input (``n`` channels each; the first two with a bias):

    z = sigmoid(a_z),   cand = a_x + 1/2  if a_x >= 0  else sigmoid(a_x),
    S_t = (1 - z) S_(t-1) + z cand,       out = Wo (S_t * silu(a_g))

``Retention``: linear attention with a fixed decay per head, no softmax and no denominator.  Per head, with q and k of
``dim`` and v of ``vdim`` elements:

    S_t = decay S_(t-1) + (k_t k_scale) v_t^T,   o_t = S_t^T q_t,
    out = Wo (o_t / rms(o_t) * silu(a_g))        (unit norm and gate optional)

``MLSTM``: a matrix memory per head with exponential gates and a running maximum that keeps them in range.  Per head,
with ``q`` (times ``dim^-1/2``) and ``k`` of ``dim`` and ``v`` of ``vdim`` elements, log gates
``i = cap tanh((Wi x + bi) / cap)`` and ``f = logsigmoid(cap tanh((Wf x + bf) / cap))``:

    m_t = max(f + m_(t-1), i),           S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T,
    n_t = the same with k alone,         o_t = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6),
    out = Wo (o_t / rms(o_t) * gain * sigmoid(Wg x))        (S, n and m start at 0)

All states start at zero, live in 32-bit in the cache's per-sequence state storage and go on from step to step; the
gates, decays, norms and sums are 32-bit whatever the compute dtype.  Both parts can run alone (they own their
projections) or ``shared``: beside other mixers under one owner that stacks the projections of all of them
(``input_parts``, ``output_part``, ``mix``).
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional, Sequence

import torch

from .. import ops
from ..cache.store import BundleRequest, StateRequest
from ..weights.loader import TensorSpec
from .base import Mixer, Part, Runtime, StepContext, to_device_f32
from .linear import Linear


class MinGRU(Mixer):
    accepts_lazy_input = False
    can_defer_output = True

    NAMES = {"z": "z", "x": "x", "g": "g", "o": "o", "z_bias": "z.b", "x_bias": "x.b"}

    def __init__(self, prefix: str, width: int, channels: int, *, names: Optional[Mapping[str, str]] = None):
        self.prefix, self.width, self.n = prefix, width, channels
        self.names = dict(self.NAMES, **(names or {}))
        p, n = prefix, self.names
        self.zxg = Linear([p + n["z"], p + n["x"], p + n["g"]], width, [channels] * 3)
        self.o = Linear(p + n["o"], channels, width)
        self.bias_z: Optional[torch.Tensor] = None
        self.bias_x: Optional[torch.Tensor] = None

    def children(self) -> List[Part]:
        return [self.zxg, self.o]

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.prefix + self.names["z_bias"]: TensorSpec((self.n,), "bias"),
                self.prefix + self.names["x_bias"]: TensorSpec((self.n,), "bias")}

    def bind(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        self.bias_z = to_device_f32(tensors[self.prefix + self.names["z_bias"]], rt)
        self.bias_x = to_device_f32(tensors[self.prefix + self.names["x_bias"]], rt)

    def cache_request(self):
        return StateRequest((self.n,), torch.float32)

    def forward(self, x: torch.Tensor, ctx: StepContext, state: torch.Tensor, write_cache: bool = True,
                defer_output: bool = False):
        a = self.zxg.forward(x)
        y = ops.mingru(a, 0, self.n, 2 * self.n, self.n, self.bias_z, self.bias_x, state, ctx)
        return self.o.deferred(y) if defer_output else self.o.forward(y)


class Retention(Mixer):
    accepts_lazy_input = False
    can_defer_output = True

    NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o"}

    def __init__(self, prefix: str, width: int, heads: int, dim: int, vdim: int, decay: Sequence[float], *,
                 k_scale: Optional[float] = None, unit_norm_eps: Optional[float] = None, gated: bool = True,
                 names: Optional[Mapping[str, str]] = None, shared: bool = False):
        if len(decay) != heads:
            raise ValueError(f"{len(decay)} decays for {heads} heads")
        self.prefix, self.width = prefix, width
        self.heads, self.dim, self.vdim = heads, dim, vdim
        self.decay_values = [float(d) for d in decay]
        self.k_scale = float(k_scale) if k_scale is not None else float(dim) ** -0.5
        self.unit_norm_eps = unit_norm_eps
        self.gated = bool(gated)
        self.names = dict(self.NAMES, **(names or {}))
        self.shared = bool(shared)
        self.proj = self.o = None
        if not shared:
            names_in, outs = zip(*self.input_parts())
            self.proj = Linear(list(names_in), width, list(outs))
            self.o = Linear(self.output_part()[0], self.output_part()[1], width)
        self.decay: Optional[torch.Tensor] = None

    def input_parts(self):
        p, n = self.prefix, self.names
        parts = [(p + n["q"], self.heads * self.dim), (p + n["k"], self.heads * self.dim), (p + n["v"], self.heads * self.vdim)]
        if self.gated:
            parts.append((p + n["g"], self.heads * self.vdim))
        return parts

    def output_part(self):
        return self.prefix + self.names["o"], self.heads * self.vdim

    def children(self) -> List[Part]:
        return [] if self.shared else [self.proj, self.o]

    def bind(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32).to(rt.device)

    def cache_request(self):
        return StateRequest((self.heads, self.dim, self.vdim), torch.float32)

    def mix(self, proj: torch.Tensor, col: int, ctx: StepContext, state: torch.Tensor, write_cache: bool = True,
            out: Optional[torch.Tensor] = None, out_col: int = 0, out_scale: float = 1.0) -> torch.Tensor:
        hq, hv = self.heads * self.dim, self.heads * self.vdim
        return ops.retention(proj, col, col + hq, col + 2 * hq, col + 2 * hq + hv if self.gated else None,
                             self.heads, self.dim, self.vdim, self.decay, self.k_scale,
                             self.unit_norm_eps if self.unit_norm_eps is not None else 0.0,
                             self.unit_norm_eps is not None, state, ctx, out=out, out_col=out_col, out_scale=out_scale)

    def forward(self, x: torch.Tensor, ctx: StepContext, state: torch.Tensor, write_cache: bool = True,
                defer_output: bool = False):
        y = self.mix(self.proj.forward(x), 0, ctx, state, write_cache)
        return self.o.deferred(y) if defer_output else self.o.forward(y)


class MLSTM(Mixer):
    accepts_lazy_input = False
    can_defer_output = False

    NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "i": "i", "f": "f", "i_bias": "i.b", "f_bias": "f.b",
             "norm": "norm"}
    DENOMINATOR_EPS = 1e-6          # added to the denominator max(|n . q|, exp(-m))

    def __init__(self, prefix: str, width: int, heads: int, dim: int, vdim: int, *, gate_cap: float,
                 unit_norm_eps: float, q_scale: Optional[float] = None, names: Optional[Mapping[str, str]] = None,
                 shared: bool = False):
        """``shared``: an owner stacks ``input_parts()`` with other mixers' projections and calls ``mix(proj, col, ..., x=x)``
        (the gates' product stays this part's own: it reads the input ``x`` and leaves 32-bit results)."""
        self.prefix, self.width = prefix, width
        self.shared = bool(shared)
        self.heads, self.dim, self.vdim = heads, dim, vdim
        self.gate_cap = float(gate_cap)
        self.unit_norm_eps = float(unit_norm_eps)
        self.q_scale = float(q_scale) if q_scale is not None else float(dim) ** -0.5
        self.names = n = dict(self.NAMES, **(names or {}))
        p = prefix
        self.proj = self.o = None
        if not shared:
            names_in, outs = zip(*self.input_parts())
            self.proj = Linear(list(names_in), width, list(outs))
            self.o = Linear(self.output_part()[0], self.output_part()[1], width)
        # the gates' pre-activations leave their product in 32-bit: they are summed over the whole sequence
        self.gates = Linear([p + n["i"], p + n["f"]], width, [heads, heads])
        self.bias: Optional[torch.Tensor] = None
        self.norm_gain: Optional[torch.Tensor] = None

    needs_input = True              # mix() wants the mixer's input beside the stacked projection

    def input_parts(self):
        p, n = self.prefix, self.names
        return [(p + n["q"], self.heads * self.dim), (p + n["k"], self.heads * self.dim), (p + n["v"], self.heads * self.vdim),
                (p + n["g"], self.heads * self.vdim)]

    def output_part(self):
        return self.prefix + self.names["o"], self.heads * self.vdim

    def children(self) -> List[Part]:
        return [self.gates] if self.shared else [self.proj, self.gates, self.o]

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        p, n = self.prefix, self.names
        return {p + n["i_bias"]: TensorSpec((self.heads,), "bias"), p + n["f_bias"]: TensorSpec((self.heads,), "bias"),
                p + n["norm"]: TensorSpec((self.heads * self.vdim,), "gain")}

    def bind(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        p, n = self.prefix, self.names
        self.bias = to_device_f32(torch.cat([tensors[p + n["i_bias"]].float(), tensors[p + n["f_bias"]].float()]), rt)
        self.norm_gain = to_device_f32(tensors[p + n["norm"]], rt)

    def cache_request(self):
        return BundleRequest((StateRequest((self.heads, self.dim, self.vdim), torch.float32),
                              StateRequest((self.heads, self.dim), torch.float32),
                              StateRequest((self.heads,), torch.float32)))

    def mix(self, proj: torch.Tensor, col: int, ctx: StepContext, state, write_cache: bool = True, *, x=None, **_):
        """From a projection whose columns from ``col`` on are this part's q, k, v and output gate, and the mixer's input
        ``x`` (for the gates): what the output projection reads, ``[T, heads * vdim]``."""
        g = self.gates.forward(x, out_dtype=torch.float32)
        hq, hv = self.heads * self.dim, self.heads * self.vdim
        return ops.mlstm(proj, col, col + hq, col + 2 * hq, col + 2 * hq + hv, g, self.bias, self.gate_cap, self.q_scale,
                         self.heads, self.dim, self.vdim, self.norm_gain, self.unit_norm_eps, self.DENOMINATOR_EPS,
                         state[0], state[1], state[2], ctx)

    def forward(self, x: torch.Tensor, ctx: StepContext, state, write_cache: bool = True):
        return self.o.forward(self.mix(self.proj.forward(x), 0, ctx, state, write_cache, x=x))
