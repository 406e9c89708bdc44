"""Several mixers side by side on the same input, their outputs added with a weight each:
``sum_i scale_i * mixer_i(x)``.

The mixers are built ``shared`` (see ``Attention``, ``Retention``): this part stacks all their input projections
into ONE product, lets each mixer write what its output projection reads, times its scale, into its columns of one
buffer, and runs the output projections as ONE product over the joined inputs.  The cache entry is the bundle of the
mixers' requests, in their order.

``NormedParallelMixers``: the same arrangement where every mixer's output goes through an RMS norm of its own over the
model width before the sum: ``factor * sum_i rms_norm(mixer_i(x)) * gain_i``.  The input projections are still ONE
product; the output projections cannot be joined (each result is normed alone), and the norms and the sum are handed on
as a ``NormedSum`` to a block that can fold them into its own kernel.
"""
from __future__ import annotations

from typing import List, Sequence

import torch

from .. import ops
from ..cache.store import BundleRequest
from ..weights.loader import TensorSpec
from .base import Mixer, NormedSum, Part, Runtime, StepContext, to_device_f32
from .linear import JoinedLinear, Linear


class ParallelMixers(Mixer):
    accepts_lazy_input = False
    can_defer_output = True

    def __init__(self, width: int, mixers: Sequence[Mixer], scales: Sequence[float]):
        if len(mixers) != len(scales) or not mixers:
            raise ValueError("one scale per mixer")
        self.width = width
        self.mixers = list(mixers)
        self.scales = [float(s) for s in scales]
        names, outs, self.cols = [], [], []
        for m in self.mixers:
            self.cols.append(sum(outs))
            for n, o in m.input_parts():
                names.append(n)
                outs.append(o)
        self.proj = Linear(names, width, outs)
        o_names, o_ins = zip(*[m.output_part() for m in self.mixers])
        self.out_cols = [sum(o_ins[:i]) for i in range(len(o_ins))]
        self.o = JoinedLinear(list(o_names), list(o_ins), width)

    def children(self) -> List[Part]:
        return [self.proj, self.o] + self.mixers

    def cache_request(self):
        return BundleRequest(tuple(m.cache_request() for m in self.mixers))

    def forward(self, x: torch.Tensor, ctx: StepContext, views, write_cache: bool = True, defer_output: bool = False):
        a = self.proj.forward(x)
        y = torch.empty((a.shape[0], self.o.in_features), dtype=a.dtype, device=a.device)
        for m, col, view, oc, sc in zip(self.mixers, self.cols, views, self.out_cols, self.scales):
            m.mix(a, col, ctx, view, write_cache, out=y, out_col=oc, out_scale=sc)
        return self.o.deferred(y) if defer_output else self.o.forward(y)


class NormedParallelMixers(Mixer):
    """``factor * sum_i rms_norm(mixer_i(x)) * gain_i`` with ``gain_names`` the tensors of the gains (over the model width).
    The mixers are built ``shared``; one that sets ``needs_input`` is also handed the input ``x`` (for a product that
    is its own, such as gates that leave 32-bit results)."""
    accepts_lazy_input = False
    can_defer_output = False
    returns_normed_sum = True      # forward(..., normed_sum=True) may return a NormedSum instead of the tensor

    def __init__(self, width: int, mixers: Sequence[Mixer], gain_names: Sequence[str], *, eps: float, factor: float):
        if len(mixers) != len(gain_names) or not 1 <= len(mixers) <= 2:
            raise ValueError("one or two mixers, a gain each")
        self.width = width
        self.mixers = list(mixers)
        self.gain_names = list(gain_names)
        self.eps, self.factor = float(eps), float(factor)
        names, outs, self.cols = [], [], []
        for m in self.mixers:
            self.cols.append(sum(outs))
            for n, o in m.input_parts():
                names.append(n)
                outs.append(o)
        self.proj = Linear(names, width, outs)
        self.outs = [Linear(m.output_part()[0], m.output_part()[1], width) for m in self.mixers]
        self.gains: List[torch.Tensor] = []

    def children(self) -> List[Part]:
        return [self.proj] + self.outs + self.mixers

    def tensor_specs(self):
        return {n: TensorSpec((self.width,), "gain") for n in self.gain_names}

    def bind(self, tensors, rt: Runtime) -> None:
        self.gains = [to_device_f32(tensors[n], rt) for n in self.gain_names]

    def cache_request(self):
        return BundleRequest(tuple(m.cache_request() for m in self.mixers))

    def _branch(self, i: int, a, x, ctx, views, write_cache):
        m = self.mixers[i]
        kw = {"x": x} if getattr(m, "needs_input", False) else {}
        return self.outs[i].forward(m.mix(a, self.cols[i], ctx, views[i], write_cache, **kw))

    def forward(self, x: torch.Tensor, ctx: StepContext, views, write_cache: bool = True, normed_sum: bool = False):
        """In single-token steps, where each mixer is a chain of small kernels, the second mixer runs on a second stream
        beside the first (option ``branch_streams``; inside a captured step: two branches of the graph).  It begins behind
        the stacked projection (an event) and the step's stream waits for its end before anything reads its result; what
        crosses the streams lives until this function returns or is read on the step's stream behind that wait, and the
        second stream does nothing more before the next such event, so nothing is handed out again too early."""
        a = self.proj.forward(x)
        if len(self.mixers) == 2 and ctx.all_single and ops.OPTIONS.branch_streams and x.is_cuda:
            from .block import _side_stream
            main, side = torch.cuda.current_stream(x.device), _side_stream(x.device)
            fork = torch.cuda.Event()
            fork.record(main)
            side.wait_event(fork)
            with torch.cuda.stream(side):
                y1 = self._branch(1, a, x, ctx, views, write_cache)
                join = torch.cuda.Event()
                join.record(side)
            y0 = self._branch(0, a, x, ctx, views, write_cache)
            main.wait_event(join)
            ys = [y0, y1]
        else:
            ys = [self._branch(i, a, x, ctx, views, write_cache) for i in range(len(self.mixers))]
        s = NormedSum(list(zip(ys, self.gains)), self.factor, self.eps)
        return s if normed_sum else s.materialize()
