"""The arrangement of parts in a layer.

``PreNormBlock`` (crates/synaptix-models/llm/common/src/model.rs:1179-1199):
``h += mixer(norm1(h)); h += ffn(norm2(h))``.  The residual stream ``h`` is
float32; each branch output is handed on as ``pending`` and added by the next
norm's kernel, so a sum and a norm are one pass over memory.

``ConvPreNormBlock``: the same arrangement with a short causal convolution over time
between each norm and its sublayer: what a sublayer reads is ``y + conv(y)`` with
``y = norm(h)``, ``conv(y)_t = sum_j w[:, j] * y_(t - taps + 1 + j)`` per channel, zeros
before the sequence's start (``TokenConv``).  The last ``taps - 1`` inputs of each
convolution are part of a sequence's state; the feed-forward half may be absent.

``ParallelBlock``: mixer and feed-forward side by side on the SAME stream, each behind a
norm of its own and times a learned vector over the width (a layer scale):
``h += mult * (ls1 * mixer(norm1(h)) + ls2 * ffn(norm2(h)))``.  Both norms share the
row's root mean square, so one kernel makes both; the sum is handed on as a
``ScaledSum`` and added by the next norm's kernel.  The feed-forward half may be absent.

``SandwichBlock``: every sublayer between two norms, ``h += mult * post(sublayer(pre(h)))``,
with an optional ``TokenShift`` of what the mixer reads.

``PostNormBlock``: a norm on every sublayer's OUTPUT only: ``h += norm1(mixer(h))``, then ``h += norm2(ffn(h))``; the
sublayers read the stream itself.
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional, Tuple

import torch

from .. import ops
from ..cache.store import BundleRequest, StateRequest
from ..weights.loader import TensorSpec
from .base import (FeedForward, Mixer, Norm, NormedDelta, NormedSum, Part, PendingLinear, PendingNorm, Runtime, ScaledRows, ScaledSum,
                   StepContext, plain, to_device_f32)


class PreNormBlock(Part):
    takes_pending_product = True   # forward's ``pending`` may be a PendingLinear

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm, ffn: FeedForward):
        self.norm1, self.mixer, self.norm2, self.ffn = norm1, mixer, norm2, ffn

    def children(self) -> List[Part]:
        return [self.norm1, self.mixer, self.norm2, self.ffn]

    def cache_request(self):
        return self.mixer.cache_request()

    def forward(self, h: torch.Tensor, pending: Optional[torch.Tensor], ctx: StepContext,
                cache_view, write_cache: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
        """``pending`` and the second result may be a ``PendingLinear``: a branch's last product handed on unrun,
        so that the norm after it can let it add itself into ``h`` (only between parts that say they can)."""
        if isinstance(pending, PendingLinear) and not self.norm1.takes_pending_product:
            pending = pending.materialize()
        x = self.norm1.add_forward(h, pending, lazy=self.mixer.accepts_lazy_input)
        if self.mixer.can_defer_output and self.norm2.takes_pending_product:
            a = self.mixer.forward(x, ctx, cache_view, write_cache, defer_output=True)
        else:
            a = self.mixer.forward(x, ctx, cache_view, write_cache)
        if isinstance(x, (PendingNorm, ScaledRows)):
            h = x.h_after()
        y = self.norm2.add_forward(h, a, lazy=self.ffn.accepts_lazy_input)
        m = self.ffn.forward(y, ctx, defer_output=True) if self.ffn.can_defer_output else self.ffn.forward(y, ctx)
        if isinstance(y, (PendingNorm, ScaledRows)):
            h = y.h_after()
        return h, m


class TokenConv(Part):
    """The taps of a short causal convolution over time, one filter per channel: tensor ``[width, taps]``, no bias."""

    def __init__(self, weight_name: str, width: int, taps: int):
        if taps < 1:
            raise ValueError("a convolution has at least one tap")
        self.weight_name, self.width, self.taps = weight_name, width, taps
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.weight_name: TensorSpec((self.width, self.taps), "bias")}

    def bind(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        self.weight = to_device_f32(tensors[self.weight_name], rt)

    def state_request(self) -> StateRequest:
        """The last ``taps - 1`` inputs of a sequence, oldest first, in 32-bit."""
        return StateRequest((self.taps - 1, self.width), torch.float32)


class ConvPreNormBlock(Part):
    """``h += mixer(c1(norm1(h))); h += ffn(c2(norm2(h)))`` with ``c(y) = y + conv(y)``; ``norm2, conv2, ffn`` may all
    be ``None`` (a layer without a feed-forward).  The norms are RMS norms with a plain gain (the fused kernel computes
    them).  Cache entry: the bundle (mixer's request, conv1's inputs[, conv2's inputs])."""
    takes_pending_product = False

    def __init__(self, norm1: Norm, conv1: TokenConv, mixer: Mixer, norm2: Optional[Norm] = None,
                 conv2: Optional[TokenConv] = None, ffn: Optional[FeedForward] = None):
        if (norm2 is None) != (ffn is None) or (conv2 is None) != (ffn is None):
            raise ValueError("norm2, conv2 and ffn come together or not at all")
        self.norm1, self.conv1, self.mixer = norm1, conv1, mixer
        self.norm2, self.conv2, self.ffn = norm2, conv2, ffn

    def children(self) -> List[Part]:
        return [p for p in (self.norm1, self.conv1, self.mixer, self.norm2, self.conv2, self.ffn) if p is not None]

    def cache_request(self):
        items = [self.mixer.cache_request(), self.conv1.state_request()]
        if self.ffn is not None:
            items.append(self.conv2.state_request())
        return BundleRequest(tuple(items))

    def forward(self, h: torch.Tensor, pending, ctx: StepContext, views, write_cache: bool = True):
        dtype = ctx.runtime.dtype
        x = ops.add_rmsnorm_conv(h, plain(pending), self.norm1.weight, self.norm1.eps, self.conv1.weight, views[1], ctx, dtype)
        a = self.mixer.forward(x, ctx, views[0], write_cache)
        if self.ffn is None:
            return h, a
        y = ops.add_rmsnorm_conv(h, plain(a), self.norm2.weight, self.norm2.eps, self.conv2.weight, views[2], ctx, dtype)
        return h, self.ffn.forward(y, ctx)


_SIDE_STREAMS = {}


def _side_stream(device) -> "torch.cuda.Stream":
    """One second stream per device, for a branch that runs beside another."""
    key = torch.device(device).index or 0
    if key not in _SIDE_STREAMS:
        _SIDE_STREAMS[key] = torch.cuda.Stream(device=device)
    return _SIDE_STREAMS[key]


class ParallelBlock(Part):
    """``h += mult * (ls1 * mixer(norm1(h)) + ls2 * ffn(norm2(h)))``, both branches of the same ``h``.  ``norm1`` and
    ``norm2`` are RMS norms (their gains may differ, their eps not); ``scale_names`` are the tensors ``ls1`` and
    ``ls2`` (vectors over the width).  ``norm2`` and ``ffn`` may both be ``None``.

    The branches do not depend on each other.  In single-token steps, where a layer is a chain of small kernels, the
    feed-forward runs on a second stream (option ``branch_streams``): it begins behind the norm kernel (an event) and the
    step's stream waits for its end before anything reads its result; inside a captured step these are two branches of
    the graph.  What crosses the streams needs no word to the allocator: the feed-forward's input lives until this
    function returns, by when the step's stream already waits for the feed-forward's end, so its memory is not handed
    out again before that; the feed-forward's result is read by the next norm on the step's stream, and the second
    stream does nothing more before an event that is recorded behind such a norm."""
    takes_pending_product = False

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Optional[Norm], ffn: Optional[FeedForward], *,
                 scale_names: Tuple[str, str], mult: float = 1.0):
        if (norm2 is None) != (ffn is None):
            raise ValueError("norm2 and ffn come together or not at all")
        if norm2 is not None and norm2.eps != norm1.eps:
            raise ValueError("the two norms of a parallel block share their eps")
        self.norm1, self.mixer, self.norm2, self.ffn = norm1, mixer, norm2, ffn
        self.scale_names = tuple(scale_names)
        self.mult = float(mult)
        self.width = norm1.width
        self.s1: Optional[torch.Tensor] = None
        self.s2: Optional[torch.Tensor] = None

    def children(self) -> List[Part]:
        return [p for p in (self.norm1, self.mixer, self.norm2, self.ffn) if p is not None]

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs = {self.scale_names[0]: TensorSpec((self.width,), "gain")}
        if self.ffn is not None:
            specs[self.scale_names[1]] = TensorSpec((self.width,), "gain")
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        # mult * (ls1 * a + ls2 * b) as (mult ls1) * a + (mult ls2) * b, the factors formed once in 32-bit
        self.s1 = to_device_f32(tensors[self.scale_names[0]].to(torch.float32) * self.mult, rt)
        if self.ffn is not None:
            self.s2 = to_device_f32(tensors[self.scale_names[1]].to(torch.float32) * self.mult, rt)

    def cache_request(self):
        return self.mixer.cache_request()

    def forward(self, h: torch.Tensor, pending, ctx: StepContext, cache_view, write_cache: bool = True):
        if isinstance(pending, ScaledSum):
            terms = pending.terms
        else:
            pending = plain(pending)
            terms = [] if pending is None else [(pending, None)]
        gains = [self.norm1.weight] + ([self.norm2.weight] if self.ffn is not None else [])
        xs = ops.add_scaled_rmsnorm(h, terms, gains, self.norm1.eps, ctx.runtime.dtype)
        if self.ffn is None:
            return h, ScaledSum([(self.mixer.forward(xs[0], ctx, cache_view, write_cache), self.s1)])
        if ctx.all_single and ops.OPTIONS.branch_streams and h.is_cuda:
            main, side = torch.cuda.current_stream(h.device), _side_stream(h.device)
            fork = torch.cuda.Event()
            fork.record(main)
            side.wait_event(fork)
            with torch.cuda.stream(side):
                b = self.ffn.forward(xs[1], ctx)
                join = torch.cuda.Event()
                join.record(side)
            a = self.mixer.forward(xs[0], ctx, cache_view, write_cache)
            main.wait_event(join)
        else:
            a = self.mixer.forward(xs[0], ctx, cache_view, write_cache)
            b = self.ffn.forward(xs[1], ctx)
        return h, ScaledSum([(a, self.s1), (b, self.s2)])


class TokenShift(Part):
    """What a sublayer reads is blended with what it read for the token before: ``y_t + (y_(t-1) - y_t) * s`` with a
    learned vector ``s`` over the width and ``y_(-1) = 0``.  The last ``y`` of a sequence is part of its state."""

    def __init__(self, weight_name: str, width: int):
        self.weight_name, self.width = weight_name, width
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.weight_name: TensorSpec((self.width,), "bias")}

    def bind(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        self.weight = to_device_f32(tensors[self.weight_name], rt)

    def state_request(self) -> StateRequest:
        return StateRequest((self.width,), torch.float32)


class SandwichBlock(Part):
    """Sublayers normed on both sides: ``h += mult * post1(mixer(shift(pre1(h))))``, then
    ``h += mult * post2(ffn(pre2(h)))``.  The four norms take ``NormedDelta`` (layer norms); ``shift`` (a
    ``TokenShift``, optional) blends the mixer's input with the previous token's; ``pre2, post2, ffn`` may all be
    ``None``.  A branch's output travels on as a ``NormedDelta`` so that its own norm, the sum into the stream and the
    next norm are one kernel.  ``mixer.output_bias`` (a float32 vector or ``None``), when the mixer has one, is the
    bias of its last product, added inside that kernel.  Cache entry: the mixer's request, or the bundle (mixer's
    request, the shift's last input)."""
    takes_pending_product = False

    def __init__(self, pre1: Norm, mixer: Mixer, post1: Norm, pre2: Optional[Norm] = None, ffn: Optional[FeedForward] = None,
                 post2: Optional[Norm] = None, *, mult: float = 1.0, shift: Optional[TokenShift] = None):
        if (pre2 is None) != (ffn is None) or (post2 is None) != (ffn is None):
            raise ValueError("pre2, ffn and post2 come together or not at all")
        for n in (pre1, post1, pre2, post2):
            if n is not None and not n.takes_normed_delta:
                raise ValueError("the norms of a sandwich block take a branch with a norm of its own")
        self.pre1, self.mixer, self.post1 = pre1, mixer, post1
        self.pre2, self.ffn, self.post2 = pre2, ffn, post2
        self.mult = float(mult)
        self.shift = shift

    def children(self) -> List[Part]:
        return [p for p in (self.pre1, self.shift, self.mixer, self.post1, self.pre2, self.ffn, self.post2) if p is not None]

    def cache_request(self):
        if self.shift is None:
            return self.mixer.cache_request()
        return BundleRequest((self.mixer.cache_request(), self.shift.state_request()))

    def forward(self, h: torch.Tensor, pending, ctx: StepContext, views, write_cache: bool = True):
        if self.shift is not None:
            mixer_view, shift_state = views
            # a block reads its neighbour's row of the stream before the sum, so the sums go to a new tensor unless
            # every sequence brings one row
            x, h = self.pre1.add_forward(h, pending, shift=self.shift.weight, state=shift_state, ctx=ctx,
                                         in_place=bool(ctx.all_single))
        else:
            mixer_view = views
            x = self.pre1.add_forward(h, pending)
        a = self.mixer.forward(x, ctx, mixer_view, write_cache)
        a = NormedDelta(a, self.post1, self.mult, getattr(self.mixer, "output_bias", None))
        if self.ffn is None:
            return h, a
        y = self.pre2.add_forward(h, a)
        return h, NormedDelta(self.ffn.forward(y, ctx), self.post2, self.mult)


class PostNormBlock(Part):
    """``h += norm1(mixer(h))``, then ``h += norm2(ffn(h))``: the sublayers read the stream itself (rounded to the compute
    dtype), and only what they return is normed (RMS norms).  ``norm2`` and ``ffn`` may both be ``None``.

    A branch travels on as a ``NormedDelta`` (whose ``x`` may be a mixer's ``NormedSum``), so that the branch's norm, the
    sum into the 32-bit stream and the rows the next sublayer reads are one kernel (``ops.add_normed``); the final norm
    takes the last branch the same way."""
    takes_pending_product = False

    def __init__(self, mixer: Mixer, norm1: Norm, ffn: Optional[FeedForward] = None, norm2: Optional[Norm] = None):
        if (norm2 is None) != (ffn is None):
            raise ValueError("norm2 and ffn come together or not at all")
        for n in (norm1, norm2):
            if n is not None and hasattr(n, "bias"):
                raise ValueError("the norms of a post-norm block are RMS norms")
        self.mixer, self.norm1, self.ffn, self.norm2 = mixer, norm1, ffn, norm2

    def children(self) -> List[Part]:
        return [p for p in (self.mixer, self.norm1, self.ffn, self.norm2) if p is not None]

    def cache_request(self):
        return self.mixer.cache_request()

    @staticmethod
    def _read(h: torch.Tensor, pending, dtype) -> torch.Tensor:
        """``h += pending`` and the rows a sublayer reads: the stream in the compute dtype (the stream itself in 32-bit)."""
        want = None if dtype == torch.float32 else dtype
        if isinstance(pending, NormedDelta) and pending.is_rms:
            terms, factor = pending.rms_terms()
            x = ops.add_normed(h, terms, pending.norm.weight, pending.norm.eps, want, factor=factor)
        else:
            pending = plain(pending)
            if pending is None and want is None:
                return h
            x = ops.add_normed(h, [] if pending is None else [(pending, None)], None, 0.0, want)
        return h if want is None else x

    def forward(self, h: torch.Tensor, pending, ctx: StepContext, cache_view, write_cache: bool = True):
        dtype = ctx.runtime.dtype
        x = self._read(h, pending, dtype)
        if getattr(self.mixer, "returns_normed_sum", False):
            a = self.mixer.forward(x, ctx, cache_view, write_cache, normed_sum=True)
        else:
            a = self.mixer.forward(x, ctx, cache_view, write_cache)
        a = NormedDelta(a, self.norm1)
        if self.ffn is None:
            return h, a
        y = self._read(h, a, dtype)
        if getattr(self.ffn, "can_defer_combine", False):
            return h, NormedDelta(self.ffn.forward(y, ctx, defer_combine=True), self.norm2)
        return h, NormedDelta(self.ffn.forward(y, ctx), self.norm2)
