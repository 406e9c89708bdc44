"""The Tamovik decoder put together from parts.

The embedding adds a row of a hashed table of token pairs (``BigramEmbedding``; the token before is a sequence's
state).  A layer is a ``PostNormBlock``: ``h += norm1(mixer(h))``, then ``h += norm2(ffn(h))``, the sublayers reading the
stream itself.  Mixers by layer type:

* ``latent_attention``: ``LatentAttention`` without a query latent (``q = Wq x``) and without a gate: keys and values of
  all heads made from one cached latent, a rotated part of ``rot_dim`` elements in the rotate-half layout
  (``RotaryHalf``, optionally with stretched frequencies, ``FrequencyRamp``), every earlier key visible;
* ``parallel``: ``NormedParallelMixers`` of ``ConvNormAttention`` (short convolutions on q and k, values = keys, norm over
  the whole projection, chunks, an output gate per element) and ``MLSTM``, each output RMS-normed over the width, half
  their sum.

Feed-forwards: ``GeluGLU`` (dense) or ``MixtureOfExperts`` with sigmoid scores, a correction per expert for the choice,
groups of experts, weights that are not renormalised, and capped experts.

Tensor names: ``embed``, ``bigram``, ``head``, ``final.norm``, and per layer ``l<i>.norm1|norm2``, ``l<i>.mix.*``
(``left.*``, ``right.*``, ``left.out``, ``right.out`` in a parallel layer), ``l<i>.mlp.gate|up|down`` or
``l<i>.mlp.router|correction|e<j>.gate|up|down``.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.tamovik import TamovikConfig
from ..parts import (BigramEmbedding, ConvNormAttention, FrequencyRamp, GeluGLU, LatentAttention, MixtureOfExperts, MLSTM,
                     NoPosition, NormedParallelMixers, OutputHead, PostNormBlock, RMSNorm, RotaryHalf)
from .decoder import DecoderModel

EXPERT_ALPHA = 1.702        # the experts' activation g * sigmoid(1.702 g) * (u + 1)
PARALLEL_FACTOR = 0.5       # a parallel layer's mixers: half the sum of their normed outputs


def build_tamovik(cfg: TamovikConfig) -> DecoderModel:
    W, eps = cfg.width, cfg.norm_eps
    embedding = BigramEmbedding("embed", "bigram", cfg.vocab, W, cfg.bigram_buckets, cfg.bigram_mul_prev, cfg.bigram_mul_cur)
    layers = []
    for i, spec in enumerate(cfg.layers):
        p = f"l{i}."
        if spec.type == "latent_attention":
            a = spec.latent
            position = NoPosition()
            if a.rot is not None:
                r = a.rot
                ramp = FrequencyRamp(r.factor, r.original, r.fast, r.slow) if r.factor is not None else None
                position = RotaryHalf(a.rot_dim, r.base, rotary_dim=r.dims, scaling=ramp)
            mixer = LatentAttention(p + "mix.", W, a.heads, a.dim, a.rot_dim, a.vdim, None, a.kv_rank, scale=a.scale,
                                    position=position, norm_eps=eps, window=None, gated=False)
        else:
            l, r = spec.left, spec.right
            left = ConvNormAttention(p + "mix.left.", W, l.heads, l.kv_heads, l.dim, taps=l.conv, scale=l.scale, norm_eps=eps,
                                     chunk=l.chunk, gated=True, shared=True)
            right = MLSTM(p + "mix.right.", W, r.heads, r.dim, r.vdim, gate_cap=r.gate_cap, unit_norm_eps=eps, shared=True)
            mixer = NormedParallelMixers(W, [left, right], [p + "mix.left.out", p + "mix.right.out"], eps=eps,
                                         factor=PARALLEL_FACTOR)
        norm2 = ffn = None
        if spec.mlp is not None:
            f = spec.mlp
            norm2 = RMSNorm(p + "norm2", W, eps)
            if f.kind == "dense":
                ffn = GeluGLU(p + "mlp.", W, f.ff, names={"gate": "gate", "up": "up", "down": "down"})
            else:
                ffn = MixtureOfExperts(p + "mlp.", W, f.ff, f.experts, f.top, scoring="sigmoid", renormalize=False,
                                       correction=True, groups=f.groups, activation=(EXPERT_ALPHA, f.limit))
        layers.append(PostNormBlock(mixer, RMSNorm(p + "norm1", W, eps), ffn, norm2))
    return DecoderModel(cfg, embedding, layers, RMSNorm("final.norm", W, eps), OutputHead("head", cfg.vocab, W, False, embedding))


register_architecture(TamovikConfig, build_tamovik)
