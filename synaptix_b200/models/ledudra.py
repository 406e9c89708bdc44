"""The Ledudra decoder put together from parts.

A layer is a ``SandwichBlock``: layer norms before and after each sublayer, every branch times ``residual_mult``, and a
token shift of what the mixer reads.  Both mixers are ``ScoredAttention`` with a sliding window, grouped heads and
values blended with those of the first layer that says ``v_mix``:

* ``attention``: biases on the four projections, rotation of neighbouring pairs (optionally with stretched slow
  frequencies), scores mixed over the heads, sigmoid weights with a bias per head, a sigmoid gate per head;
* ``attention_2``: q/k RMS norm with one gain for all heads, a learned bias per head and distance bucket, softmax.

The feed-forward (absent where ``mlp`` is null) is SwiGLU.  The final norm is a layer norm.

Tensor names: ``embed``, ``head``, ``final.norm[.b]`` and per layer ``l<i>.norm1|norm1b|norm2|norm2b[.b]``,
``l<i>.shift``, ``l<i>.mix.*``, ``l<i>.mlp.gate|up|down``.
"""
from __future__ import annotations

from ..config.ledudra import LedudraConfig
from ..config.registry import register_architecture
from ..parts import (Embedding, FrequencyRamp, LayerNorm, OutputHead, RotaryPairs, SandwichBlock, ScoredAttention, SwiGLU,
                     TokenShift)
from .decoder import DecoderModel

FF_NAMES = {"gate": "gate", "up": "up", "down": "down"}


def build_ledudra(cfg: LedudraConfig) -> DecoderModel:
    W, eps = cfg.width, cfg.norm_eps
    embedding = Embedding("embed", cfg.vocab, W)
    first_values = cfg.first_value_layer()
    layers = []
    for i, spec in enumerate(cfg.layers):
        p, m = f"l{i}.", spec.mixer
        value_mix = None if not m.v_mix else ("source" if i == first_values else "blend")
        common = dict(scale=m.scale, window=m.window, value_mix=value_mix, value_key="first")
        if spec.type == "attention":
            position = None
            if m.rot is not None:
                ramp = None if m.rot.factor is None else FrequencyRamp(m.rot.factor, m.rot.original, m.rot.fast, m.rot.slow)
                position = RotaryPairs(m.dim, m.rot.base, rotary_dim=m.rot.dims, scaling=ramp)
            mixer = ScoredAttention(p + "mix.", W, m.heads, m.kv_heads, m.dim, m.vdim, position=position, biases=True,
                                    talk=True, head_bias=True, weights="sigmoid", head_gate=True, **common)
        else:
            mixer = ScoredAttention(p + "mix.", W, m.heads, m.kv_heads, m.dim, m.vdim, qk_norm_eps=eps,
                                    distance_bias=(m.bias_rows, m.bias_max), weights="softmax", **common)
        ff = [None, None, None]
        if spec.ff is not None:
            ff = [LayerNorm(p + "norm2", W, eps), SwiGLU(p + "mlp.", W, spec.ff, names=FF_NAMES), LayerNorm(p + "norm2b", W, eps)]
        layers.append(SandwichBlock(LayerNorm(p + "norm1", W, eps), mixer, LayerNorm(p + "norm1b", W, eps), *ff,
                                    mult=cfg.residual_mult, shift=TokenShift(p + "shift", W)))
    return DecoderModel(cfg, embedding, layers, LayerNorm("final.norm", W, eps), OutputHead("head", cfg.vocab, W, False, embedding))


register_architecture(LedudraConfig, build_ledudra)
