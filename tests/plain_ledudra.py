"""A plain, slow implementation of the Ledudra decoder on the CPU: one function per mechanism, straight from the
equations, whole sequences only, no cache and no batching.  It shares nothing with the package (it reads model
folders with the ``safetensors`` package) and is what the GPU tests compare the engine with.

Notation: ``x`` is the residual stream ``[T, width]``, ``h`` what a sublayer reads, positions count from 0.
"""
import json
import math
import os

import torch


def load_folder(path, dtype=torch.float64):
    from safetensors.torch import load_file
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in load_file(os.path.join(path, "model.safetensors")).items()}
    return cfg, W


def layer_norm(x, w, b, eps):
    """(x - mean) / sqrt(var + eps) * w + b over the last axis, var = mean of the squared deviations."""
    mu = x.mean(dim=-1, keepdim=True)
    d = x - mu
    return d / torch.sqrt((d * d).mean(dim=-1, keepdim=True) + eps) * w + b


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def token_shift(h, s):
    """h_t + (h_(t-1) - h_t) * s with h_(-1) = 0; h_(t-1) is the row before the replacement."""
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)
    return h + (prev - h) * s


def scaled_frequencies(dims, base, scaling):
    """f_i = base^(-2i/dims), i < dims/2; with ``scaling`` (factor, original, fast, slow) the blend of f_i and f_i / factor
    by a ramp over i, and the factor ``0.1 ln(factor) + 1`` on cos and sin.  Returns (frequencies, magnitude)."""
    n = dims // 2
    f = [base ** (-2.0 * i / dims) for i in range(n)]
    if not scaling:
        return f, 1.0
    factor, original = scaling["factor"], scaling["original"]

    def dim_of(t):
        return dims * math.log(original / (2 * math.pi * t)) / (2 * math.log(base))
    lo = max(math.floor(dim_of(scaling["fast"])), 0)
    hi = min(math.ceil(dim_of(scaling["slow"])), dims - 1)
    out = []
    for i in range(n):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f[i] / factor * ramp + f[i] * (1 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_pairs(x, pos, dims, base, scaling=None):
    """x [T, heads, dim]: element 2i of the first ``dims`` paired with 2i + 1, rotated by pos * f_i."""
    f, mag = scaled_frequencies(dims, base, scaling)
    a = pos.to(x.dtype)[:, None] * torch.tensor(f, dtype=x.dtype)[None, :]
    c, s = (torch.cos(a) * mag)[:, None, :], (torch.sin(a) * mag)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def visible(pos, window):
    d = pos[:, None] - pos[None, :]
    see = d >= 0
    if window is not None:
        see = see & (d < window)
    return see, d


def distance_bucket(n, B, D):
    """n for n < B/2, else min(B - 1, B/2 + floor(ln(n / (B/2)) / ln(D / (B/2)) * (B - B/2)))."""
    half = B // 2
    if n < half:
        return n
    return min(B - 1, half + int(math.floor(math.log(n / half) / math.log(D / half) * (B - half))))


def sigmoid_mixed_heads(q, k, v, pos, scale, talk, pb, window):
    """q [T, H, D], k [T, G, D], v [T, G, Dv]: scores of all heads, mixed over heads by ``talk [H, H]``, weight of a
    visible key sigmoid(mixed + pb_h), no normalisation.  Returns [T, H, Dv]."""
    T, H = q.shape[0], q.shape[1]
    G = k.shape[1]
    see, _ = visible(pos, window)
    s = torch.stack([(q[:, h] @ k[:, h // (H // G)].T) * scale for h in range(H)])      # [H, T, T]
    s = torch.einsum("hg,gij->hij", talk, s)
    w = torch.sigmoid(s + pb[:, None, None]) * see[None].to(q.dtype)
    return torch.stack([w[h] @ v[:, h // (H // G)] for h in range(H)], dim=1)


def biased_softmax_heads(q, k, v, pos, scale, rel, bias_max, window):
    """Softmax attention with rel[bucket(i - j), h] added to the scaled score."""
    T, H = q.shape[0], q.shape[1]
    G = k.shape[1]
    see, d = visible(pos, window)
    B = rel.shape[0]
    bucket = torch.tensor([[distance_bucket(int(n), B, bias_max) if n >= 0 else 0 for n in row] for row in d.tolist()])
    out = []
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale + rel[:, h][bucket]
        s = s.masked_fill(~see, float("-inf"))
        out.append(torch.softmax(s, dim=-1) @ v[:, g])
    return torch.stack(out, dim=1)


def mix_values(v, v_first, lam):
    return (1 - lam) * v + lam * v_first


def attention(h, W, p, m, pos, v_first):
    """The mixer 'attention'.  Returns (output, this layer's values before they are cached)."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T + W[p + "q.b"]).view(T, H, D)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).view(T, G, D)
    v = (h @ W[p + "v"].T + W[p + "v.b"]).view(T, G, Dv)
    rot = m.get("rot")
    if rot:
        q = rotate_pairs(q, pos, rot["dims"], rot["base"], rot.get("scaling"))
        k = rotate_pairs(k, pos, rot["dims"], rot["base"], rot.get("scaling"))
    if m.get("v_mix") and v_first is not None:
        v = mix_values(v, v_first, W[p + "vmix"])
    window = (m.get("mask") or {}).get("size")
    o = sigmoid_mixed_heads(q, k, v, pos, m["scale"], W[p + "talk"], W[p + "pb"], window)
    gate = torch.sigmoid(h @ W[p + "g"].T)                    # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(T, H * Dv) @ W[p + "o"].T + W[p + "o.b"], v


def attention_2(h, W, p, m, pos, v_first, eps):
    """The mixer 'attention_2'."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_unit((h @ W[p + "q"].T).view(T, H, D), eps) * W[p + "q.norm"]
    k = rms_unit((h @ W[p + "k"].T).view(T, G, D), eps) * W[p + "k.norm"]
    v = (h @ W[p + "v"].T).view(T, G, Dv)
    if m.get("v_mix") and v_first is not None:
        v = mix_values(v, v_first, W[p + "vmix"])
    window = (m.get("mask") or {}).get("size")
    o = biased_softmax_heads(q, k, v, pos, m["scale"], W[p + "rel"], m["bias_max"], window)
    return o.reshape(T, H * Dv) @ W[p + "o"].T, v


def swiglu(h, W, p):
    return (torch.nn.functional.silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def forward(cfg, W, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence (and the stream after every layer)."""
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    tok = torch.tensor(tokens, dtype=torch.long)
    pos = torch.arange(len(tokens))
    x = W["embed"][tok]
    v_first = None
    streams = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        h = layer_norm(x, W[p + "norm1"], W[p + "norm1.b"], eps)
        h = token_shift(h, W[p + "shift"])
        if layer["type"] == "attention":
            y, v = attention(h, W, p + "mix.", m, pos, v_first)
        elif layer["type"] == "attention_2":
            y, v = attention_2(h, W, p + "mix.", m, pos, v_first, eps)
        else:
            raise ValueError(layer["type"])
        if m.get("v_mix") and v_first is None:
            v_first = v
        x = x + mult * layer_norm(y, W[p + "norm1b"], W[p + "norm1b.b"], eps)
        if layer.get("mlp") is not None:
            h = layer_norm(x, W[p + "norm2"], W[p + "norm2.b"], eps)
            x = x + mult * layer_norm(swiglu(h, W, p + "mlp."), W[p + "norm2b"], W[p + "norm2b.b"], eps)
        streams.append(x)
    logits = layer_norm(x, W["final.norm"], W["final.norm.b"], eps) @ W["head"].T
    return (logits, streams) if return_layers else logits
