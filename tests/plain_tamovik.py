"""A plain, slow implementation of the Tamovik decoder: one function per mechanism, written from the equations, whole
sequences only, float64 on the CPU.  It shares nothing with the package: it reads a configuration as the nested dict of
config.json and weights as a dict ``name -> tensor``.

Notation: ``x [T, W]`` the stream of ONE sequence, ``t`` a position (from 0), ``rms(v) = sqrt(mean(v^2) + eps)``.

    embedding     x_t = E[id_t] + B[(id_(t-1) a + id_t b) mod n]           (row n of B for t = 0)
    layer         x <- x + rms_norm(mixer(x)) g1 ;  x <- x + rms_norm(ff(x)) g2        (the sublayers read x itself)
    latent attn   c_t = rms_norm(Wd x_t)[:r] g, kr_t = rot(Wd x_t)[r:] ; head h: k = [Wuk_h c | kr], v = Wuv_h c,
                  q = [q_h | rot(qr_h)], softmax_j<=t (q . k_j scale), Wo over the heads
    rotation      rotate-half of the first d elements by angle t f_i, f_i stretched by a ramp, cos and sin times m
    left mixer    q, k = conv(Wq x), conv(Wk x); v = k; q, k <- rms_norm over ALL their channels; chunks; the heads'
                  results times sigmoid(Wg x); Wo
    right mixer   mLSTM: m_t = max(f + m_(t-1), i), S_t = e^(f + m_(t-1) - m_t) S_(t-1) + e^(i - m_t) k v^T, n_t alike,
                  o = S^T q / (max(|n . q|, e^(-m_t)) + 1e-6), per head o / rms(o), times gain, times sigmoid(Wg x), Wo
    parallel      (rms_norm(left) gl + rms_norm(right) gr) / 2
    dense ff      Wd (gelu_tanh(Wg x) * (Wu x))
    experts       s = sigmoid(Wr x); choice = s + b; groups keep the best by the sum of their two largest choices;
                  top-k of the choices inside kept groups; y = sum_e s_e expert_e(x)
"""
import json
import math
import os

import torch

F = torch.float64


def load_folder(path):
    from safetensors.torch import load_file
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    return cfg, {k: v.to(F) for k, v in load_file(os.path.join(path, "model.safetensors")).items()}


def rms_norm(x, gain, eps):
    x = x.to(F)
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * gain.to(F)


def unit_rms(x, eps):
    x = x.to(F)
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def embed(tokens, table, bigram, spec):
    """``table [vocab, W]``, ``bigram [buckets + 1, W]``; ``spec`` = {buckets, mul_cur, mul_prev}."""
    n = spec["buckets"]
    rows = []
    for t, tok in enumerate(tokens):
        row = n if t == 0 else (tokens[t - 1] * spec["mul_prev"] + tok * spec["mul_cur"]) % n
        rows.append(table[tok].to(F) + bigram[row].to(F))
    return torch.stack(rows)


def stretched_frequencies(rot):
    """Frequencies of the ``dims / 2`` pairs and the factor on cos and sin."""
    dims, base = rot["dims"], rot["base"]
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0

    def dim_of(turns):
        return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(sc["fast"])), 0)
    hi = min(math.ceil(dim_of(sc["slow"])), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / sc["factor"] * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(sc["factor"]) + 1.0


def rotate_half(v, pos, rot, angle_dtype=torch.float32):
    """``v [..., n]`` at position ``pos`` (a number, or one position per row of ``v [T, n]``): the first ``rot.dims``
    elements rotated, element i with i + dims/2.  The design forms positions and angles in 32-bit (``angle_dtype``): the
    frequency and the product ``pos * f_i`` are rounded to that type before the cosine and sine are taken."""
    if not rot:
        return v
    dims = rot["dims"]
    f, mag = stretched_frequencies(rot)
    half = dims // 2
    a = (torch.as_tensor(pos, dtype=angle_dtype)[..., None] * torch.tensor(f, dtype=angle_dtype)).to(F)          # [..., half]
    c, s = torch.cos(a) * mag, torch.sin(a) * mag
    u, w = v[..., :half], v[..., half:dims]
    return torch.cat([u * c - w * s, w * c + u * s, v[..., dims:]], dim=-1)


def latent_attention(x, w, p, m, eps):
    """``w``: name -> tensor, ``p``: the mixer's prefix, ``m``: its sizes."""
    T = x.shape[0]
    H, D, R, V, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m.get("rot")
    q = x @ w[p + "q"].to(F).T                                  # [T, H (D + R)]
    d = x @ w[p + "dkv"].to(F).T                                # [T, rank + R]
    c = rms_norm(d[:, :rank], w[p + "dkv.norm"], eps)
    kr = rotate_half(d[:, rank:], torch.arange(T), rot)
    uk, uv = w[p + "uk"].to(F), w[p + "uv"].to(F)
    heads = []
    for h in range(H):
        qh = q[:, h * (D + R):(h + 1) * (D + R)]
        qu = qh[:, :D]
        qr = rotate_half(qh[:, D:], torch.arange(T), rot)
        ku = c @ uk[h * D:(h + 1) * D].T                        # [T, D]
        vh = c @ uv[h * V:(h + 1) * V].T                        # [T, V]
        s = (qu @ ku.T + qr @ kr.T) * m["scale"]
        mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
        s = s.masked_fill(~mask, -math.inf)
        heads.append(torch.softmax(s, -1) @ vh)
    return torch.cat(heads, -1) @ w[p + "o"].to(F).T


def time_conv(u, taps):
    """``u [T, C]``, ``taps [C, n]``: ``y_t = sum_j taps[:, j] u_(t - n + 1 + j)``, zeros before the start."""
    T, C = u.shape
    n = taps.shape[1]
    taps = taps.to(F)
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(n):
            s = t - n + 1 + j
            if s >= 0:
                y[t] += taps[:, j] * u[s]
    return y


def chunked_attention(x, w, p, m, eps):
    T = x.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = time_conv(x @ w[p + "q"].to(F).T, w[p + "q.conv"])
    k = time_conv(x @ w[p + "k"].to(F).T, w[p + "k.conv"])
    v = k                                                        # values are the keys as they leave the convolution
    q = rms_norm(q, w[p + "q.norm"], eps)                        # over all heads' channels at once
    k = rms_norm(k, w[p + "k.norm"], eps)
    size = m["mask"]["size"] if m.get("mask") else None
    i = torch.arange(T)
    mask = i[None, :] <= i[:, None]
    if size:
        mask &= (i[None, :] // size) == (i[:, None] // size)
    heads = []
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h * D:(h + 1) * D] @ k[:, g * D:(g + 1) * D].T) * m["scale"]
        s = s.masked_fill(~mask, -math.inf)
        heads.append(torch.softmax(s, -1) @ v[:, g * V:(g + 1) * V])
    y = torch.cat(heads, -1) * torch.sigmoid(x @ w[p + "g"].to(F).T)
    return y @ w[p + "o"].to(F).T


def matrix_memory(x, w, p, m, eps):
    T = x.shape[0]
    H, D, V, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (x @ w[p + "q"].to(F).T) * D ** -0.5
    k = x @ w[p + "k"].to(F).T
    v = x @ w[p + "v"].to(F).T
    zi = x @ w[p + "i"].to(F).T + w[p + "i.b"].to(F)
    zf = x @ w[p + "f"].to(F).T + w[p + "f.b"].to(F)
    gi = cap * torch.tanh(zi / cap)
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh(zf / cap))
    out = torch.zeros(T, H * V, dtype=F)
    for h in range(H):
        S = torch.zeros(D, V, dtype=F)
        n = torch.zeros(D, dtype=F)
        mx = 0.0
        for t in range(T):
            i_t, f_t = float(gi[t, h]), float(gf[t, h])
            m_new = max(f_t + mx, i_t)
            kt, vt, qt = k[t, h * D:(h + 1) * D], v[t, h * V:(h + 1) * V], q[t, h * D:(h + 1) * D]
            S = math.exp(f_t + mx - m_new) * S + math.exp(i_t - m_new) * torch.outer(kt, vt)
            n = math.exp(f_t + mx - m_new) * n + math.exp(i_t - m_new) * kt
            mx = m_new
            den = max(abs(float(n @ qt)), math.exp(-mx)) + 1e-6
            out[t, h * V:(h + 1) * V] = unit_rms(S.T @ qt / den, eps)
    y = out * w[p + "norm"].to(F) * torch.sigmoid(x @ w[p + "g"].to(F).T)
    return y @ w[p + "o"].to(F).T


def parallel_mixer(x, w, p, m, eps):
    a = rms_norm(chunked_attention(x, w, p + "left.", m["left"], eps), w[p + "left.out"], eps)
    b = rms_norm(matrix_memory(x, w, p + "right.", m["right"], eps), w[p + "right.out"], eps)
    return 0.5 * (a + b)


def dense_ff(x, w, p):
    return (gelu_tanh(x @ w[p + "gate"].to(F).T) * (x @ w[p + "up"].to(F).T)) @ w[p + "down"].to(F).T


def choose_experts(choice, top, groups):
    """``choice [E]`` -> the indices of the chosen experts (of equal values the lower index first)."""
    E = choice.shape[0]
    allowed = [True] * E
    if groups:
        n, keep = groups["count"], groups["keep"]
        size = E // n
        score = []
        for g in range(n):
            vals = sorted((float(v) for v in choice[g * size:(g + 1) * size]), reverse=True)
            score.append(sum(vals[:2]))
        best = sorted(range(n), key=lambda g: (-score[g], g))[:keep]
        allowed = [(e // size) in best for e in range(E)]
    order = sorted((e for e in range(E) if allowed[e]), key=lambda e: (-float(choice[e]), e))
    return order[:top]


def expert_ff(x, w, p, limit):
    g = torch.clamp(x @ w[p + "gate"].to(F).T, max=limit)
    u = torch.clamp(x @ w[p + "up"].to(F).T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].to(F).T


def experts_ff(x, w, p, spec):
    r = spec["router"]
    s = torch.sigmoid(x @ w[p + "router"].to(F).T)                # [T, E]
    choice = s + w[p + "correction"].to(F)
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for e in choose_experts(choice[t], r["top"], r.get("groups")):
            out[t] += s[t, e] * expert_ff(x[t:t + 1], w, f"{p}e{e}.", spec["expert"]["limit"])[0]
    return out


def forward(cfg, w, tokens, layers_out=None, read=None):
    """Logits float64 ``[T, vocab]`` of one sequence; ``layers_out`` (a list) takes the stream after every layer.
    ``read``: a function applied to the stream where a sublayer reads it (say, a rounding to 16 bits: how far the result
    moves under it tells how well-conditioned an input is)."""
    eps = cfg["norm"]["eps"]
    read = read or (lambda v: v)
    x = embed(list(tokens), w["embed"], w["bigram"], cfg["embedding"]["bigram"])
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        if layer["type"] == "latent_attention":
            a = latent_attention(read(x), w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "parallel":
            a = parallel_mixer(read(x), w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(a, w[p + "norm1"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            b = dense_ff(read(x), w, p + "mlp.") if mlp["kind"] == "dense" else experts_ff(read(x), w, p + "mlp.", mlp)
            x = x + rms_norm(b, w[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].to(F).T
