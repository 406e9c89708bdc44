"""Small Tamovik configurations for the tests: they differ in every size and option."""
import functools
import tempfile

import torch

import plain_tamovik as PT


def _lat(heads, dim, rot_dim, vdim, kv_rank, scale, rot, mlp):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, scale=scale)
    if rot:
        m["rot"] = dict(dims=rot[0], base=rot[1])
        if len(rot) > 2:
            m["rot"]["scaling"] = dict(factor=rot[2], original=rot[3], fast=rot[4], slow=rot[5])
    return dict(type="latent_attention", mixer=m, mlp=mlp)


def _par(heads, kv_heads, dim, conv, scale, chunk, mheads, mdim, mvdim, cap, mlp):
    left = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, conv=conv, scale=scale)
    if chunk:
        left["mask"] = dict(size=chunk)
    return dict(type="parallel", mixer=dict(left=left, right=dict(heads=mheads, dim=mdim, vdim=mvdim, gate_cap=cap)), mlp=mlp)


def _dense(ff):
    return dict(kind="dense", ff=ff)


def _moe(ff, limit, experts, top, groups=None):
    router = dict(experts=experts, top=top)
    if groups:
        router["groups"] = dict(count=groups[0], keep=groups[1])
    return dict(kind="moe", expert=dict(ff=ff, limit=limit), router=router)


def _cfg(vocab, width, eps, buckets, mul_prev, mul_cur, layers):
    return dict(architecture="Tamovik", vocab=vocab, width=width, norm=dict(eps=eps),
                embedding=dict(bigram=dict(buckets=buckets, mul_prev=mul_prev, mul_cur=mul_cur)), layers=layers)


# a parallel layer first, odd sizes no fast product takes, chunks of 23 (shorter than a page), 4 taps, one kv head, groups
# of ONE expert each (a group's value is its expert's), a layer without feed-forward, rotation without stretching,
# every expert chosen (top = experts), a latent layer whose rot.dims is less than rot_dim
TA = _cfg(101, 52, 1e-5, 37, 5, 3,
          [_par(3, 1, 12, 4, 0.3, 23, 2, 12, 20, 6.0, _moe(24, 1.25, 6, 2, (6, 3))),
           _lat(3, 12, 8, 10, 28, 0.3, (8, 1.0e4), _dense(72)),
           _lat(2, 6, 12, 14, 20, 0.45, (8, 500.0, 4.0, 40, 8.0, 1.0), None),
           _par(4, 4, 8, 2, 0.35, 70, 1, 16, 8, 15.0, _moe(40, 0.75, 3, 3)),
           _lat(5, 4, 8, 6, 36, 0.25, None, _moe(8, 2.0, 9, 3, (3, 2)))])
TA_INIT = dict(seed=5, std_matrix=0.12, std_embedding=0.5, std_gain=0.2, std_bias=0.5)

# latent layers first, chunks of one page and one token (65) and of 1 (a token sees itself alone), one tap (no
# convolution), nine attention heads, a dense feed-forward beside experts, groups of which all are kept, multipliers
# whose products pass 32 bits of a hash only with 64-bit arithmetic
TB = _cfg(77, 64, 1e-6, 211, 40009, 59999,
          [_lat(9, 8, 12, 8, 36, 0.2, (12, 5.0e5, 2.0, 64, 16.0, 2.0), _moe(48, 1.5, 4, 2, (2, 2))),
           _lat(1, 16, 4, 32, 24, 0.35, (4, 100.0), _dense(40)),
           _par(2, 1, 24, 1, 0.2, 65, 4, 8, 8, 9.0, _dense(96)),
           _par(6, 3, 8, 3, 0.4, 1, 2, 24, 12, 11.0, None),
           _par(2, 2, 16, 5, 0.25, None, 1, 8, 40, 12.0, _moe(16, 1.0, 8, 1, (4, 1)))])
TB_INIT = dict(seed=9, std_matrix=0.1, std_embedding=0.7, std_gain=0.15, std_bias=0.4)

# sizes the fast bfloat16 products and the tensor-core attention kernels take: attention heads of 64 with chunks of 100,
# latent heads whose dim + rot_dim equals vdim (64 and 128), so that whole prompts of 256 tokens and more run over
# per-head keys and values; memory heads of 64 x 32
TF = _cfg(256, 128, 1e-5, 251, 13, 7,
          [_lat(4, 32, 32, 64, 64, 0.11, (32, 2.0e5, 3.0, 128, 16.0, 2.0), _dense(256)),
           _par(4, 2, 64, 3, 0.12, 100, 2, 64, 32, 10.0, _moe(64, 1.75, 8, 2, (4, 2))),
           _lat(2, 96, 32, 128, 64, 0.09, (32, 3.0e5), _moe(64, 2.5, 8, 2, (2, 1))),
           _par(2, 2, 128, 3, 0.09, 200, 4, 32, 64, 8.0, _moe(96, 1.25, 4, 3)),
           _par(8, 2, 32, 2, 0.18, None, 2, 32, 32, 14.0, _dense(128))])
TF_INIT = dict(seed=13, std_matrix=0.08, std_embedding=0.4, std_gain=0.1, std_bias=0.3)

# attention WITHOUT chunks at head sizes 128 and 64 (the library's plain attention kernels: tcgen05 for prompts, pages by
# TMA for single tokens, with values read from pages of their own that hold the unnormed keys), four taps, a latent layer
# between them whose whole prompts run over per-head keys of 128, experts in groups of four of which one is kept
TG = _cfg(300, 256, 1e-5, 127, 3, 11,
          [_par(4, 2, 128, 4, 0.09, None, 2, 64, 64, 12.0, _dense(512)),
           _lat(2, 64, 64, 128, 64, 0.09, (64, 1.0e5, 2.0, 256, 32.0, 1.0), _moe(128, 1.5, 8, 2, (2, 1))),
           _par(4, 1, 64, 2, 0.125, None, 1, 128, 128, 15.0, _moe(64, 2.0, 4, 1))])
TG_INIT = dict(seed=21, std_matrix=0.06, std_embedding=0.4, std_gain=0.1, std_bias=0.3)

CONFIGS = {"TA": (TA, TA_INIT), "TB": (TB, TB_INIT), "TF": (TF, TF_INIT), "TG": (TG, TG_INIT)}

_FOLDERS = {}


def folder(name: str) -> str:
    if name not in _FOLDERS:
        from synaptix_b200.config import TamovikConfig
        from synaptix_b200.weights import write_model_folder
        cfg_dict, init = CONFIGS[name]
        init = dict(init)
        _FOLDERS[name] = write_model_folder(TamovikConfig.from_dict(cfg_dict), tempfile.mkdtemp(prefix=f"sx_{name}_"),
                                            init.pop("seed"), **init)
    return _FOLDERS[name]


@functools.lru_cache(maxsize=None)
def oracle(name: str):
    return PT.load_folder(folder(name))


def _to_bf16(v):
    return v.to(torch.bfloat16).to(torch.float64)


@functools.lru_cache(maxsize=256)
def oracle_logits(name: str, tokens: tuple, dtype: str = "float32") -> torch.Tensor:
    """``dtype="bfloat16"``: the sublayers read the stream rounded to 16 bits, as the library's bfloat16 path has it;
    everything else stays 64-bit."""
    cfg, W = oracle(name)
    return PT.forward(cfg, W, list(tokens), read=_to_bf16 if dtype == "bfloat16" else None).float()


@functools.lru_cache(maxsize=None)
def steady_first_tokens(name: str) -> tuple:
    """Tokens that may begin a test's sequence.  With a single token behind it a matrix memory's normed output is
    ``sign(q . k) v / rms(v)``: where ``q . k`` is nearly zero, any rounding of the layer's input flips the head's output
    (and everything behind it, in models this small).  Such a first token says nothing about a kernel, so the tests
    begin their sequences with tokens whose logits move little when the sublayers read the stream rounded to 16 bits."""
    cfg, W = oracle(name)
    good = []
    for t in range(cfg["vocab"]):
        a = PT.forward(cfg, W, [t])
        b = PT.forward(cfg, W, [t], read=lambda v: v.to(torch.bfloat16).to(torch.float64))
        if float((a - b).abs().max()) <= 0.01 * float(a.abs().max()):
            good.append(t)
        if len(good) == 12:
            break
    assert len(good) >= 4, name
    return tuple(good)


@functools.lru_cache(maxsize=None)
def _steady_tokens(name: str, n: int, seed: int) -> tuple:
    from tiny import random_tokens
    good = steady_first_tokens(name)
    toks = None
    for attempt in range(8):
        toks = random_tokens(CONFIGS[name][0]["vocab"], n, seed + 1000 * attempt)
        toks[0] = good[seed % len(good)]
        a, b = oracle_logits(name, tuple(toks)), oracle_logits(name, tuple(toks), "bfloat16")
        rel = (a - b).abs().max(dim=1).values / a.abs().max()
        if float(rel.median()) <= 0.01 and float((rel <= 0.03).float().mean()) >= 0.9:
            break
    return tuple(toks)


def tokens(name: str, n: int, seed: int) -> list:
    """``n`` random tokens for a test's sequence: the first one from ``steady_first_tokens``, and the whole sequence one
    on which the plain implementation itself moves little when its sublayers read the stream rounded to 16 bits.  (On
    some sequences an early near tie, a router's choice between two experts, decides differently under any rounding,
    and every later row that reads that token's keys, values or state moves with it: such a sequence measures the tie,
    not a kernel.)"""
    return list(_steady_tokens(name, n, seed))
