"""What needs no GPU of the Tamovik decoder: its configuration, the model as data (tensor names, cache requests), and
the plain implementation against other forms of its own equations."""
import copy
import math

import pytest
import torch

import plain_tamovik as PT
from tiny_tamovik import CONFIGS

F = torch.float64


def cfg_of(name):
    from synaptix_b200.config import TamovikConfig
    return TamovikConfig.from_dict(CONFIGS[name][0])


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_configuration_round_trip_and_registry(name):
    from synaptix_b200.config import TamovikConfig, resolve_architecture
    d = CONFIGS[name][0]
    cfg = cfg_of(name)
    assert TamovikConfig.from_dict(cfg.to_dict()) == cfg and cfg.to_dict() == d
    assert resolve_architecture(d).config_cls is TamovikConfig
    assert [l.type for l in cfg.layers] == [l["type"] for l in d["layers"]]
    assert cfg.bigram_buckets == d["embedding"]["bigram"]["buckets"]


def test_configuration_errors():
    from synaptix_b200.config import ConfigError, TamovikConfig
    base = CONFIGS["TA"][0]

    def broken(change):
        d = copy.deepcopy(base)
        change(d)
        with pytest.raises(ConfigError):
            TamovikConfig.from_dict(d)
    broken(lambda d: d["embedding"]["bigram"].pop("mul_prev"))
    broken(lambda d: d["layers"][0].update(type="other"))
    broken(lambda d: d["layers"][1]["mlp"].update(kind="other"))
    broken(lambda d: d["layers"][0]["mlp"]["router"].update(top=4))                   # more than the kept groups hold
    broken(lambda d: d["layers"][0]["mlp"]["router"]["groups"].update(count=4))       # 6 experts in 4 groups
    broken(lambda d: d["layers"][0]["mlp"]["expert"].pop("limit"))
    broken(lambda d: d["layers"][0]["mixer"]["left"].update(vdim=10))                 # the values are the keys
    broken(lambda d: d["layers"][0]["mixer"]["left"].update(kv_heads=2))              # 3 heads over 2
    broken(lambda d: d["layers"][0]["mixer"]["right"].pop("gate_cap"))
    broken(lambda d: d["layers"][1]["mixer"]["rot"].update(dims=10))                  # more than rot_dim
    broken(lambda d: d["layers"][2]["mixer"]["rot"]["scaling"].pop("fast"))
    broken(lambda d: d.update(layers=[]))


def test_model_as_data():
    from synaptix_b200.cache.store import BundleRequest, KVRequest, StateRequest
    from synaptix_b200.models import model_skeleton
    m = model_skeleton(cfg_of("TA"))
    reqs = m.cache_requests()
    assert len(reqs) == 6 and reqs[-1] == StateRequest((), torch.int32)      # the embedding's token before, behind the layers
    assert reqs[1] == KVRequest(1, 28 + 8, None, keys_only=True)
    left, right = reqs[0].items
    assert left.items[0] == KVRequest(1, 12, None, None, 23) and left.items[1] == StateRequest((3, 36 + 12), torch.float32)
    assert [tuple(i.shape) for i in right.items] == [(2, 12, 20), (2, 12), (2,)]
    specs = m.all_tensor_specs()
    assert tuple(specs["bigram"].shape) == (38, 52) and tuple(specs["l0.mix.left.q.conv"].shape) == (36, 4)
    assert "l2.norm2" not in specs and "l0.mlp.correction" in specs and "l1.mlp.gate" in specs and "l1.mix.q" in specs
    assert "l0.mix.left.v" not in specs and tuple(specs["l0.mix.left.out"].shape) == (52,)
    assert "l1.mix.dq" not in specs and "l1.mix.g" not in specs


def test_convolution_against_its_matrix_form():
    g = torch.Generator().manual_seed(1)
    u, taps = torch.randn(9, 5, generator=g).double(), torch.randn(5, 4, generator=g).double()
    y = PT.time_conv(u, taps)
    for c in range(5):
        M = torch.zeros(9, 9, dtype=F)
        for t in range(9):
            for j in range(4):
                if t - 3 + j >= 0:
                    M[t, t - 3 + j] = taps[c, j]
        assert torch.allclose(y[:, c], M @ u[:, c])
    assert torch.allclose(PT.time_conv(u, torch.ones(5, 1, dtype=F)), u)            # one tap: no convolution


def test_matrix_memory_against_the_sum_over_the_past():
    """The recurrence with its running maximum equals the closed sum ``sum_j exp(i_j + sum_(l>j) f_l) k_j v_j^T`` scaled
    by ``exp(-m_t)``, with ``m_t = max(sum_l f_l, max_j (i_j + sum_(l>j) f_l))`` (the maximum starts at 0)."""
    g = torch.Generator().manual_seed(2)
    T, K, D, V = 12, 6, 4, 5
    m = dict(heads=1, dim=D, vdim=V, gate_cap=7.0)
    W = {"p." + n: torch.randn(*s, generator=g).double() for n, s in
         [("q", (D, K)), ("k", (D, K)), ("v", (V, K)), ("g", (V, K)), ("i", (1, K)), ("f", (1, K)), ("i.b", (1,)), ("f.b", (1,))]}
    W["p.norm"], W["p.o"] = torch.ones(V, dtype=F), torch.eye(V, dtype=F)
    x = torch.randn(T, K, generator=g).double()
    got = PT.matrix_memory(x, W, "p.", m, 1e-6)
    gi = 7.0 * torch.tanh((x @ W["p.i"].T + W["p.i.b"]) / 7.0)[:, 0]
    gf = torch.nn.functional.logsigmoid(7.0 * torch.tanh((x @ W["p.f"].T + W["p.f.b"]) / 7.0))[:, 0]
    q, k, v = (x @ W["p.q"].T) * D ** -0.5, x @ W["p.k"].T, x @ W["p.v"].T
    for t in range(T):
        logw = torch.stack([gi[j] + gf[j + 1:t + 1].sum() for j in range(t + 1)])
        mt = max(float(gf[:t + 1].sum()), float(logw.max()))
        wgt = torch.exp(logw - mt)
        num = sum(wgt[j] * (q[t] @ k[j]) * v[j] for j in range(t + 1))
        den = max(abs(float(sum(wgt[j] * (q[t] @ k[j]) for j in range(t + 1)))), math.exp(-mt)) + 1e-6
        o = PT.unit_rms(num / den, 1e-6) * torch.sigmoid(x[t] @ W["p.g"].T)
        assert torch.allclose(got[t], o, atol=1e-9)


def test_groups_and_choice():
    c = torch.tensor([0.9, 0.1, 0.5, 0.5, 0.2, 0.8, -0.3, -0.2], dtype=F)
    assert PT.choose_experts(c, 3, None) == [0, 5, 2]                                 # of equal values the lower index
    # groups of two: values 1.0, 1.0, 1.0, -0.5: of equal groups the lower ones stay
    assert PT.choose_experts(c, 2, dict(count=4, keep=2)) == [0, 2]
    assert PT.choose_experts(c, 2, dict(count=4, keep=3)) == [0, 5]
    # negative choices inside a kept group still beat everything outside of it
    c = torch.tensor([-0.5, -0.6, 0.4, -9.0, 0.3, -9.0], dtype=F)
    assert PT.choose_experts(c, 2, dict(count=3, keep=1)) == [0, 1]
    assert PT.choose_experts(c, 2, dict(count=6, keep=2)) == [2, 4]                   # groups of one expert


def test_rotation_keeps_relative_angles_and_scales_by_its_factor():
    g = torch.Generator().manual_seed(3)
    rot = dict(dims=8, base=500.0, scaling=dict(factor=4.0, original=40, fast=8.0, slow=1.0))
    f, mag = PT.stretched_frequencies(rot)
    plain_f, _ = PT.stretched_frequencies(dict(dims=8, base=500.0))
    assert mag == pytest.approx(0.1 * math.log(4.0) + 1.0)
    assert f[0] == pytest.approx(plain_f[0]) and f[-1] == pytest.approx(plain_f[-1] / 4.0)       # fast pairs stay, slow ones stretch
    a, b = torch.randn(12, generator=g).double(), torch.randn(12, generator=g).double()
    d1 = PT.rotate_half(a, 7, rot, F) @ PT.rotate_half(b, 3, rot, F)
    d2 = PT.rotate_half(a, 107, rot, F) @ PT.rotate_half(b, 103, rot, F)
    assert float(d1) == pytest.approx(float(d2), abs=1e-9)
    d3 = PT.rotate_half(a, 107, rot) @ PT.rotate_half(b, 103, rot)                  # angles rounded to 32 bits, as the design has them
    assert float(d3) == pytest.approx(float(d1), abs=1e-4) and float(d3) != float(d2)
    assert float(PT.rotate_half(a, 5, rot)[:8].norm()) == pytest.approx(mag * float(a[:8].norm()))
    assert torch.equal(PT.rotate_half(a, 5, rot)[8:], a[8:])


def test_first_token_and_hash_of_the_embedding():
    table, big = torch.arange(20, dtype=F).reshape(10, 2), 100 + torch.arange(12, dtype=F).reshape(6, 2)
    spec = dict(buckets=5, mul_prev=7, mul_cur=3)
    x = PT.embed([4, 9, 9], table, big, spec)
    assert torch.equal(x[0], table[4] + big[5])
    assert torch.equal(x[1], table[9] + big[(4 * 7 + 9 * 3) % 5]) and torch.equal(x[2], table[9] + big[(9 * 7 + 9 * 3) % 5])
