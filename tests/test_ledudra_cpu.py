"""The plain Ledudra implementation against other forms of the same equations, and the parts of the package that need
no GPU (configuration, tensor names, the tables made when weights are bound) against the plain implementation."""
import math

import pytest
import torch

import plain_ledudra as PL
from tiny_ledudra import CONFIGS, folder, oracle


def test_token_shift_is_a_blend_with_the_row_before():
    g = torch.Generator().manual_seed(0)
    h, s = torch.randn(6, 5, generator=g).double(), torch.rand(5, generator=g).double()
    out = PL.token_shift(h, s)
    assert torch.allclose(out[0], h[0] * (1 - s))
    for t in range(1, 6):
        assert torch.allclose(out[t], (1 - s) * h[t] + s * h[t - 1])


def test_layer_norm_has_zero_mean_and_unit_variance_before_gain_and_bias():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(4, 33, generator=g).double() * 3 + 2
    y = PL.layer_norm(x, torch.ones(33).double(), torch.zeros(33).double(), 0.0)
    assert torch.allclose(y.mean(-1), torch.zeros(4).double(), atol=1e-12)
    assert torch.allclose((y * y).mean(-1), torch.ones(4).double(), atol=1e-12)


def test_rotation_of_pairs_keeps_relative_angles():
    g = torch.Generator().manual_seed(2)
    q, k = torch.randn(1, 1, 12, generator=g).double(), torch.randn(1, 1, 12, generator=g).double()
    sc = dict(factor=4.0, original=64, fast=16.0, slow=2.0)
    dots = []
    for p in (0, 5, 40):
        a = PL.rotate_pairs(q, torch.tensor([p + 7]), 8, 1.0e4, sc)
        b = PL.rotate_pairs(k, torch.tensor([p]), 8, 1.0e4, sc)
        dots.append(float((a * b).sum()))
    assert abs(dots[0] - dots[1]) < 1e-9 and abs(dots[0] - dots[2]) < 1e-9
    _, mag = PL.scaled_frequencies(8, 1.0e4, sc)
    a = PL.rotate_pairs(q, torch.tensor([3]), 8, 1.0e4, sc)
    assert torch.allclose(a[..., 8:], q[..., 8:])                      # elements past rot.dims pass unchanged
    assert abs(float((a[..., :8] ** 2).sum()) - mag ** 2 * float((q[..., :8] ** 2).sum())) < 1e-9


def test_stretched_frequencies_of_the_package_equal_the_plain_ones():
    import numpy as np
    from synaptix_b200.parts import FrequencyRamp
    for dims, base, sc in [(8, 1.0e4, dict(factor=4.0, original=64, fast=16.0, slow=2.0)), (32, 5.0e5, dict(factor=6.0, original=128, fast=24.0, slow=1.5)),
                           (6, 100.0, dict(factor=2.0, original=16, fast=4.0, slow=1.0)), (64, 5.0e5, dict(factor=16.0, original=4096, fast=8.0, slow=0.5))]:
        ref, mag = PL.scaled_frequencies(dims, base, sc)
        ramp = FrequencyRamp(**sc)
        f = np.power(np.float64(base), -2.0 * np.arange(dims // 2) / dims)
        assert np.allclose(ramp.apply(f, base, dims), np.asarray(ref), rtol=1e-13, atol=0)
        assert ramp.magnitude() == mag
        assert any(a != b for a, b in zip(ref, f)) and ref[0] <= f[0]


def test_distance_buckets():
    for rows, far in [(16, 120), (10, 50), (2, 3), (6, 7), (32, 128), (8, 1000)]:
        b = [PL.distance_bucket(n, rows, far) for n in range(3 * int(far))]
        assert b[:rows // 2] == list(range(rows // 2))                 # one bucket a distance at first
        assert all(x <= y for x, y in zip(b, b[1:])) and b[-1] == rows - 1 and b[int(far)] == rows - 1
        from synaptix_b200.parts.scored import distance_columns
        for window in (None, 5, 70):
            cols = distance_columns(rows, far, window)
            upto = len(b) if window is None else min(window, len(b))
            assert all(cols[min(n, len(cols) - 1)] == b[n] for n in range(upto))


def test_mixing_with_the_identity_is_a_sigmoid_per_head():
    g = torch.Generator().manual_seed(3)
    T, H, G, D = 20, 4, 2, 6
    q, k, v = (torch.randn(T, n, D, generator=g).double() for n in (H, G, G))
    pos = torch.arange(T)
    got = PL.sigmoid_mixed_heads(q, k, v, pos, 0.3, torch.eye(H).double(), torch.zeros(H).double(), 7)
    for i in (0, 6, 7, 19):
        for h in range(H):
            want = sum(torch.sigmoid(0.3 * (q[i, h] @ k[j, h // 2])) * v[j, h // 2] for j in range(max(0, i - 6), i + 1))
            assert torch.allclose(got[i, h], want)


def test_softmax_with_a_zero_table_is_plain_windowed_attention():
    g = torch.Generator().manual_seed(4)
    T, H, D = 15, 2, 4
    q, k, v = (torch.randn(T, H, D, generator=g).double() for _ in range(3))
    got = PL.biased_softmax_heads(q, k, v, torch.arange(T), 0.5, torch.zeros(6, H).double(), 9, 4)
    i, h = 10, 1
    w = torch.softmax(torch.stack([0.5 * (q[i, h] @ k[j, h]) for j in range(7, 11)]), 0)
    assert torch.allclose(got[i, h], (w[:, None] * v[7:11, h]).sum(0))


@pytest.mark.parametrize("name", list(CONFIGS))
def test_configuration_round_trip_and_tensor_names(name):
    from synaptix_b200.config import LedudraConfig, load_config
    from synaptix_b200.models import model_skeleton
    cfg = load_config(folder(name))
    assert isinstance(cfg, LedudraConfig) and LedudraConfig.from_dict(cfg.to_dict()) == cfg
    specs = model_skeleton(cfg).all_tensor_specs()
    _, W = oracle(name)
    assert set(specs) == set(W)
    first = cfg.first_value_layer()
    for i, layer in enumerate(cfg.layers):
        assert (f"l{i}.mix.talk" in specs) == (layer.type == "attention")
        assert (f"l{i}.mix.rel" in specs) == (layer.type == "attention_2")
        assert (f"l{i}.norm2b.b" in specs) == (layer.ff is not None)
        assert (f"l{i}.mix.vmix" in specs) == layer.mixer.v_mix
    assert first is None or cfg.layers[first].mixer.v_mix


def test_configuration_errors():
    from synaptix_b200.config import ConfigError, LedudraConfig
    import copy
    base = CONFIGS["LA"][0]
    for change in (lambda d: d["layers"][0].__setitem__("type", "attention_3"),
                   lambda d: d["layers"][1]["mixer"].pop("bias_max"),
                   lambda d: d["layers"][0]["mixer"].__setitem__("heads", 5),
                   lambda d: d["layers"][0]["mixer"]["rot"].__setitem__("dims", 7),
                   lambda d: d["layers"][1]["mixer"].__setitem__("vdim", 8),       # blended values of another size
                   lambda d: d.pop("width")):
        d = copy.deepcopy(base)
        change(d)
        with pytest.raises(ConfigError):
            LedudraConfig.from_dict(d)
    d = copy.deepcopy(base)
    d["layers"][1]["mixer"].pop("bias_rows")                            # the table's size is then the tensor's own
    assert LedudraConfig.from_dict(d).layers[1].mixer.bias_rows is None
