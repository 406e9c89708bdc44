"""Small Ledudra configurations for the tests: they differ in every size and option."""
import functools
import tempfile

import torch

import plain_ledudra as PL


def _att(heads, kv, dim, vdim, scale, window, v_mix, rot=None, ff=None):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale, v_mix=v_mix)
    if window:
        m["mask"] = dict(size=window)
    if rot:
        m["rot"] = rot
    return dict(type="attention", mixer=m, mlp=None if ff is None else dict(kind="dense", ff=ff))


def _att2(heads, kv, dim, vdim, scale, window, v_mix, rows, far, ff=None):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale, v_mix=v_mix, bias_max=far, bias_rows=rows)
    if window:
        m["mask"] = dict(size=window)
    return dict(type="attention_2", mixer=m, mlp=None if ff is None else dict(kind="dense", ff=ff))


def _yarn(dims, base, factor, original, fast, slow):
    return dict(dims=dims, base=base, scaling=dict(factor=factor, original=original, fast=fast, slow=slow))


# the sigmoid mixer first (so its values are the ones the others blend with), windows of 37, 70 and 9 positions (none a
# multiple or a divisor of a page), three query heads a kv head, a layer without feed-forward, a layer that does not
# blend, half of a head rotated with stretched frequencies, values larger than keys in one layer
LA = dict(architecture="Ledudra", vocab=101, width=48, norm=dict(eps=1e-5), residual_mult=0.7,
          layers=[_att(6, 2, 16, 12, 0.25, 37, True, _yarn(8, 1.0e4, 4.0, 64, 16.0, 2.0), ff=64),
                  _att2(4, 2, 8, 12, 0.35, 70, True, 10, 50, ff=None),
                  _att2(2, 1, 24, 20, 0.2, 9, False, 6, 7, ff=40),
                  _att(2, 2, 12, 12, 0.3, 70, True, dict(dims=12, base=500.0), ff=56)])
LA_INIT = dict(seed=3, std_matrix=0.12, std_embedding=0.7, std_gain=0.1, std_bias=0.25)

# no window in the first layer (every earlier key is seen) and none in the last, a window of one page, one head, no
# rotation in a sigmoid layer, nothing blended anywhere, residual_mult 1, a distance table of two rows
LB = dict(architecture="Ledudra", vocab=131, width=64, norm=dict(eps=1e-6), residual_mult=1.0,
          layers=[_att2(3, 3, 16, 16, 0.25, None, False, 2, 3, ff=96),
                  _att(1, 1, 32, 8, 0.15, 64, False, None, ff=72),
                  _att(4, 1, 8, 24, 0.4, None, False, _yarn(6, 100.0, 2.0, 16, 4.0, 1.0), ff=None)])
LB_INIT = dict(seed=7, std_matrix=0.1, std_embedding=0.6, std_gain=0.2, std_bias=0.3)

# head sizes of 64 for keys and values, four and eight query heads a kv head, a window of 130, a long distance table
LF = dict(architecture="Ledudra", vocab=203, width=128, norm=dict(eps=1e-5), residual_mult=0.6,
          layers=[_att2(4, 1, 64, 64, 0.125, 130, True, 32, 128, ff=256),
                  _att(8, 1, 64, 64, 0.11, 100, True, _yarn(32, 5.0e5, 6.0, 128, 24.0, 1.5), ff=128),
                  _att2(4, 1, 32, 64, 0.2, 200, True, 16, 100, ff=128)])
LF_INIT = dict(seed=11, std_matrix=0.06, std_embedding=0.5, std_gain=0.1, std_bias=0.3)

CONFIGS = {"LA": (LA, LA_INIT), "LB": (LB, LB_INIT), "LF": (LF, LF_INIT)}

_FOLDERS = {}


def folder(name: str) -> str:
    if name not in _FOLDERS:
        from synaptix_b200.config import LedudraConfig
        from synaptix_b200.weights import write_model_folder
        cfg_dict, init = CONFIGS[name]
        init = dict(init)
        _FOLDERS[name] = write_model_folder(LedudraConfig.from_dict(cfg_dict), tempfile.mkdtemp(prefix=f"sx_{name}_"),
                                            init.pop("seed"), **init)
    return _FOLDERS[name]


@functools.lru_cache(maxsize=None)
def oracle(name: str):
    return PL.load_folder(folder(name))


@functools.lru_cache(maxsize=256)
def oracle_logits(name: str, tokens: tuple) -> torch.Tensor:
    cfg, W = oracle(name)
    return PL.forward(cfg, W, list(tokens)).float()
