"""Shape lists and seeded input generation shared by make_golden.py (which stores aten's outputs for them) and the
tests (which regenerate the same inputs). Inputs come from numpy's PCG64 (`default_rng(seed)`), which is stable across
platforms and numpy versions, so only expected outputs need to be stored."""
import numpy as np
import torch

# (ci, co, ks, groups) at n=4, 14x14, "same" padding -- notes/scripts/conv_kinds_check.py:5
CONV_KINDS = [(8, 8, 5, 8), (8, 8, 7, 8), (8, 8, 3, 8), (6, 10, 5, 1), (6, 10, 3, 1), (6, 10, 1, 1)]
# (ci, co, ks, stride, pad, hw) at n=3 with bias -- notes/scripts/alexnet_ops_check.py:6
CONV_STRIDED = [(3, 8, 11, 4, 2, 63), (4, 6, 5, 1, 2, 17), (3, 6, 3, 2, 1, 15), (4, 6, 1, 1, 0, 9), (6, 10, 3, 1, 0, 12), (5, 7, 5, 2, 0, 21)]
# (k, s, p, hw) at [2,4,hw,hw] -- notes/scripts/alexnet_ops_check.py:12
MAXPOOL = [(3, 2, 0, 13), (3, 2, 0, 27), (3, 2, 1, 14), (3, 1, 1, 9), (2, 2, 0, 12), (5, 3, 2, 17)]
# (hw, out) at [2,5,hw,hw] -- notes/scripts/alexnet_ops_check.py:16
ADAPOOL = [(6, 6), (13, 6), (10, 4), (7, 1)]
# extra depthwise strides/pads the general depthwise kernels cover (csrc/conv.cpp:175: any ks<=11, stride<=4, pad<=ks)
DW_GENERAL = [(8, 3, 2, 1, 15), (8, 5, 2, 2, 17), (6, 3, 1, 0, 9), (4, 7, 3, 3, 21), (4, 4, 2, 1, 12)]  # (c, ks, s, p, hw)
# BN cases: (n, c, h, w)
BN = [(4, 6, 5, 7), (16, 8, 4, 4), (2, 3, 1, 9)]


def rnd(seed, *shape, scale=1.0):
    return torch.from_numpy((np.random.default_rng(seed).standard_normal(shape) * scale).astype(np.float32))


def conv_inputs(seed, n, ci, co, ks, stride, pad, hw, groups, bias):
    """x, w, b, gy for one conv case (the layout make_golden.py's conv_case uses)."""
    x = rnd(seed, n, ci, hw, hw)
    w = rnd(seed + 1, co, ci // groups, ks, ks, scale=0.2)
    b = rnd(seed + 2, co) if bias else None
    oh = (hw + 2 * pad - ks) // stride + 1
    gy = rnd(seed + 3, n, co, oh, oh)
    return x, w, b, gy


def conv_cases():
    """name -> (seed, n, ci, co, ks, stride, pad, hw, groups, bias) for every conv fixture in ops.npz."""
    out = {}
    for i, (ci, co, ks, groups) in enumerate(CONV_KINDS):
        out[f"kinds{i}"] = (100 + 10 * i, 4, ci, co, ks, 1, ks // 2, 14, groups, False)
    for i, (ci, co, ks, s, p, hw) in enumerate(CONV_STRIDED):
        out[f"strided{i}"] = (300 + 10 * i, 3, ci, co, ks, s, p, hw, 1, True)
    for i, (c, ks, s, p, hw) in enumerate(DW_GENERAL):
        out[f"dwgen{i}"] = (500 + 10 * i, 2, c, c, ks, s, p, hw, c, True)
    return out
