"""Pins the CPU oracle (oracle/oracle.c) to the golden fixtures: aten-CPU outputs on the reference's own shape lists
(tests/golden/make_golden.py). Runs without a GPU."""
import numpy as np
import pytest
import torch

import cases
import oracle
from conftest import TOL, rel_err

CONV = cases.conv_cases()


@pytest.mark.parametrize("name", sorted(CONV))
def test_conv_cases_match_aten(name, golden):
    seed, n, ci, co, ks, s, p, hw, groups, bias = CONV[name]
    x, w, b, gy = (t.numpy() if t is not None else None for t in cases.conv_inputs(*CONV[name]))
    if groups == 1:
        y = oracle.c.conv_fwd(x, w, b, s, p)
        dx = oracle.c.conv_dgrad(gy, w, (hw, hw), s, p)
        dxp = oracle.c.conv_dgrad(gy, w, (hw, hw), s, p, phases=True)
        dw = oracle.c.conv_wgrad(x, gy, ks, s, p)
        assert rel_err(dxp, golden[f"{name}_dx"]) <= TOL  # stride-phase algebra of csrc/conv.cpp:78-95
        np.testing.assert_allclose(dxp, dx, rtol=0, atol=1e-5 * np.abs(dx).max())
    else:
        y = oracle.c.dw_fwd(x, w, b, s, p)
        dx = oracle.c.dw_dgrad(gy, w, (hw, hw), s, p)
        dw = oracle.c.dw_wgrad(x, gy, ks, s, p)
    assert rel_err(y, golden[f"{name}_y"]) <= TOL
    assert rel_err(dx, golden[f"{name}_dx"]) <= TOL
    assert rel_err(dw, golden[f"{name}_dw"]) <= TOL
    if bias:
        assert rel_err(oracle.c.bias_grad(gy), golden[f"{name}_db"]) <= TOL


def test_conv_relu_epilogue_and_empty_phase():
    rng = np.random.default_rng(5)
    x = rng.standard_normal((2, 3, 9, 9)).astype(np.float32)
    w = rng.standard_normal((4, 3, 3, 3)).astype(np.float32)
    y = oracle.c.conv_fwd(x, w, None, 1, 1, relu=True)
    ref = torch.relu(torch.nn.functional.conv2d(torch.tensor(x), torch.tensor(w), padding=1)).numpy()
    assert rel_err(y, ref) <= TOL
    # ks=1, stride=2: three of the four stride phases receive no tap and must come out as zeros (K = 0 phases)
    w1 = rng.standard_normal((4, 3, 1, 1)).astype(np.float32)
    gy = rng.standard_normal((2, 4, 5, 5)).astype(np.float32)
    dx = oracle.c.conv_dgrad(gy, w1, (9, 9), 2, 0, phases=True)
    _, ref_dx, _, _ = oracle.aten_conv(torch.tensor(x), torch.tensor(w1), None, 2, 0, torch.tensor(gy), mask=(True, False, False))
    assert rel_err(dx, ref_dx.numpy()) <= TOL
    assert np.all(dx[:, :, 1::2, :] == 0) and np.all(dx[:, :, :, 1::2] == 0)


def test_wgrad_slices_follow_reference_host():
    # csrc/conv.cpp:106-109 for AlexNet conv1 (M=64, N=363, K=48400) with the 64x64 tile: 6 tiles -> 512/6 = 85 slices of 576
    slices, kslice = oracle.c.wgrad_slices(64, 363, 48400, 64, 64, 1.0)
    assert (slices, kslice) == (85, 576)
    assert oracle.c.wgrad_slices(64, 363, 100, 64, 64, 1.0) == (1, 112)  # K/64 = 1 bounds the split


@pytest.mark.parametrize("i", range(len(cases.BN)))
def test_bn_matches_aten(i, golden):
    n, c, h, w = cases.BN[i]
    x = (cases.rnd(900 + i, n, c, h, w) * 2 + 3).numpy()
    gamma, beta = cases.rnd(910 + i, c).numpy(), cases.rnd(920 + i, c).numpy()
    rm, rv = cases.rnd(930 + i, c).numpy().copy(), (cases.rnd(940 + i, c).abs() + 0.5).numpy().copy()
    g = cases.rnd(950 + i, n, c, h, w).numpy()
    rm0, rv0 = rm.copy(), rv.copy()
    mean, var = oracle.c.bn_stats(x, 0.1, rm, rv)
    invstd = (1.0 / np.sqrt(var.astype(np.float64) + 1e-5)).astype(np.float32)
    G = lambda k: golden[f"bn{i}_{k}"]
    assert rel_err(mean, G("mean")) <= TOL and rel_err(invstd, G("invstd")) <= TOL
    assert rel_err(rm, G("rm")) <= TOL and rel_err(rv, G("rv")) <= TOL
    y = oracle.c.bn_apply(x, mean, invstd, gamma, beta)
    assert rel_err(y, G("y")) <= TOL
    dx, dg, db = oracle.c.bn_backward(g, x, None, mean, invstd, gamma)
    assert rel_err(dx, G("dx")) <= TOL and rel_err(dg, G("dgamma")) <= TOL and rel_err(db, G("dbeta")) <= TOL
    yr = oracle.c.bn_apply(x, mean, invstd, gamma, beta, relu=True)
    dx, dg, db = oracle.c.bn_backward(g, x, yr, mean, invstd, gamma, relu=True)
    assert rel_err(dx, G("relu_dx")) <= TOL and rel_err(dg, G("relu_dgamma")) <= TOL and rel_err(db, G("relu_dbeta")) <= TOL
    ye = oracle.c.bn_apply(x, rm0, (1.0 / np.sqrt(rv0.astype(np.float64) + 1e-5)).astype(np.float32), gamma, beta)
    assert rel_err(ye, G("yeval")) <= TOL


def test_fold_bn_equals_conv_then_bn():
    rng = np.random.default_rng(9)
    x = rng.standard_normal((2, 3, 8, 8)).astype(np.float32)
    cw = rng.standard_normal((5, 3, 3, 3)).astype(np.float32); cb = rng.standard_normal(5).astype(np.float32)
    gamma, beta, rm = (rng.standard_normal(5).astype(np.float32) for _ in range(3))
    rv = (np.abs(rng.standard_normal(5)) + 0.3).astype(np.float32)
    fw, fb = oracle.c.fold_bn(cw, cb, gamma, beta, rm, rv, 1e-5)
    y = oracle.c.conv_fwd(x, fw, fb, 1, 1, relu=True)
    t = torch.nn.functional.conv2d(torch.tensor(x), torch.tensor(cw), torch.tensor(cb), padding=1)
    ref = torch.relu(torch.nn.functional.batch_norm(t, torch.tensor(rm), torch.tensor(rv), torch.tensor(gamma), torch.tensor(beta), False, 0.1, 1e-5))
    assert rel_err(y, ref.numpy()) <= TOL


@pytest.mark.parametrize("i", range(len(cases.MAXPOOL)))
def test_maxpool_matches_aten(i, golden):
    k, s, p, hw = cases.MAXPOOL[i]
    x = cases.rnd(700 + i, 2, 4, hw, hw).numpy()
    y, idx = oracle.c.maxpool_fwd(x, k, s, p)
    assert np.array_equal(y, golden[f"maxpool{i}_y"]) and np.array_equal(idx, golden[f"maxpool{i}_idx"])
    g = cases.rnd(720 + i, *y.shape).numpy()
    assert rel_err(oracle.c.maxpool_bwd(g, idx, (hw, hw)), golden[f"maxpool{i}_gx"]) <= TOL


def test_maxpool_nan_and_pool2_ties():
    x = np.zeros((1, 1, 4, 4), np.float32)
    x[0, 0, 0, 1] = np.nan
    y, idx = oracle.c.maxpool_fwd(x, 2, 2, 0)
    ref_y, ref_idx = torch.nn.functional.max_pool2d(torch.tensor(x), 2, 2, return_indices=True)
    assert np.isnan(y[0, 0, 0, 0]) and idx[0, 0, 0, 0] == 1 and np.array_equal(idx, ref_idx.numpy())
    # plan pool: all-equal window -> index 0 (strict >, first maximum wins), gradient goes to the top-left element
    y2, i2 = oracle.c.pool2_fwd(np.ones((1, 2, 4, 6), np.float32))
    assert np.all(i2 == 0) and np.all(y2 == 1)
    gx = oracle.c.pool2_bwd(np.full((1, 2, 2, 3), 2.0, np.float32), i2, (4, 6))
    assert gx.sum() == 2 * 12 and np.all(gx[:, :, ::2, ::2] == 2)
    # agrees with aten on random data (no ties)
    xr = np.random.default_rng(3).standard_normal((2, 3, 6, 8)).astype(np.float32)
    yr, ir = oracle.c.pool2_fwd(xr)
    ty, ti = torch.nn.functional.max_pool2d(torch.tensor(xr), 2, 2, return_indices=True)
    assert np.array_equal(yr, ty.numpy())
    oy, ox = np.meshgrid(np.arange(3), np.arange(4), indexing="ij")
    flat = (2 * oy + ir // 2) * 8 + 2 * ox + ir % 2
    assert np.array_equal(flat, ti.numpy())


@pytest.mark.parametrize("i", range(len(cases.ADAPOOL)))
def test_adapool_matches_aten(i, golden):
    hw, o = cases.ADAPOOL[i]
    x = cases.rnd(800 + i, 2, 5, hw, hw).numpy()
    assert rel_err(oracle.c.adapool_fwd(x, o), golden[f"adapool{i}_y"]) <= TOL


OPT = {"sgd_nesterov_wd": ("sgd", dict(lr=0.1, mom=0.9, nesterov=True, wd=1e-4)), "sgd_plain": ("sgd", dict(lr=0.05)),
       "sgd_damp_max": ("sgd", dict(lr=0.05, mom=0.8, damp=0.3, maximize=True)),
       "adam_wd": ("adam", dict(lr=1e-3, wd=0.01)), "adamw": ("adam", dict(lr=1e-3, wd=0.01, decoupled=True))}


@pytest.mark.parametrize("name", sorted(OPT))
def test_optimizers_match_torch_optim(name, golden):
    kind, kw = OPT[name]
    p = cases.rnd(1000, 37, 11).numpy().copy()
    m, v = np.zeros_like(p), np.zeros_like(p)
    for step in range(3):
        g = cases.rnd(1001 + step, 37, 11).numpy()
        if kind == "sgd":
            oracle.c.sgd(p, g, m if kw.get("mom") else None, first=(step == 0), **kw)
        else:
            oracle.c.adam(p, g, m, v, step + 1, **kw)
        assert rel_err(p, golden[f"optim_{name}_p{step}"]) <= 1e-6


def test_recorded_reference_curves_are_reproduced(golden_losses):
    """The CPU curves of the reference's own models, regenerated here, agree with the curves the reference recorded
    (results/acceptance.json) to its own 'matches' threshold of 1e-2 (tools/acceptance.py:103)."""
    for name in ("resnet18", "mobilenetv3"):
        ours, rec = golden_losses[name]["losses"], golden_losses[name]["recorded_reference_cpu"]
        assert max(abs(a - b) / max(abs(b), 1e-6) for a, b in zip(ours, rec)) < 1e-2
