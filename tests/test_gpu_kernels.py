"""Parity of the CUDA kernels, called through the C ABI (libomt_b200.so via ctypes), against the golden fixtures
(aten-CPU outputs on the reference's shape lists) and the CPU oracle. Needs a B200: run with -m gpu."""
import numpy as np
import pytest
import torch

import cases
import oracle
from conftest import TOL, rel_err

pytestmark = pytest.mark.gpu

CONV = cases.conv_cases()


@pytest.fixture(scope="module")
def capi():
    from omarchy_mac_torch_b200 import capi as m
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    m.lib()
    return m


def dev(t, cl=False):
    if t is None:
        return None
    t = torch.as_tensor(t).cuda()
    return t.contiguous(memory_format=torch.channels_last) if cl else t


def host(t):
    return t.detach().cpu().numpy()


@pytest.mark.parametrize("cl", [False, True], ids=["nchw", "nhwc"])
@pytest.mark.parametrize("name", sorted(CONV))
def test_conv_golden(capi, golden, name, cl):
    """Every conv fixture (dense: notes/scripts/conv_kinds_check.py, alexnet_ops_check.py; depthwise incl. general
    stride/pad) in both layouts, exact-fp32 path."""
    seed, n, ci, co, ks, s, p, hw, groups, bias = CONV[name]
    x, w, b, gy = cases.conv_inputs(*CONV[name])
    xd, wd, bd, gd = dev(x, cl), dev(w), dev(b), dev(gy, cl)
    if groups == 1:
        y = capi.conv_fwd(xd, wd, bd, s, p, flags=capi.FORCE_SIMT, cl=cl)
        dx = capi.conv_dgrad(gd, wd, (hw, hw), s, p, flags=capi.FORCE_SIMT, cl=cl)
        dw = capi.conv_wgrad(xd, gd, ks, s, p, flags=capi.FORCE_SIMT)
    else:
        y = capi.dw_fwd(xd, wd, bd, s, p, cl=cl)
        dx = capi.dw_dgrad(gd, wd, (hw, hw), s, p, cl=cl)
        dw = capi.dw_wgrad(xd, gd, ks, s, p)
    assert rel_err(host(y), golden[f"{name}_y"]) <= TOL
    assert rel_err(host(dx), golden[f"{name}_dx"]) <= TOL
    assert rel_err(host(dw), golden[f"{name}_dw"]) <= TOL
    if bias:
        assert rel_err(host(capi.conv_bias_grad(gd)), golden[f"{name}_db"]) <= TOL


def test_conv_default_path_matches_golden(capi, golden):
    """Without OMT_FORCE_SIMT the library picks its own path (tensor cores where supported); results must still hold."""
    for name in sorted(CONV):
        seed, n, ci, co, ks, s, p, hw, groups, bias = CONV[name]
        if groups != 1:
            continue
        x, w, b, gy = cases.conv_inputs(*CONV[name])
        for cl in (False, True):
            xd, wd, bd, gd = dev(x, cl), dev(w), dev(b), dev(gy, cl)
            assert rel_err(host(capi.conv_fwd(xd, wd, bd, s, p, cl=cl)), golden[f"{name}_y"]) <= TOL
            assert rel_err(host(capi.conv_dgrad(gd, wd, (hw, hw), s, p, cl=cl)), golden[f"{name}_dx"]) <= TOL
            assert rel_err(host(capi.conv_wgrad(xd, gd, ks, s, p)), golden[f"{name}_dw"]) <= TOL


TC_SHAPES = [(2, 3, 64, 32, 7, 2, 3), (3, 3, 24, 63, 11, 4, 2), (2, 4, 24, 20, 5, 2, 2), (2, 1, 16, 28, 3, 1, 1), (2, 32, 64, 16, 1, 1, 0), (2, 64, 128, 16, 3, 1, 1), (4, 64, 200, 15, 3, 1, 1), (3, 24, 40, 17, 5, 1, 2), (2, 64, 64, 16, 3, 2, 1),
             (2, 128, 256, 14, 1, 2, 0), (8, 256, 512, 14, 3, 1, 1), (2, 16, 32, 20, 7, 2, 3), (1, 8, 8, 9, 3, 1, 0), (2, 32, 32, 19, 3, 3, 1),
             (2, 32, 48, 16, 1, 4, 0), (2, 16, 16, 21, 5, 2, 0), (1, 520, 264, 9, 3, 1, 1),
             # weight-gradient operand modes: [pixels, ci] matrix with several 32-channel blocks; pixel rectangles for 7-, 8-, 9-
             # and 12-wide outputs with stride 1 and 2, odd batch; window mode with 32-multiple output channels
             (2, 64, 128, 16, 1, 1, 0), (4, 256, 512, 14, 1, 1, 0), (3, 128, 128, 7, 3, 1, 1), (5, 512, 64, 7, 3, 2, 1), (2, 96, 160, 9, 3, 1, 1),
             (2, 64, 96, 12, 5, 2, 2), (3, 256, 64, 8, 1, 2, 0), (3, 3, 64, 63, 11, 4, 2), (2, 4, 32, 20, 5, 2, 2), (2, 1, 32, 28, 3, 1, 1), (2, 3, 96, 40, 3, 1, 1),
             # few output tiles and a long reduction: split-K in forward and input gradient (also per stride phase)
             (2, 256, 256, 4, 3, 1, 1), (4, 512, 512, 2, 3, 1, 1), (8, 128, 256, 8, 3, 2, 1), (2, 512, 136, 4, 1, 1, 0),
             # more 128 x 256 tiles than SMs with a short reduction: one accumulator per tile, two tiles in flight in TMEM
             (32, 256, 512, 28, 1, 1, 0), (40, 288, 264, 24, 1, 1, 0)]


@pytest.mark.parametrize("shape", TC_SHAPES)
def test_tensor_core_path_vs_aten_and_exact_path(capi, shape):
    """tcgen05 3xTF32 kernels (OMT_FORCE_TC: fails instead of silently taking the CUDA-core path) on channels-last inputs:
    forward with bias+ReLU into both layouts, input gradient for every stride (stride phases), weight gradient with
    scale; against float64 aten on the CPU and against the exact-fp32 kernels. Shapes cover 1-4 stride, channel counts
    that are not multiples of 32 / 64 / 128, ragged pixel tails, >256 output channels and k-blocks beyond one stage ring."""
    n, ci, co, hw, ks, s, p = shape
    torch.manual_seed(0)
    x = torch.randn(n, ci, hw, hw)
    w = torch.randn(co, ci, ks, ks) * 0.05
    b = torch.randn(co)
    oh = (hw + 2 * p - ks) // s + 1
    gy = torch.randn(n, co, oh, oh)
    y, dx, dw, _ = oracle.aten_conv(x.double(), w.double(), b.double(), s, p, gy.double())
    y, dx, dw = y.relu().float().numpy(), dx.float().numpy(), dw.float().numpy()
    xd, wd, bd, gd = dev(x, True), dev(w), dev(b), dev(gy, True)
    before = capi.kernel_counts()
    for cl in (True, False):
        got = capi.conv_fwd(xd, wd, bd, s, p, flags=capi.FORCE_TC | capi.EPI_RELU, cl=cl)
        assert rel_err(host(got), y) <= TOL
    # few input channels: forward and weight gradient run in window mode (the weight gradient when co is a multiple of
    # 32); the input gradient takes the library's default path
    few = ci <= 4
    wg_tc = not few or co % 32 == 0
    got_dx = capi.conv_dgrad(gd, wd, (hw, hw), s, p, flags=0 if few else capi.FORCE_TC, cl=True)
    assert rel_err(host(got_dx), dx) <= TOL
    got_dw = capi.conv_wgrad(xd, gd, ks, s, p, flags=capi.FORCE_TC if wg_tc else 0, scale=0.5)
    assert rel_err(2 * host(got_dw), dw) <= TOL
    if few and wg_tc:  # window mode stages x itself: an NCHW x is as good
        got_dw = capi.conv_wgrad(dev(x), gd, ks, s, p, flags=capi.FORCE_TC, scale=0.5)
        assert rel_err(2 * host(got_dw), dw) <= TOL
    capi.call("omt_sync")  # a tensor-core kernel that gave up on a barrier would be reported here
    after = capi.kernel_counts()
    assert sum(v - before.get(k, 0) for k, v in after.items() if k.startswith(("conv_tc_1", "conv_tc_2", "conv_tc_window", "wgrad_tc_1", "wgrad_tc_2"))) >= (2 + wg_tc if few else 4)
    # the two paths agree with each other far inside the tolerance, with the cross terms in their own accumulator or not
    exact = capi.conv_fwd(xd, wd, bd, s, p, flags=capi.FORCE_SIMT | capi.EPI_RELU, cl=True)
    assert rel_err(host(capi.conv_fwd(xd, wd, bd, s, p, flags=capi.FORCE_TC | capi.EPI_RELU, cl=True)), host(exact)) <= 5e-5
    assert rel_err(host(capi.conv_fwd(xd, wd, bd, s, p, flags=capi.FORCE_TC | capi.EPI_RELU | capi.PRECISE_ACCUM, cl=True)), host(exact)) <= 5e-5
    if n == 32:  # (the n = 40 shape is split into 128-column tiles: fewer rounds of the persistent loop on 148 SMs)
        acc1 = lambda kc: sum(v for k, v in kc.items() if k.endswith("_acc1"))  # single-accumulator tiles, one CTA or a CTA pair
        assert acc1(after) > acc1(before), after


@pytest.mark.parametrize("shape,cl_out", [((4, 64, 96, 14, 3, 1, 1), True), ((2, 32, 64, 16, 1, 2, 0), True), ((2, 64, 64, 16, 3, 2, 1), True),
                                          ((2, 32, 40, 15, 3, 1, 1), False), ((2, 64, 256, 4, 3, 1, 1), True),
                                          # 256-column tiles on CTA pairs: one accumulator (8 k-blocks) and two (72 k-blocks)
                                          ((32, 256, 256, 28, 1, 1, 0), True), ((32, 256, 256, 28, 3, 1, 1), True)])
def test_input_gradient_accumulates_in_the_epilogue(capi, shape, cl_out):
    """OMT_EPI_ACCUM: dx += conv^T(gy, w) (TMA reduce-add for dense channels-last outputs, read-add-write for stride phases
    and NCHW outputs) against a separate input gradient plus add; a geometry outside the tensor-core path is refused."""
    n, ci, co, hw, ks, s, p = shape
    torch.manual_seed(1)
    w = torch.randn(co, ci, ks, ks) * 0.05
    oh = (hw + 2 * p - ks) // s + 1
    gy, base = torch.randn(n, co, oh, oh), torch.randn(n, ci, hw, hw)
    x = torch.zeros(n, ci, hw, hw, dtype=torch.float64)
    _, dx, _, _ = oracle.aten_conv(x, w.double(), None, s, p, gy.double())
    want = (base.double() + dx).float().numpy()
    acc = dev(base, cl_out).clone(memory_format=torch.preserve_format)
    got = capi.conv_dgrad(dev(gy, True), dev(w), (hw, hw), s, p, acc=acc)
    assert got.data_ptr() == acc.data_ptr()
    assert rel_err(host(got), want) <= TOL
    capi.call("omt_sync")
    small = torch.randn(2, 3, 8, 8, device="cuda")  # ci = 3: the tensor cores do not take this input gradient
    with pytest.raises(capi.OmtError, match="OMT_EPI_ACCUM"):
        capi.conv_dgrad(torch.randn(2, 8, 8, 8, device="cuda"), torch.randn(8, 3, 3, 3, device="cuda"), (8, 8), 1, 1, acc=small)


def test_exact_path_takes_more_than_65535_row_tiles(capi):
    """9.4 million output pixels on the exact-fp32 kernels: more GEMM row tiles than a launch grid's y or z extent holds
    (the row tiles therefore run along x). Forward and input gradient, against aten on the CPU."""
    torch.manual_seed(0)
    x, w = torch.randn(64, 3, 384, 384), torch.randn(4, 3, 3, 3) * 0.2
    y = torch.nn.functional.conv2d(x, w, padding=1)
    assert y.shape[0] * y.shape[2] * y.shape[3] > 65535 * 128
    got = capi.conv_fwd(dev(x), dev(w), None, 1, 1, flags=capi.FORCE_SIMT)
    assert rel_err(host(got), y.numpy()) <= TOL
    gy = torch.randn_like(y)
    dx = torch.ops.aten.convolution_backward(gy, x, w, None, [1, 1], [1, 1], [1, 1], False, [0, 0], 1, [True, False, False])[0]
    assert rel_err(host(capi.conv_dgrad(dev(gy), dev(w), (384, 384), 1, 1, flags=capi.FORCE_SIMT)), dx.numpy()) <= TOL
    capi.call("omt_check_errors")


def test_tensor_core_path_refuses_what_it_cannot_take(capi):
    x = torch.randn(2, 16, 16, 16, device="cuda")           # 16 channels but NCHW: not a TMA-loadable operand
    w = torch.randn(8, 16, 3, 3, device="cuda")
    with pytest.raises(capi.OmtError, match="tensor-core"):
        capi.conv_fwd(x, w, None, 1, 1, flags=capi.FORCE_TC)
    assert rel_err(host(capi.conv_fwd(x, w, None, 1, 1)), torch.nn.functional.conv2d(x.cpu(), w.cpu(), padding=1).numpy()) <= TOL


def test_conv_epilogues_and_scale(capi):
    rng = np.random.default_rng(11)
    x = rng.standard_normal((2, 5, 10, 9)).astype(np.float32)
    w = rng.standard_normal((7, 5, 3, 3)).astype(np.float32)
    b = rng.standard_normal(7).astype(np.float32)
    y = capi.conv_fwd(dev(x), dev(w), dev(b), 1, 1, flags=capi.EPI_RELU | capi.FORCE_SIMT)
    assert rel_err(host(y), oracle.c.conv_fwd(x, w, b, 1, 1, relu=True)) <= TOL
    gy = rng.standard_normal((2, 7, 10, 9)).astype(np.float32)
    dw = capi.conv_wgrad(dev(x), dev(gy), 3, 1, 1, flags=capi.FORCE_SIMT, scale=0.25)
    assert rel_err(host(dw), 0.25 * oracle.c.conv_wgrad(x, gy, 3, 1, 1)) <= TOL
    # K = 0 stride phases: ks=1 stride=2 leaves three of four phases without taps -> zeros
    w1 = rng.standard_normal((7, 5, 1, 1)).astype(np.float32)
    g1 = rng.standard_normal((2, 7, 5, 5)).astype(np.float32)
    dx = host(capi.conv_dgrad(dev(g1), dev(w1), (10, 9), 2, 0, flags=capi.FORCE_SIMT))
    ref = oracle.c.conv_dgrad(g1, w1, (10, 9), 2, 0)
    assert rel_err(dx, ref) <= TOL and np.all(dx[:, :, 1::2, :] == 0)


@pytest.mark.parametrize("shape", [(16, 3, 64, 11, 4, 2, 63), (8, 64, 192, 5, 1, 2, 27), (32, 128, 128, 3, 1, 1, 16), (4, 32, 48, 3, 2, 1, 30),
                                   (2, 256, 64, 1, 1, 0, 14), (3, 16, 300, 3, 1, 1, 7)])
def test_conv_larger_shapes_vs_aten(capi, shape):
    """AlexNet / ResNet style shapes (tools/gemm_bench.py:8-9, scaled to keep the CPU side quick) against aten CPU."""
    n, ci, co, ks, s, p, hw = shape
    torch.manual_seed(0)
    x, w = torch.randn(n, ci, hw, hw), torch.randn(co, ci, ks, ks) * 0.05
    b = torch.randn(co)
    oh = (hw + 2 * p - ks) // s + 1
    gy = torch.randn(n, co, oh, oh)
    y, dx, dw, db = oracle.aten_conv(x, w, b, s, p, gy)
    for cl in (False, True):
        xd, gd = dev(x, cl), dev(gy, cl)
        assert rel_err(host(capi.conv_fwd(xd, dev(w), dev(b), s, p, cl=cl)), y.numpy()) <= TOL
        assert rel_err(host(capi.conv_dgrad(gd, dev(w), (hw, hw), s, p, cl=cl)), dx.numpy()) <= TOL
        assert rel_err(host(capi.conv_wgrad(xd, gd, ks, s, p)), dw.numpy()) <= TOL
        assert rel_err(host(capi.conv_bias_grad(gd)), db.numpy()) <= TOL


# the distinct convolution geometries of ResNet-50 on 224x224 inputs: (ci, co, input height, ks, stride)
R50_LAYERS = [(3, 64, 224, 7, 2), (64, 64, 56, 1, 1), (64, 64, 56, 3, 1), (64, 256, 56, 1, 1), (256, 64, 56, 1, 1), (256, 128, 56, 1, 1), (128, 128, 56, 3, 2),
              (128, 512, 28, 1, 1), (256, 512, 56, 1, 2), (512, 128, 28, 1, 1), (128, 128, 28, 3, 1), (512, 256, 28, 1, 1), (256, 256, 28, 3, 2),
              (256, 1024, 14, 1, 1), (512, 1024, 28, 1, 2), (1024, 256, 14, 1, 1), (256, 256, 14, 3, 1), (1024, 512, 14, 1, 1), (512, 512, 14, 3, 2),
              (512, 2048, 7, 1, 1), (1024, 2048, 14, 1, 2), (2048, 512, 7, 1, 1), (512, 512, 7, 3, 1)]


@pytest.mark.parametrize("layer", R50_LAYERS, ids=lambda l: "ci%d_co%d_hw%d_k%d_s%d" % l)
def test_resnet50_layer_geometries_on_tensor_cores(capi, layer):
    """Every convolution geometry of the ResNet-50 training step (batch reduced to 4) on the tcgen05 kernels, channels-last:
    forward, input gradient (also accumulating into an existing gradient, as the residual joins of the backward graph do)
    and weight gradient against float64 aten on the CPU."""
    ci, co, hw, ks, s = layer
    n, p = 4, ks // 2
    torch.manual_seed(ci + co + hw)
    x, w = torch.randn(n, ci, hw, hw), torch.randn(co, ci, ks, ks) * (2.0 / (ci * ks * ks)) ** 0.5
    oh = (hw + 2 * p - ks) // s + 1
    gy = torch.randn(n, co, oh, oh)
    y, dx, dw, _ = oracle.aten_conv(x.double(), w.double(), None, s, p, gy.double())
    xd, wd, gd = dev(x, True), dev(w), dev(gy, True)
    assert rel_err(host(capi.conv_fwd(xd, wd, None, s, p, flags=capi.FORCE_TC, cl=True)), y.float().numpy()) <= TOL
    assert rel_err(host(capi.conv_wgrad(xd, gd, ks, s, p, flags=capi.FORCE_TC)), dw.float().numpy()) <= TOL
    if ci > 4:  # the network input needs no gradient
        assert rel_err(host(capi.conv_dgrad(gd, wd, (hw, hw), s, p, flags=capi.FORCE_TC, cl=True)), dx.float().numpy()) <= TOL
        base = torch.randn(n, ci, hw, hw)
        acc = dev(base, True).clone(memory_format=torch.preserve_format)
        capi.conv_dgrad(gd, wd, (hw, hw), s, p, acc=acc)
        assert rel_err(host(acc), (base.double() + dx).float().numpy()) <= TOL
    capi.call("omt_sync")


@pytest.mark.parametrize("shape", [(3, 64, 64, 13, 9), (2, 32, 64, 56, 56), (5, 96, 32, 7, 20), (4, 64, 64, 33, 1), (2, 128, 64, 1, 17)],
                         ids=lambda s: "n%d_ci%d_co%d_%dx%d" % s)
def test_weight_gradient_of_narrow_3x3_layers_pairs_taps(capi, shape):
    """3x3 stride-1 pad-1 layers with at most 64 output channels: the weight-gradient kernel fills the empty half of its 128-row
    gy tile with gy shifted by one pixel, so that one x column yields two taps. Image edges (the shifted operand's zero fill
    and the padding the identity relies on), widths of one pixel and pixel counts that do not fill a block, against float64
    aten on the CPU."""
    n, ci, co, h, w_ = shape
    torch.manual_seed(n * 1000 + ci + co + h)
    x, gy = torch.randn(n, ci, h, w_), torch.randn(n, co, h, w_)
    wt = torch.zeros(co, ci, 3, 3, dtype=torch.float64)
    _, _, dw, _ = oracle.aten_conv(x.double(), wt, None, 1, 1, gy.double())
    before = capi.kernel_counts()
    got = host(capi.conv_wgrad(dev(x, True), dev(gy, True), 3, 1, 1, flags=capi.FORCE_TC))
    after = capi.kernel_counts()
    pairs = lambda kc: sum(v for k, v in kc.items() if k.endswith("_tap_pairs"))
    assert pairs(after) == pairs(before) + 1, after
    assert rel_err(got, dw.float().numpy()) <= TOL
    for tap in range(9):  # per tap: an error in one tap's columns must not hide behind the others' magnitude
        assert rel_err(got[:, :, tap // 3, tap % 3], dw[:, :, tap // 3, tap % 3].float().numpy()) <= 2 * TOL, tap
    capi.call("omt_sync")


@pytest.mark.parametrize("shape", [(2, 3, 64, 7, 2, 3, 37, 41), (3, 3, 32, 5, 1, 2, 19, 23), (2, 4, 64, 3, 2, 1, 16, 9), (2, 1, 64, 11, 4, 2, 63, 63),
                                   (2, 3, 64, 3, 1, 0, 12, 40), (1, 2, 32, 4, 3, 0, 31, 10)],
                         ids=lambda s: "n%d_ci%d_co%d_k%d_s%d_p%d_%dx%d" % s)
def test_weight_gradient_of_first_layers_pairs_filter_rows(capi, shape):
    """At most 4 input and at most 64 output channels (network stems): the weight-gradient kernel fills the empty half of its
    gy tile with gy shifted by one row, so that the x columns of filter row ky also yield row ky - stride; its pixel blocks
    start one row above the image so that the shifted operand's first row has a partner. Strides 1-4, with and without
    padding, odd image sizes; per filter row against float64 aten on the CPU."""
    n, ci, co, ks, s_, p_, h, w_ = shape
    torch.manual_seed(n + ci + co + ks + h)
    oh, ow = (h + 2 * p_ - ks) // s_ + 1, (w_ + 2 * p_ - ks) // s_ + 1
    x, gy = torch.randn(n, ci, h, w_), torch.randn(n, co, oh, ow)
    wt = torch.zeros(co, ci, ks, ks, dtype=torch.float64)
    _, _, dw, _ = oracle.aten_conv(x.double(), wt, None, s_, p_, gy.double())
    before = capi.kernel_counts()
    got = host(capi.conv_wgrad(dev(x), dev(gy, True), ks, s_, p_, flags=capi.FORCE_TC))
    after = capi.kernel_counts()
    pairs = lambda kc: sum(v for k, v in kc.items() if k.endswith("_tap_pairs"))
    assert pairs(after) == pairs(before) + 1, after
    assert rel_err(got, dw.float().numpy()) <= TOL
    for ky in range(ks):
        assert rel_err(got[:, :, ky], dw[:, :, ky].float().numpy()) <= 2 * TOL, ky
    capi.call("omt_sync")


@pytest.mark.parametrize("shape", [(8, 64, 256, 28, 1, 1), (4, 128, 128, 28, 3, 1), (4, 256, 512, 28, 1, 2), (16, 96, 160, 14, 3, 1)],
                         ids=lambda s: "n%d_ci%d_co%d_hw%d_k%d_s%d" % s)
def test_conv_plan_overrides_and_the_tuning_pass(capi, shape):
    """Every tile width / slice factor the tuning pass may choose gives the same results as the planner's rules (against
    float64 aten on the CPU), also with a caller-provided workspace of omt_conv_workspace_bytes under the override; then the
    pass itself: it leaves either no override or one of its candidates, and the results stand."""
    n, ci, co, hw, ks, s_ = shape
    p_ = ks // 2
    torch.manual_seed(sum(shape))
    x, w = torch.randn(n, ci, hw, hw), torch.randn(co, ci, ks, ks) * (2.0 / (ci * ks * ks)) ** 0.5
    oh = (hw + 2 * p_ - ks) // s_ + 1
    gy = torch.randn(n, co, oh, oh)
    y, dx, dw, _ = oracle.aten_conv(x.double(), w.double(), None, s_, p_, gy.double())
    y, dx, dw = y.float().numpy(), dx.float().numpy(), dw.float().numpy()
    xd, wd, gd = dev(x, True), dev(w), dev(gy, True)
    g = capi.geo(n, ci, co, hw, hw, ks, s_, p_)

    def check_all():
        assert rel_err(host(capi.conv_fwd(xd, wd, None, s_, p_, flags=capi.FORCE_TC, cl=True)), y) <= TOL
        assert rel_err(host(capi.conv_dgrad(gd, wd, (hw, hw), s_, p_, flags=capi.FORCE_TC, cl=True)), dx) <= TOL
        assert rel_err(host(capi.conv_wgrad(xd, gd, ks, s_, p_, flags=capi.FORCE_TC)), dw) <= TOL

    try:
        for tile in (64, 128, 256):
            capi.call("omt_conv_plan_set", 0, g, tile, 1.0)
            capi.call("omt_conv_plan_set", 1, g, tile, 1.0)
            for wt, mult in ((64, 2.0), (128, 0.5), (192, 1.0), (256, 2.0), (0, 0.5)):
                capi.call("omt_conv_plan_set", 2, g, wt, mult)
                check_all()
            # the caller's workspace, sized under the override
            nbytes = capi.lib().omt_conv_workspace_bytes(2, g, 0)
            ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
            got = torch.empty(co, ci, ks, ks, device="cuda")
            capi.call("omt_conv_wgrad", g, capi.act(xd), capi.act(gd), capi.ptr(got), 1.0, capi.FORCE_TC, capi.ptr(ws), nbytes, capi.stream_handle())
            assert rel_err(host(got), dw) <= TOL
        for kind in (0, 1, 2):
            capi.call("omt_conv_plan_set", kind, g, 0, 1.0)
        assert capi.conv_plans_dump() == {}
        for kind in (0, 1, 2):
            tile, mult, best, rule = capi.conv_autotune(kind, g)
            assert tile in (0, 64, 128, 192, 256) and mult in (0.5, 1.0, 2.0) and 0 <= best <= rule + 1e-6
            stored = capi.conv_plan_get(kind, g)
            assert stored == ((tile, mult) if (tile or mult != 1.0) else None)
        check_all()
    finally:
        for kind in (0, 1, 2):
            capi.call("omt_conv_plan_set", kind, g, 0, 1.0)
    capi.call("omt_sync")


def test_alexnet_conv1_full_size_per_tensor_vs_aten(capi):
    """AlexNet conv1 at full size (x [16,3,224,224], w [64,3,11,11], stride 4, pad 2; tools/gemm_bench.py:26-38): y, dx, dw
    and db each compared per tensor with aten's convolution and convolution_backward on the CPU, on the library's default
    path (NCHW operands, as the reference benchmarks the layer) and with channels-last operands."""
    torch.manual_seed(0)
    x = torch.randn(16, 3, 224, 224)
    conv = torch.nn.Conv2d(3, 64, 11, stride=4, padding=2)
    w, b = conv.weight.detach(), conv.bias.detach()
    gy = torch.randn(16, 64, 55, 55)
    y, dx, dw, db = oracle.aten_conv(x, w, b, 4, 2, gy)
    for cl in (False, True):
        xd, gd = dev(x, cl), dev(gy, cl)
        assert rel_err(host(capi.conv_fwd(xd, dev(w), dev(b), 4, 2, cl=cl)), y.numpy()) <= TOL
        assert rel_err(host(capi.conv_dgrad(gd, dev(w), (224, 224), 4, 2, cl=cl)), dx.numpy()) <= TOL
        assert rel_err(host(capi.conv_wgrad(xd, gd, 11, 4, 2)), dw.numpy()) <= TOL
        assert rel_err(host(capi.conv_bias_grad(gd)), db.numpy()) <= TOL
    capi.call("omt_sync")


def test_alexnet_conv1_full_size_properties(capi):
    """AlexNet conv1 at full size through size-independent properties: linearity of each pass in its activation
    argument and the adjoint identity <conv(x), gy> == <x, dgrad(gy)> == <w, wgrad(x, gy)>."""
    torch.manual_seed(0)
    x = torch.randn(16, 3, 224, 224, device="cuda")
    conv = torch.nn.Conv2d(3, 64, 11, stride=4, padding=2)
    w, b = conv.weight.detach().cuda(), conv.bias.detach().cuda()
    gy = torch.randn(16, 64, 55, 55, device="cuda")
    y = capi.conv_fwd(x, w, None, 4, 2)
    dx = capi.conv_dgrad(gy, w, (224, 224), 4, 2)
    dw = capi.conv_wgrad(x, gy, 11, 4, 2)
    a = (y.double() * gy.double()).sum().item()
    assert abs(a - (x.double() * dx.double()).sum().item()) <= 1e-4 * abs(a)
    assert abs(a - (w.double() * dw.double()).sum().item()) <= 1e-4 * abs(a)
    y2 = capi.conv_fwd(2.0 * x, w, None, 4, 2)
    assert rel_err(host(y2), 2.0 * host(y)) <= 1e-6
    yb = capi.conv_fwd(x, w, b, 4, 2)
    assert rel_err(host(yb - y), np.broadcast_to(host(b)[None, :, None, None], yb.shape)) <= 1e-4
    # and a slice of the result against the CPU oracle
    ys = oracle.c.conv_fwd(host(x[:1]), host(w), host(b), 4, 2)
    assert rel_err(host(yb[:1]), ys) <= TOL


@pytest.mark.parametrize("cl", [False, True], ids=["nchw", "nhwc"])
@pytest.mark.parametrize("i", range(len(cases.BN)))
def test_bn_golden(capi, golden, i, cl):
    n, c, h, w = cases.BN[i]
    if cl and c % 4:
        pytest.skip("channels-last BN kernels need c % 4 == 0")
    G = lambda k: golden[f"bn{i}_{k}"]
    x = dev(cases.rnd(900 + i, n, c, h, w) * 2 + 3, cl)
    gamma, beta = dev(cases.rnd(910 + i, c)), dev(cases.rnd(920 + i, c))
    rm, rv = dev(cases.rnd(930 + i, c)), dev(cases.rnd(940 + i, c).abs() + 0.5)
    g = dev(cases.rnd(950 + i, n, c, h, w), cl)
    ye = capi.bn_eval(x, gamma, beta, rm, rv)
    assert rel_err(host(ye), G("yeval")) <= TOL
    rm0 = rm.clone()
    y, mean, invstd, nrm, nrv = capi.bn_train(x, gamma, beta, rm, rv, functional=True)
    assert torch.equal(rm, rm0)  # functional mode leaves the running stats alone
    assert rel_err(host(nrm), G("rm")) <= TOL and rel_err(host(nrv), G("rv")) <= TOL
    y, mean, invstd = capi.bn_train(x, gamma, beta, rm, rv)
    for got, key in ((y, "y"), (mean, "mean"), (invstd, "invstd"), (rm, "rm"), (rv, "rv")):
        assert rel_err(host(got), G(key)) <= TOL, key
    dx, dg, db = capi.bn_backward(g, x, None, mean, invstd, gamma)
    assert rel_err(host(dx), G("dx")) <= TOL and rel_err(host(dg), G("dgamma")) <= TOL and rel_err(host(db), G("dbeta")) <= TOL
    yr, _, _, _, _ = capi.bn_train(x, gamma, beta, rm, rv, relu=True, functional=True)
    assert rel_err(host(yr), np.maximum(G("y"), 0)) <= TOL
    dx, dg, db = capi.bn_backward(g, x, yr, mean, invstd, gamma, relu=True)
    assert rel_err(host(dx), G("relu_dx")) <= TOL and rel_err(host(dg), G("relu_dgamma")) <= TOL and rel_err(host(db), G("relu_dbeta")) <= TOL


BNSTATS_SHAPES = [  # n, ci, co, hw, ks, stride, pad, bias, expect the statistics from the epilogue
    (4, 32, 96, 14, 1, 1, 0, False, True),      # 784 pixels: the last row tile holds 16 valid rows
    (2, 32, 40, 15, 1, 1, 0, True, True),       # 40 output channels: a ragged channel chunk
    (8, 3, 64, 32, 3, 1, 1, True, True),        # <= 4 input channels: rectangles of output pixels as GEMM rows
    (2, 3, 32, 35, 7, 2, 3, False, True),       # the same with a stride, odd sizes: rows outside the image are not counted
    (16, 64, 64, 28, 3, 1, 1, False, True),     # 128 x 64 tiles
    (16, 128, 128, 28, 3, 1, 1, True, True),    # 128 x 128 tiles
    (32, 256, 512, 28, 1, 1, 0, False, True),   # 128 x 256 tiles, one accumulator per tile, more tiles than SMs
    (32, 64, 256, 28, 1, 1, 0, False, True),    # a reduction of two k-blocks on a small output: one launch less wins
    (64, 64, 256, 56, 1, 1, 0, False, False),   # the same on a large output: bound by storing y, statistics left to a separate pass
    (4, 256, 512, 8, 1, 1, 0, False, False),    # few tiles and a long reduction: split over CTAs, no statistics from the epilogue
]


@pytest.mark.parametrize("shape", BNSTATS_SHAPES, ids=lambda s: "n%d_ci%d_co%d_hw%d_k%d_s%d" % s[:6])
def test_conv_epilogue_batch_norm_statistics(capi, shape):
    """OMT_EPI_BNSTATS: the forward convolution reduces the batch-norm statistics of what it stores; merged, they must equal
    the statistics of y taken in float64, y itself must be bit-identical to a call without the flag, and the running
    statistics must follow. Twice in a row (the merge kernel's ticket counters reset themselves)."""
    n, ci, co, hw, ks, s, p, bias, expect = shape
    torch.manual_seed(3)
    x = torch.randn(n, ci, hw, hw) + 0.5
    w = torch.randn(co, ci, ks, ks) * 0.1
    b = torch.randn(co) * 3 if bias else None
    xd, wd, bd = dev(x, True), dev(w), dev(b)
    plain = capi.conv_fwd(xd, wd, bd, s, p, cl=True)
    for _ in range(2):
        y, part, groups = capi.conv_fwd_bnstats(xd, wd, bd, s, p)
        assert (groups > 0) == expect, groups
        if not expect:
            return
        assert torch.equal(y, plain)
        rm, rv = torch.randn(co, device="cuda"), torch.rand(co, device="cuda") + 0.5
        mean, var, invstd, nrm, nrv = capi.bn_stats_from_partials(part, groups, co, rm, rv, momentum=0.1, eps=1e-5, functional=True)
        y64 = y.double().cpu()
        m64, v64 = y64.mean(dim=(0, 2, 3)), y64.var(dim=(0, 2, 3), unbiased=False)
        cnt = y64.numel() // co
        assert rel_err(host(mean), m64.float().numpy()) <= 1e-6
        assert rel_err(host(var), v64.float().numpy()) <= 1e-5
        assert rel_err(host(invstd), (1 / torch.sqrt(v64 + 1e-5)).float().numpy()) <= 1e-5
        assert rel_err(host(nrm), (rm.cpu().double() * 0.9 + 0.1 * m64).float().numpy()) <= 1e-6
        assert rel_err(host(nrv), (rv.cpu().double() * 0.9 + 0.1 * v64 * cnt / (cnt - 1)).float().numpy()) <= 1e-5
    capi.call("omt_sync")


def test_conv_epilogue_statistics_survive_a_large_mean(capi):
    """Outputs whose mean is 1000 standard deviations away from zero (a large bias on tiny activations): the grouped, exactly
    merged moments keep the variance, where sums of y and y^2 in float32 would lose it entirely."""
    torch.manual_seed(4)
    x, w = torch.randn(16, 32, 28, 28), torch.randn(64, 32, 3, 3) * 0.006
    b = torch.full((64,), 100.0)
    y, part, groups = capi.conv_fwd_bnstats(dev(x, True), dev(w), dev(b), 1, 1)
    assert groups > 0
    mean, var, invstd = capi.bn_stats_from_partials(part, groups, 64)
    y64 = y.double().cpu()
    v64 = y64.var(dim=(0, 2, 3), unbiased=False)
    assert float((y64.mean(dim=(0, 2, 3)) / v64.sqrt()).min()) > 500
    assert rel_err(host(invstd), (1 / torch.sqrt(v64 + 1e-5)).float().numpy()) <= 1e-3
    assert rel_err(host(mean), y64.mean(dim=(0, 2, 3)).float().numpy()) <= 1e-6


@pytest.mark.parametrize("cl", [False, True], ids=["nchw", "nhwc"])
@pytest.mark.parametrize("shape", [(3, 8, 6, 10), (2, 5, 4, 6), (4, 32, 16, 16)])
def test_bn_apply_with_max_pool(capi, shape, cl):
    """omt_bn_apply_pool2 against omt_bn_apply followed by omt_pool2_fwd: same y, same pooled values, same argmax bytes."""
    n, c, h, w = shape
    if cl and c % 4:
        pytest.skip("channels-last BN kernels need c % 4 == 0")
    torch.manual_seed(5)
    x = dev(torch.randn(n, c, h, w) * 2 + 1, cl)
    gamma, beta = dev(torch.randn(c)), dev(torch.randn(c))
    rm, rv = torch.zeros(c, device="cuda"), torch.ones(c, device="cuda")
    y_ref, mean, invstd = capi.bn_train(x, gamma, beta, rm, rv, relu=True)
    z_ref, idx_ref = capi.pool2_fwd(y_ref)
    y = torch.empty_like(x)
    z = torch.empty_like(z_ref)
    idx = torch.empty_like(idx_ref)
    capi.call("omt_bn_apply_pool2", capi.act(x), capi.act(y), capi.act(z), capi.ptr(idx), n, c, h, w, capi.ptr(mean), capi.ptr(invstd), capi.ptr(gamma),
              capi.ptr(beta), capi.BN_RELU, capi.stream_handle())
    assert torch.equal(y, y_ref) and torch.equal(z, z_ref) and torch.equal(idx, idx_ref)
    z2 = torch.empty_like(z_ref)   # without y and without the argmax (an eval caller)
    capi.call("omt_bn_apply_pool2", capi.act(x), capi.null_act(), capi.act(z2), None, n, c, h, w, capi.ptr(mean), capi.ptr(invstd), capi.ptr(gamma),
              capi.ptr(beta), capi.BN_RELU, capi.stream_handle())
    assert torch.equal(z2, z_ref)
    with pytest.raises(capi.OmtError, match="even"):
        odd = dev(torch.randn(1, 4, 5, 6), cl)
        capi.call("omt_bn_apply_pool2", capi.act(odd), capi.null_act(), capi.act(torch.empty(1, 4, 2, 3, device="cuda")), None, 1, 4, 5, 6, capi.ptr(mean),
                  capi.ptr(invstd), capi.ptr(gamma), capi.ptr(beta), 0, capi.stream_handle())


@pytest.mark.parametrize("cl", [False, True], ids=["nchw", "nhwc"])
@pytest.mark.parametrize("shape", [(3, 8, 6, 10), (2, 5, 3, 7), (4, 32, 16, 16), (2, 12, 5, 5), (5, 64, 9, 11)])
def test_bn_relu_mask_as_bits(capi, shape, cl):
    """OMT_BN_MASKBITS: the apply pass leaves the ReLU mask as one bit per element behind y, the backward passes take the
    mask from those bits. Checked: the bits are (y > 0) in memory order; a backward that sees only the bits (y's values
    overwritten first) equals the backward that reads y; with and without the identity-branch gradient."""
    n, c, h, w = shape
    if cl and c % 4:
        pytest.skip("channels-last BN kernels need c % 4 == 0")
    torch.manual_seed(7)
    numel = n * c * h * w
    words = (numel + 31) // 32
    x = dev(torch.randn(n, c, h, w) * 2 + 0.3, cl)
    g = dev(torch.randn(n, c, h, w), cl)
    res = dev(torch.randn(n, c, h, w), cl)
    gamma, beta = dev(torch.randn(c)), dev(torch.randn(c))
    rm, rv = torch.zeros(c, device="cuda"), torch.ones(c, device="cuda")
    _, mean, invstd = capi.bn_train(x, gamma, beta, rm, rv, relu=True)
    for with_res in (False, True):
        flat = torch.full((numel + words,), float("nan"), device="cuda")
        strides = (h * w * c, 1, w * c, c) if cl else (c * h * w, h * w, w, 1)
        y = flat.as_strided((n, c, h, w), strides, 0)
        capi.call("omt_bn_apply_add", capi.act(x), capi.act(res) if with_res else capi.null_act(), capi.act(y), n, c, h, w, capi.ptr(mean), capi.ptr(invstd),
                  capi.ptr(gamma), capi.ptr(beta), capi.BN_RELU | capi.BN_MASKBITS, capi.stream_handle())
        torch.cuda.synchronize()
        y_ref = torch.empty_like(x)
        capi.call("omt_bn_apply_add", capi.act(x), capi.act(res) if with_res else capi.null_act(), capi.act(y_ref), n, c, h, w, capi.ptr(mean),
                  capi.ptr(invstd), capi.ptr(gamma), capi.ptr(beta), capi.BN_RELU, capi.stream_handle())
        assert torch.equal(y, y_ref)
        got = flat[numel:].view(torch.int32).cpu().numpy().view(np.uint32)
        want = np.packbits((flat[:numel] > 0).cpu().numpy().astype(np.uint8), bitorder="little")
        want = np.concatenate([want, np.zeros(-len(want) % 4, np.uint8)]).view(np.uint32)
        valid = np.full(words * 32, False); valid[:numel] = True
        keep = np.packbits(valid.astype(np.uint8), bitorder="little").view(np.uint32)  # bits past the end are unspecified
        assert np.array_equal(got & keep, want & keep)
        ref = capi.bn_backward(g, x, y_ref, mean, invstd, gamma, relu=True)
        dres_ref = torch.empty_like(x)
        dres = torch.empty_like(x)
        dx_ref, dx, dgb_ref, dgb = torch.empty_like(x), torch.empty_like(x), torch.empty(2, c, device="cuda"), torch.empty(2, c, device="cuda")
        capi.call("omt_bn_backward_add", capi.act(g), capi.act(x), capi.act(y_ref), capi.act(dx_ref), capi.act(dres_ref), n, c, h, w, capi.ptr(mean),
                  capi.ptr(invstd), capi.ptr(gamma), capi.ptr(dgb_ref), 1.0, capi.BN_RELU, capi.stream_handle())
        flat[:numel] = -1.0  # the values of y are gone: only the bits can tell the mask now
        capi.call("omt_bn_backward_add", capi.act(g), capi.act(x), capi.act(y), capi.act(dx), capi.act(dres), n, c, h, w, capi.ptr(mean), capi.ptr(invstd),
                  capi.ptr(gamma), capi.ptr(dgb), 1.0, capi.BN_RELU | capi.BN_MASKBITS, capi.stream_handle())
        assert torch.equal(dx, dx_ref) and torch.equal(dres, dres_ref) and torch.equal(dgb, dgb_ref)
        assert torch.equal(dx_ref, ref[0])


@pytest.mark.parametrize("cl", [False, True], ids=["nchw", "nhwc"])
def test_bn_large_mean_is_stable(capi, cl):
    """Shifted sums keep the variance accurate when |mean| >> std (bn_stats_part.wgsl:22-31)."""
    torch.manual_seed(1)
    x = torch.randn(32, 64, 28, 28) * 0.1 + 100.0
    xd = dev(x, cl)
    gamma, beta = torch.ones(64, device="cuda"), torch.zeros(64, device="cuda")
    rm, rv = torch.zeros(64, device="cuda"), torch.ones(64, device="cuda")
    y, mean, invstd = capi.bn_train(xd, gamma, beta, rm, rv)
    ref_var = x.double().var(dim=(0, 2, 3), unbiased=False)
    assert rel_err(host(invstd), (1 / torch.sqrt(ref_var + 1e-5)).float().numpy()) <= 1e-3
    assert rel_err(host(mean), x.double().mean(dim=(0, 2, 3)).float().numpy()) <= 1e-6


@pytest.mark.parametrize("cl", [False, True], ids=["nchw", "nhwc"])
@pytest.mark.parametrize("i", range(len(cases.MAXPOOL)))
def test_maxpool_golden(capi, golden, i, cl):
    k, s, p, hw = cases.MAXPOOL[i]
    x = dev(cases.rnd(700 + i, 2, 4, hw, hw), cl)
    y, idx = capi.maxpool_fwd(x, k, s, p)
    assert np.array_equal(host(y), golden[f"maxpool{i}_y"]) and np.array_equal(host(idx), golden[f"maxpool{i}_idx"])
    g = dev(cases.rnd(720 + i, *y.shape), cl)
    gx = capi.maxpool_bwd(g, idx, (hw, hw), k, s, p)
    assert rel_err(host(gx), golden[f"maxpool{i}_gx"]) <= TOL


def test_pool_edge_cases(capi):
    x = torch.zeros(1, 1, 4, 4)
    x[0, 0, 0, 1] = float("nan")
    y, idx = capi.maxpool_fwd(dev(x), 2, 2, 0)
    assert torch.isnan(y[0, 0, 0, 0]).item() and idx[0, 0, 0, 0].item() == 1
    ones = np.ones((1, 2, 4, 6), np.float32)
    y2, i2 = capi.pool2_fwd(dev(ones))
    ry, ri = oracle.c.pool2_fwd(ones)
    assert np.array_equal(host(i2), ri) and np.array_equal(host(y2), ry)
    xr = np.random.default_rng(3).standard_normal((3, 8, 6, 10)).astype(np.float32)
    for cl in (False, True):
        yr, ir = capi.pool2_fwd(dev(xr, cl))
        oy, oi = oracle.c.pool2_fwd(xr)
        assert np.array_equal(host(yr), oy) and np.array_equal(host(ir), oi)
        g = np.random.default_rng(4).standard_normal(oy.shape).astype(np.float32)
        assert np.array_equal(host(capi.pool2_bwd(dev(g, cl), ir, (6, 10))), oracle.c.pool2_bwd(g, oi, (6, 10)))


@pytest.mark.parametrize("i", range(len(cases.ADAPOOL)))
def test_adapool_golden(capi, golden, i):
    hw, o = cases.ADAPOOL[i]
    for cl in (False, True):
        x = dev(cases.rnd(800 + i, 2, 5, hw, hw), cl)
        y = capi.adaptive_avgpool_fwd(x, o)
        assert rel_err(host(y), golden[f"adapool{i}_y"]) <= TOL
        g = dev(cases.rnd(820 + i, *y.shape))
        assert rel_err(host(capi.adaptive_avgpool_bwd(g, (hw, hw))), golden[f"adapool{i}_gx"]) <= TOL


def test_avgpool_general_vs_aten(capi):
    torch.manual_seed(2)
    x = torch.randn(2, 6, 13, 11)
    for k, s, p, inc, div in [(2, 2, 0, True, 0), (3, 2, 1, True, 0), (3, 2, 1, False, 0), (3, 1, 1, True, 5)]:
        ref = torch.nn.functional.avg_pool2d(x, k, s, p, count_include_pad=inc, divisor_override=div or None)
        xr = x.clone().requires_grad_()
        r2 = torch.nn.functional.avg_pool2d(xr, k, s, p, count_include_pad=inc, divisor_override=div or None)
        g = torch.randn_like(r2)
        r2.backward(g)
        n, c, ih, iw = x.shape
        oh, ow = ref.shape[2:]
        xd = dev(x)
        y = torch.empty(n, c, oh, ow, device="cuda")
        pl = capi.Pool(k, k, s, s, p, p, 1, 1)
        capi.call("omt_avgpool_fwd", capi.act(xd), capi.act(y), n, c, ih, iw, oh, ow, pl, int(inc), div, capi.stream_handle())
        assert rel_err(host(y), ref.numpy()) <= TOL
        gx = torch.empty_like(xd)
        capi.call("omt_avgpool_bwd", capi.act(dev(g)), capi.act(gx), n, c, ih, iw, oh, ow, pl, int(inc), div, capi.stream_handle())
        assert rel_err(host(gx), xr.grad.numpy()) <= TOL


OPT = {"sgd_nesterov_wd": ("sgd", dict(lr=0.1, momentum=0.9, nesterov=True, weight_decay=1e-4)), "sgd_plain": ("sgd", dict(lr=0.05)),
       "sgd_damp_max": ("sgd", dict(lr=0.05, momentum=0.8, dampening=0.3, maximize=True)),
       "adam_wd": ("adam", dict(lr=1e-3, weight_decay=0.01)), "adamw": ("adam", dict(lr=1e-3, weight_decay=0.01, decoupled=True))}


@pytest.mark.parametrize("name", sorted(OPT))
def test_optimizers_golden(capi, golden, name):
    kind, kw = OPT[name]
    p = dev(cases.rnd(1000, 37, 11))
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    step = torch.zeros((), device="cuda")
    for it in range(3):
        g = dev(cases.rnd(1001 + it, 37, 11))
        if kind == "sgd":
            capi.sgd([p], [g], [m if kw.get("momentum") else None], first=(it == 0), **kw)
        else:
            step += 1
            capi.adam([p], [g], [m], [v], [step], **kw)
        assert rel_err(host(p), golden[f"optim_{name}_p{it}"]) <= 1e-5


def test_multi_tensor_optimizer_ragged_table(capi):
    """Many tensors of ragged sizes (incl. size 1, unaligned views and an empty one) in one launch vs the oracle."""
    rng = np.random.default_rng(7)
    sizes = [1, 3, 4096, 4097, 0, 12289, 64, 5]
    slab = torch.zeros(sum(sizes) + 64, device="cuda")
    ps, gs, ms, hp, hm, hg = [], [], [], [], [], []
    off = 1  # deliberately not 16-byte aligned
    for s in sizes:
        a, g, m = (rng.standard_normal(s).astype(np.float32) for _ in range(3))
        view = slab[off:off + s]
        view.copy_(torch.from_numpy(a))
        off += s
        ps.append(view); gs.append(dev(g)); ms.append(dev(m)); hp.append(a.copy()); hg.append(g); hm.append(m.copy())
    capi.sgd(ps, gs, ms, lr=0.1, momentum=0.9, weight_decay=1e-4, nesterov=True)
    for a, g, m, pd, md in zip(hp, hg, hm, ps, ms):
        if a.size == 0:
            continue
        oracle.c.sgd(a, g, m, 0.1, 0.9, 0.0, 1e-4, nesterov=True)
        assert rel_err(host(pd), a) <= 1e-6 and rel_err(host(md), m) <= 1e-6


def test_allocator_and_streams(capi):
    l = capi.lib()
    base_alloc, base_res = l.omt_memory_allocated(), l.omt_memory_reserved()
    s = l.omt_stream_create(1)
    p = l.omt_malloc(3 << 20, s)
    assert p and l.omt_memory_allocated() - base_alloc >= 3 << 20
    l.omt_free(p)
    assert l.omt_memory_allocated() == base_alloc and l.omt_memory_reserved() > base_res  # cached, not returned
    q = l.omt_malloc(3 << 20, s)
    assert q == p  # same size class on the same stream reuses the cached block
    src = np.arange(1000, dtype=np.float32)
    dst = np.zeros_like(src)
    capi.call("omt_memcpy_h2d", q, src.ctypes.data, src.nbytes, s)
    capi.call("omt_memcpy_d2h", dst.ctypes.data, q, src.nbytes, s)
    assert np.array_equal(src, dst)
    e = l.omt_event_create(0)
    capi.call("omt_event_record", e, s)
    capi.call("omt_event_sync", e)
    assert l.omt_event_query(e) == 1 and l.omt_stream_query(s) == 1
    l.omt_free(q)
    l.omt_empty_cache()
    assert l.omt_memory_reserved() <= base_res
    capi.call("omt_event_destroy", e)
    capi.call("omt_stream_destroy", s)
    assert l.omt_check_errors() == 0 and l.omt_launch_count() > 0


def test_act_copy_layout_change(capi):
    x = torch.randn(3, 10, 7, 5, device="cuda")
    y = torch.empty_like(x).contiguous(memory_format=torch.channels_last)
    capi.call("omt_act_copy", capi.act(x), capi.act(y), 3, 10, 7, 5, capi.stream_handle())
    assert torch.equal(x, y)
    z = torch.empty_like(x)
    capi.call("omt_act_copy", capi.act(y), capi.act(z), 3, 10, 7, 5, capi.stream_handle())
    assert torch.equal(x, z)


def _np_cross_entropy(x, t, w, ignore, reduction):
    """float64 restatement of log_softmax + nll_loss (the definition the reference's softmax/nll kernels implement,
    csrc/reduce.cpp:128-201): returns logp, loss, total weight, gradient of the logits for an upstream gradient of ones."""
    x = x.astype(np.float64)
    lp = x - x.max(1, keepdims=True)
    lp = lp - np.log(np.exp(lp).sum(1, keepdims=True))
    ww = np.ones(x.shape[1]) if w is None else w.astype(np.float64)
    live = t != ignore
    wr = np.where(live, ww[np.where(live, t, 0)], 0.0)
    rows = -wr * lp[np.arange(len(t)), np.where(live, t, 0)]
    tw = wr.sum()
    hot = np.zeros_like(lp)
    hot[np.arange(len(t)), np.where(live, t, 0)] = 1.0
    scale = wr / tw if reduction == 1 else wr
    dx = (np.exp(lp) - hot) * scale[:, None]
    loss = rows if reduction == 0 else rows.sum() / tw if reduction == 1 else rows.sum()
    return lp, loss, (0.0 if reduction == 0 else tw), dx


@pytest.mark.parametrize("reduction", [0, 1, 2], ids=["none", "mean", "sum"])
@pytest.mark.parametrize("rows,cols,weighted", [(256, 1000, False), (32, 10, True), (5, 3, False), (1, 1, False), (4099, 33, True), (3, 5000, False)])
def test_log_softmax_and_nll_loss(capi, rows, cols, weighted, reduction):
    """The four loss entry points and the fused pair against a float64 restatement and against aten on the CPU; rows with the
    ignored class, class weights, every reduction; one warp per row with ragged column counts; the sum over rows is ordered."""
    rng = np.random.default_rng(rows * 31 + cols)
    x = (rng.standard_normal((rows, cols)) * 3).astype(np.float32)
    t = rng.integers(0, cols, rows)
    ignore = -100 if cols == 1 else 1
    if rows > 2:
        t[1] = ignore
    w = (rng.random(cols) + 0.5).astype(np.float32) if weighted else None
    lp_ref, loss_ref, tw_ref, dx_ref = _np_cross_entropy(x, t, w, ignore, reduction)
    xd, td, wd = dev(x), dev(t), dev(w)
    sh, P = capi.stream_handle, capi.ptr
    lp = torch.empty_like(xd)
    capi.call("omt_log_softmax", P(xd), P(lp), rows, cols, sh())
    assert rel_err(host(lp), lp_ref) <= 1e-6
    loss = torch.full((rows if reduction == 0 else 1,), 7.0, device="cuda")
    tw = torch.full((1,), 7.0, device="cuda")
    capi.call("omt_nll_loss", P(lp), P(td), P(wd), P(loss), P(tw), rows, cols, ignore, reduction, sh())
    assert rel_err(host(loss).reshape(np.shape(loss_ref)), loss_ref) <= 1e-6 and abs(float(tw) - tw_ref) <= 1e-6 * max(1.0, tw_ref)
    # aten on the CPU agrees with the restatement (pins the restatement) and with the device
    xt = torch.tensor(x, requires_grad=True)
    red = ["none", "mean", "sum"][reduction]
    at_loss = torch.nn.functional.cross_entropy(xt, torch.tensor(t), weight=None if w is None else torch.tensor(w), ignore_index=ignore, reduction=red)
    at_loss.sum().backward()
    if np.all(np.isfinite(loss_ref)):
        assert rel_err(at_loss.detach().numpy().reshape(np.shape(loss_ref)), loss_ref) <= 1e-5
        assert rel_err(xt.grad.numpy(), dx_ref) <= 1e-5
    # fused forward: same three results from the logits in one launch, bit-identical to the two-step path
    lp2, loss2, tw2 = torch.empty_like(xd), torch.empty_like(loss), torch.empty_like(tw)
    n0 = capi.lib().omt_launch_count()
    capi.call("omt_softmax_nll", P(xd), P(td), P(wd), P(lp2), P(loss2), P(tw2), rows, cols, ignore, reduction, sh())
    assert capi.lib().omt_launch_count() - n0 == 1
    assert torch.equal(lp2, lp) and torch.equal(loss2, loss) and torch.equal(tw2, tw)
    # backward, two-step and fused
    g = torch.ones(rows if reduction == 0 else 1, device="cuda")
    dlp, dx, dx2 = torch.empty_like(xd), torch.empty_like(xd), torch.empty_like(xd)
    capi.call("omt_nll_loss_backward", P(g), P(td), P(wd), P(tw), P(dlp), rows, cols, ignore, reduction, sh())
    capi.call("omt_log_softmax_backward", P(dlp), P(lp), P(dx), rows, cols, sh())
    capi.call("omt_softmax_nll_backward", P(g), P(lp), P(td), P(wd), P(tw), P(dx2), rows, cols, ignore, reduction, sh())
    if np.all(np.isfinite(dx_ref)):
        assert rel_err(host(dx), dx_ref) <= 1e-5 and rel_err(host(dx2), dx_ref) <= 1e-5
    # the fused forward is deterministic (ordered sum over rows by the last block)
    capi.call("omt_softmax_nll", P(xd), P(td), P(wd), P(lp2), P(loss2), P(tw2), rows, cols, ignore, reduction, sh())
    assert torch.equal(loss2, loss)


def test_nll_loss_refuses_bad_arguments(capi):
    x = torch.zeros(4, 3, device="cuda")
    t = torch.zeros(4, dtype=torch.int64, device="cuda")
    out = torch.zeros(4, device="cuda")
    P, sh = capi.ptr, capi.stream_handle
    with pytest.raises(capi.OmtError):
        capi.call("omt_nll_loss", P(x), P(t), None, P(out), P(out), 4, 3, -100, 3, sh())
    with pytest.raises(capi.OmtError):
        capi.call("omt_log_softmax", P(x), P(x), 0, 3, sh())
    # a target outside [0, cols): NaN loss, zero gradient row, no fault
    t[2] = 9
    lp, loss, tw, dx = torch.empty_like(x), torch.zeros(1, device="cuda"), torch.zeros(1, device="cuda"), torch.empty_like(x)
    capi.call("omt_softmax_nll", P(x), P(t), None, P(lp), P(loss), P(tw), 4, 3, -100, 1, sh())
    assert torch.isnan(loss).all() and float(tw) == 3.0
    capi.call("omt_softmax_nll_backward", P(torch.ones(1, device="cuda")), P(lp), P(t), None, P(tw), P(dx), 4, 3, -100, 1, sh())
    assert torch.all(dx[2] == 0) and torch.isfinite(dx).all()


@pytest.mark.parametrize("shape", [(2, 8, 14, 3, 1, 1), (3, 12, 23, 3, 1, 1), (2, 16, 29, 5, 1, 2), (2, 8, 31, 5, 2, 2), (2, 8, 30, 3, 2, 1),
                                   (1, 4, 33, 7, 1, 3), (2, 4, 35, 7, 2, 3), (2, 96, 28, 3, 2, 1), (2, 8, 19, 3, 1, 0), (2, 8, 22, 5, 2, 0),
                                   (2, 8, 12, 3, 1, 2), (1, 40, 9, 5, 1, 2), (4, 24, 57, 3, 1, 1), (2, 8, 6, 5, 2, 2), (1, 4, 3, 3, 1, 1)],
                         ids=lambda s: "n%d_c%d_hw%d_k%d_s%d_p%d" % s)
def test_depthwise_strip_kernels_vs_aten(capi, shape):
    """Channels-last depthwise forward, input gradient (stride 1: mirrored forward; stride 2: parity gather) and weight gradient
    for 3x3 / 5x5 / 7x7, strides 1 and 2: the kernels that walk strips of output rows with partial sums in registers. Widths
    and heights that are not multiples of the strip size, pads 0..ks-1, images smaller than one strip; bias + ReLU epilogue.
    Against float64 aten on the CPU (the reference's own oracle for dw_fwd / dw_gin / dw_gwt)."""
    n, c, hw, ks, s, p = shape
    torch.manual_seed(hw * 7 + ks)
    x = torch.randn(n, c, hw, hw + 3)
    w = torch.randn(c, 1, ks, ks) * 0.3
    b = torch.randn(c)
    oh, ow = (hw + 2 * p - ks) // s + 1, (hw + 3 + 2 * p - ks) // s + 1
    gy = torch.randn(n, c, oh, ow)
    x64 = x.double().requires_grad_()
    w64 = w.double().requires_grad_()
    y64 = torch.nn.functional.conv2d(x64, w64, b.double(), s, p, groups=c)
    y64.backward(gy.double())
    xd, wd, bd, gd = dev(x, True), dev(w), dev(b), dev(gy, True)
    y = capi.dw_fwd(xd, wd, bd, s, p, flags=capi.EPI_RELU, cl=True)
    assert rel_err(host(y), y64.detach().relu().float().numpy()) <= 2e-6
    y = capi.dw_fwd(xd, wd, None, s, p, cl=True)
    assert rel_err(host(y), (y64.detach() - b.double().view(1, -1, 1, 1)).float().numpy()) <= 2e-6
    dx = capi.dw_dgrad(gd, wd, (hw, hw + 3), s, p, cl=True)
    assert rel_err(host(dx), x64.grad.float().numpy()) <= 2e-6
    dw = capi.dw_wgrad(xd, gd, ks, s, p, scale=0.5)
    assert rel_err(2 * host(dw), w64.grad.float().numpy()) <= 1e-5
    capi.call("omt_sync")


@pytest.mark.parametrize("cl", [False, True], ids=["nchw", "nhwc"])
@pytest.mark.parametrize("shape", [(4, 3, 64, 63, 11, 4, 2), (2, 4, 32, 17, 3, 1, 1), (2, 1, 32, 20, 5, 2, 2), (3, 3, 96, 30, 7, 2, 3),
                                   (2, 3, 64, 33, 7, 2, 0), (2, 2, 32, 9, 3, 3, 1), (1, 3, 32, 12, 1, 1, 0)],
                         ids=lambda s: "n%d_ci%d_co%d_hw%d_k%d_s%d_p%d" % s)
def test_input_gradient_of_a_first_layer_by_taps(capi, shape, cl):
    """Input gradient for <= 4 input channels: one tensor-core product over all taps, then the col2im gather (stride phases of
    csrc/conv.cpp:78-95); gy in either layout, dx NCHW; against float64 aten and the exact-fp32 kernel; the kernels that ran
    are the tensor-core ones."""
    n, ci, co, hw, ks, s, p = shape
    torch.manual_seed(co + hw)
    x = torch.randn(n, ci, hw, hw + 2, dtype=torch.float64, requires_grad=True)
    w = torch.randn(co, ci, ks, ks) * 0.1
    y = torch.nn.functional.conv2d(x, w.double(), None, s, p)
    gy = torch.randn(y.shape)
    y.backward(gy.double())
    before = capi.kernel_counts()
    got = capi.conv_dgrad(dev(gy, cl), dev(w), (hw, hw + 2), s, p)
    capi.call("omt_sync")
    after = capi.kernel_counts()
    assert rel_err(host(got), x.grad.float().numpy()) <= 2e-5
    assert after.get("conv_dgrad_col2im", 0) == before.get("conv_dgrad_col2im", 0) + 1, after
    exact = capi.conv_dgrad(dev(gy, cl), dev(w), (hw, hw + 2), s, p, flags=capi.FORCE_SIMT)
    assert rel_err(host(got), host(exact)) <= 2e-5
