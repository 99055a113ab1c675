"""The "omarchy_mac_torch" PyTorch device end to end on a B200: storage semantics, the aten overrides through autograd,
fused stacks, fused optimizers, whole-model training against the golden loss curves (the reference's acceptance test,
tools/acceptance.py) and the torch.compile backend. Run with -m gpu."""
import copy
import io

import numpy as np
import pytest
import torch
import torch.nn.functional as F
from torch import nn

import cases
from conftest import TOL, rel_err

pytestmark = pytest.mark.gpu
D = "omarchy_mac_torch"


@pytest.fixture(scope="module")
def omt():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    import omarchy_mac_torch_b200 as m
    m.DEVICE  # registers the device
    return m


def e(a, b):
    return rel_err(a.detach().cpu().numpy(), b.detach().cpu().numpy())


def test_storage_semantics(omt):
    """notes/scripts/storage_check.py: save/load, deepcopy, dtype views, generator determinism, events."""
    x = torch.randn(7, 5)
    xd = x.to(D)
    assert xd.device.type == D and torch.equal(xd.cpu(), x)
    assert torch.equal(copy.deepcopy(xd).cpu(), x)
    buf = io.BytesIO()
    torch.save({"t": xd}, buf)
    buf.seek(0)
    assert torch.equal(torch.load(buf, map_location="cpu")["t"], x)
    buf.seek(0)
    back = torch.load(buf)["t"]
    assert back.device.type == D and torch.equal(back.cpu(), x)
    assert torch.equal(xd.view(torch.int32).cpu(), x.view(torch.int32))
    assert torch.equal(xd.t()[1:3].contiguous().cpu(), x.t()[1:3].contiguous())
    assert xd.sum().item() == pytest.approx(x.sum().item(), rel=1e-5, abs=1e-5 * x.abs().sum().item())
    y = torch.arange(10, device=D)
    assert y.dtype == torch.int64 and y.cpu().tolist() == list(range(10))
    torch.manual_seed(3)
    a = torch.empty(64, device=D).normal_()
    torch.manual_seed(3)
    b = torch.empty(64, device=D).normal_()
    assert torch.equal(a.cpu(), b.cpu()) and a.cpu().std() > 0.5
    ev = torch.Event(D)
    ev.record()
    ev.synchronize()
    assert ev.query()
    z = torch.zeros(3, device=D)
    z.resize_(6)
    assert z.shape == (6,)
    before = omt.memory_allocated()
    big = torch.empty(1 << 20, device=D)
    assert omt.memory_allocated() >= before + (4 << 20)
    del big
    omt.empty_cache()
    omt.synchronize()


CONV = {k: v for k, v in cases.conv_cases().items()}


@pytest.mark.parametrize("name", sorted(CONV))
def test_conv_modules_through_autograd(omt, golden, name):
    """notes/scripts/conv_kinds_check.py and alexnet_ops_check.py: nn.Conv2d forward + backward on the device."""
    seed, n, ci, co, ks, s, p, hw, groups, bias = CONV[name]
    x, w, b, gy = cases.conv_inputs(*CONV[name])
    omt.FALLBACKS.clear()
    conv = nn.Conv2d(ci, co, ks, stride=s, padding=p, groups=groups, bias=bias)
    with torch.no_grad():
        conv.weight.copy_(w)
        if bias:
            conv.bias.copy_(b)
    conv = conv.to(D)
    xd = x.to(D).requires_grad_()
    y = conv(xd)
    y.backward(gy.to(D))
    assert rel_err(y.detach().cpu().numpy(), golden[f"{name}_y"]) <= TOL
    assert rel_err(xd.grad.cpu().numpy(), golden[f"{name}_dx"]) <= TOL
    assert rel_err(conv.weight.grad.cpu().numpy(), golden[f"{name}_dw"]) <= TOL
    if bias:
        assert rel_err(conv.bias.grad.cpu().numpy(), golden[f"{name}_db"]) <= TOL
    assert not omt.FALLBACKS, dict(omt.FALLBACKS)
    # channels-last input keeps working and stays channels-last
    ycl = conv(x.to(D).contiguous(memory_format=torch.channels_last))
    assert rel_err(ycl.detach().cpu().numpy(), golden[f"{name}_y"]) <= TOL


def test_unsupported_conv_is_recorded_and_still_correct(omt):
    omt.FALLBACKS.clear()
    x, w = torch.randn(2, 4, 9, 9), torch.randn(6, 4, 3, 3)
    y = F.conv2d(x.to(D), w.to(D), dilation=2)
    assert e(y, F.conv2d(x, w, dilation=2)) <= TOL
    assert any(k.startswith("convolution (") for k in omt.FALLBACKS.keys())
    omt.FALLBACKS.clear()


@pytest.mark.parametrize("i", range(len(cases.BN)))
def test_batchnorm_module(omt, golden, i):
    n, c, h, w = cases.BN[i]
    G = lambda k: golden[f"bn{i}_{k}"]
    bn = nn.BatchNorm2d(c)
    with torch.no_grad():
        bn.weight.copy_(cases.rnd(910 + i, c)); bn.bias.copy_(cases.rnd(920 + i, c))
        bn.running_mean.copy_(cases.rnd(930 + i, c)); bn.running_var.copy_(cases.rnd(940 + i, c).abs() + 0.5)
    bn = bn.to(D)
    x = (cases.rnd(900 + i, n, c, h, w) * 2 + 3).to(D).requires_grad_()
    bn.eval()
    assert rel_err(bn(x).detach().cpu().numpy(), G("yeval")) <= TOL
    bn.train()
    y = bn(x)
    y.backward(cases.rnd(950 + i, n, c, h, w).to(D))
    for got, key in ((y, "y"), (x.grad, "dx"), (bn.weight.grad, "dgamma"), (bn.bias.grad, "dbeta"), (bn.running_mean, "rm"), (bn.running_var, "rv")):
        assert rel_err(got.detach().cpu().numpy(), G(key)) <= TOL, key
    assert not omt.FALLBACKS, dict(omt.FALLBACKS)


def test_pools_through_autograd(omt, golden):
    for i, (k, s, p, hw) in enumerate(cases.MAXPOOL):
        x = cases.rnd(700 + i, 2, 4, hw, hw).to(D).requires_grad_()
        y = F.max_pool2d(x, k, s, p)
        y.backward(cases.rnd(720 + i, *y.shape).to(D))
        assert np.array_equal(y.detach().cpu().numpy(), golden[f"maxpool{i}_y"])
        assert rel_err(x.grad.cpu().numpy(), golden[f"maxpool{i}_gx"]) <= TOL
    for i, (hw, o) in enumerate(cases.ADAPOOL):
        x = cases.rnd(800 + i, 2, 5, hw, hw).to(D).requires_grad_()
        y = F.adaptive_avg_pool2d(x, o)
        y.backward(cases.rnd(820 + i, *y.shape).to(D))
        assert rel_err(y.detach().cpu().numpy(), golden[f"adapool{i}_y"]) <= TOL
        assert rel_err(x.grad.cpu().numpy(), golden[f"adapool{i}_gx"]) <= TOL
    assert not omt.FALLBACKS, dict(omt.FALLBACKS)


OPT = {"sgd_nesterov_wd": lambda p: torch.optim.SGD(p, lr=0.1, momentum=0.9, nesterov=True, weight_decay=1e-4),
       "sgd_plain": lambda p: torch.optim.SGD(p, lr=0.05),
       "sgd_damp_max": lambda p: torch.optim.SGD(p, lr=0.05, momentum=0.8, dampening=0.3, maximize=True),
       "adam_wd": lambda p: torch.optim.Adam(p, lr=1e-3, weight_decay=0.01),
       "adamw": lambda p: torch.optim.AdamW(p, lr=1e-3, weight_decay=0.01)}


@pytest.mark.parametrize("name", sorted(OPT))
def test_torch_optim_takes_the_fused_kernels(omt, golden, name):
    from omarchy_mac_torch_b200.native import core
    p = nn.Parameter(cases.rnd(1000, 37, 11).to(D))
    opt = OPT[name]([p])
    assert opt.defaults.get("fused") is True  # optim.py wrapped the constructor
    core.kernel_counts(True)
    for it in range(3):
        p.grad = cases.rnd(1001 + it, 37, 11).to(D)
        opt.step()
        assert rel_err(p.detach().cpu().numpy(), golden[f"optim_{name}_p{it}"]) <= 1e-5
    kc = core.kernel_counts(False)
    assert kc.get("sgd_multi", 0) + kc.get("adam_multi", 0) == 3
    assert not omt.FALLBACKS, dict(omt.FALLBACKS)


def _train(model, x, y, kind, steps=5):
    opt = {"sgd": lambda p: torch.optim.SGD(p, lr=0.01, momentum=0.9), "adam": lambda p: torch.optim.Adam(p, lr=1e-3)}[kind](model.parameters())
    out = []
    for _ in range(steps + 1):
        loss = F.cross_entropy(model(x), y)
        opt.zero_grad()
        loss.backward()
        opt.step()
        out.append(loss.item())
    return out


def _assert_losses_track(dev_, cpu, exact, label):
    """Per-step relative loss difference <= 1e-3 wherever the run is that well conditioned. Where it is not (a loss that
    collapses by orders of magnitude in a few steps multiplies rounding differences by 30-100 per step), the bound for a
    step is 10x the distance between the CPU fp32 run and a CPU float64 run of the same model, and the device may be
    measured against either: it has to be as close to the exact curve as fp32 arithmetic allows."""
    def rel(a, b):
        return [abs(p - q) / max(abs(p), 1e-6) for p, q in zip(a, b)]
    for step, (d_cpu, d_exact, n) in enumerate(zip(rel(cpu, dev_), rel(exact, dev_), rel(exact, cpu))):
        bound = max(1e-3, 10 * n)
        assert min(d_cpu, d_exact) <= bound, (label, step, d_cpu, d_exact, bound, cpu, dev_, exact)


@pytest.mark.parametrize("name,tol", [("plaincnn", 1e-3), ("separablecnn", 1e-3), ("mobilenetv3", 1e-3), ("resnet18", 1e-2)])
def test_training_matches_reference_loss_curves(omt, golden_losses, name, tol):
    """tools/acceptance.py: 1 warm-up + 5 steps from the same seed; loss curves must match the CPU curves of the
    reference's own model classes (tests/golden/losses.json) with no op off the device kernels. ResNet-18's loss falls
    to 0.04 within 5 steps at lr 0.01, which amplifies rounding differences: the reference itself records 1.6e-3 there
    (results/acceptance.json) and accepts < 1e-2 (tools/acceptance.py:103); here it additionally has to stay within the
    fp32 noise floor measured against a float64 run."""
    from omarchy_mac_torch_b200 import models
    cls = {"plaincnn": models.PlainCNN, "separablecnn": models.SeparableCNN, "mobilenetv3": models.MobileNetV3Small, "resnet18": models.ResNet18}[name]
    g = golden_losses[name]
    torch.manual_seed(0)
    model = cls()
    for m in model.modules():
        if isinstance(m, nn.Dropout):
            m.p = 0.0
    assert sum(p.numel() for p in model.parameters()) == g["params"]
    x, y = torch.randn(*g["shape"]), torch.randint(0, g["classes"], (g["shape"][0],))
    exact_model = copy.deepcopy(model).double() if tol > 1e-3 else None
    omt.FALLBACKS.clear()
    losses = _train(model.to(D), x.to(D), y.to(D), g["optimizer"])
    assert not omt.FALLBACKS, dict(omt.FALLBACKS)
    diff = max(abs(a - b) / max(abs(b), 1e-6) for a, b in zip(losses, g["losses"]))
    assert diff <= tol, (diff, losses, g["losses"])
    if exact_model is not None:
        _assert_losses_track(losses, g["losses"], _train(exact_model, x.double(), y, g["optimizer"]), name)


FULL_SIZE_CONFIGS = {
    # the three small benchmark configurations at full size: (model factory, input shape, classes, optimizer factory)
    "c2_plaincnn": (lambda m: m.PlainCNN3(), (128, 3, 32, 32), 10, lambda p: torch.optim.SGD(p, lr=0.05, momentum=0.9)),
    "c3_resnet18": (lambda m: m.kaiming_normal_convs(m.ResNet18(num_classes=1000)), (32, 3, 64, 64), 1000,
                    lambda p: torch.optim.SGD(p, lr=0.1, momentum=0.9, weight_decay=1e-4)),
    "c4_mobilenetv3": (lambda m: m.MobileNetV3SE(), (32, 3, 224, 224), 1000, lambda p: torch.optim.AdamW(p, lr=1e-3, weight_decay=0.01)),
}


@pytest.mark.parametrize("name", sorted(FULL_SIZE_CONFIGS))
def test_baseline_configs_five_step_losses_match_cpu(omt, name):
    """The three-block CNN (batch 128), ResNet-18 (batch 32, 64x64, lr 0.1) and MobileNetV3-Small-SE (batch 32, 224x224, AdamW) at
    full size: 1 warm-up + 5 training steps on the device (tensor-core convs, channels-last,
    fused stacks where they apply) against the same run on the CPU, no op off the device.

    The bound is 1e-3 relative per step wherever the training run itself is that well conditioned. ResNet-18 is not:
    at lr 0.1 its loss falls from 7.1 to 0.06 in five steps and every step multiplies rounding differences by 30-100
    (the CPU run with 1 thread against 16 threads already differs by 5e-3 at step 4). So each step's bound is
    max(1e-3, 10 x the CPU fp32 run's own distance from a CPU float64 run of the same model), and the device is
    measured against the float64 run as well: it has to be as close to the exact curve as fp32 arithmetic allows."""
    from omarchy_mac_torch_b200 import models
    make, shape, classes, make_opt = FULL_SIZE_CONFIGS[name]
    torch.manual_seed(0)
    ref = make(models)
    mod, ref64 = copy.deepcopy(ref).to(D), copy.deepcopy(ref).double()
    x, y = torch.randn(*shape), torch.randint(0, classes, (shape[0],))
    omt.FALLBACKS.clear()

    def run(model, xx, yy):
        opt, out = make_opt(model.parameters()), []
        for _ in range(6):
            loss = F.cross_entropy(model(xx), yy)
            opt.zero_grad()
            loss.backward()
            opt.step()
            out.append(loss.item())
        return out

    def rel(a, b):
        return [abs(p - q) / max(abs(p), 1e-6) for p, q in zip(a, b)]

    cpu, dev_ = run(ref, x, y), run(mod, x.to(D), y.to(D))
    assert not omt.FALLBACKS, dict(omt.FALLBACKS)
    if max(rel(cpu, dev_)) <= 1e-3:
        return
    assert name == "c3_resnet18", (cpu, dev_)  # the only ill-conditioned configuration
    _assert_losses_track(dev_, cpu, run(ref64, x.double(), y), name)
    assert max(rel(cpu, dev_)[:2]) <= 1e-3


def test_fused_stacks_train_eval_and_accumulate(omt):
    """notes/scripts/native_final_check.py: fused stacks in training, eval with folded BN, gradient accumulation."""
    from omarchy_mac_torch_b200 import models, stacks
    for cls, bias in ((models.SeparableCNN, None), (models.PlainCNN, None), (models.PlainCNN3, True), (models.PlainCNN3, False)):
        torch.manual_seed(0)
        ref = cls() if bias is None else cls(bias=bias)
        mod = copy.deepcopy(ref).to(D)
        o1, o2 = torch.optim.SGD(ref.parameters(), 0.01, momentum=0.9), torch.optim.SGD(mod.parameters(), 0.01, momentum=0.9)
        shape = (64, 3, 32, 32) if cls is models.PlainCNN3 else (64, 1, 28, 28)
        X, y = torch.rand(*shape), torch.randint(0, 10, (64,))
        for _ in range(3):
            l1 = F.cross_entropy(ref(X), y, label_smoothing=0.1); o1.zero_grad(); l1.backward(); o1.step()
            l2 = F.cross_entropy(mod(X.to(D)), y.to(D), label_smoothing=0.1); o2.zero_grad(); l2.backward(); o2.step()
            assert abs(l1.item() - l2.item()) <= 1e-3 * abs(l1.item())
        assert type(mod.features) is stacks.FusedSequential
        if cls is models.PlainCNN3:  # a conv -> BatchNorm+ReLU -> max pool block is three launches forward
            from omarchy_mac_torch_b200.native import core
            core.kernel_counts(True)
            mod(X.to(D)); ref(X)  # (both, so that the running statistics compared below stay in step)
            kc = core.kernel_counts(True)
            # (the last block's conv has few output tiles and splits its reduction over CTAs: its statistics come from a
            # separate pass over y, the other two from the conv epilogue)
            assert kc.get("bn_stats_from_partials", 0) == 2 and kc.get("bn_stats_part_nhwc", 0) == 1 and kc.get("bn_apply_pool2", 0) == 3, kc
            assert not any(k in ("pool2_fwd", "bn_apply") for k in kc), kc
        # (SGD at a step size where these runs converge rather than the reference script's Adam: Adam turns
        # rounding-noise gradients into +-lr steps, which makes parameter comparisons meaningless; the Adam kernels are
        # compared step by step in the optimizer tests. Error is taken per tensor against its largest element: BatchNorm
        # biases start at zero and hold sums with heavy cancellation, and one max-pool window whose two largest values
        # differ by less than fp32 rounding sends its gradient to the other element.)
        for a, b in zip(ref.parameters(), mod.parameters()):
            assert (b.detach().cpu() - a.detach()).abs().max() <= 2e-3 * a.detach().abs().max() + 1e-5
        for a, b in zip(ref.buffers(), mod.buffers()):
            assert e(b.float(), a.float()) <= 1e-3  # running stats and num_batches_tracked
        ref.eval(); mod.eval()
        Xe = torch.rand(50, *shape[1:])
        with torch.no_grad():
            assert e(mod(Xe.to(D)), ref(Xe)) <= 1e-3  # eval plan: BN folded into the conv weights
    # two backward passes accumulate into .grad (the plan must not overwrite gradients that are still alive). Several of
    # this model's gradients are zero in exact arithmetic (the scale of a BatchNorm whose output feeds another
    # BatchNorm through a linear layer), so what either fp32 implementation holds there is rounding noise: each tensor
    # is measured against a float64 run, and must be within 1e-3 or 4x the CPU fp32 run's own error, whichever is larger.
    torch.manual_seed(0)
    ref = models.SeparableCNN(); mod = copy.deepcopy(ref).to(D); exact = copy.deepcopy(ref).double()
    for seed in (1, 2):
        g = torch.Generator().manual_seed(seed)
        xb, yb = torch.rand(64, 1, 28, 28, generator=g), torch.randint(0, 10, (64,), generator=g)
        F.cross_entropy(ref(xb), yb).backward()
        F.cross_entropy(exact(xb.double()), yb).backward()
        F.cross_entropy(mod(xb.to(D)), yb.to(D)).backward()
    for a, b, c in zip(ref.parameters(), mod.parameters(), exact.parameters()):
        assert e(b.grad.double(), c.grad) <= max(1e-3, 4 * e(a.grad.double(), c.grad))
    assert not omt.FALLBACKS, dict(omt.FALLBACKS)


def test_omt_ops_device_vs_composite(omt):
    """The omt:: custom ops: device implementation against their composite definition run on the CPU."""
    omt_ops = torch.ops.omt
    x = torch.randn(8, 6, 5, 7) * 2 + 1
    w, b, rm, rv = torch.randn(6), torch.randn(6), torch.randn(6), torch.rand(6) + 0.5
    ref = omt_ops.bn_relu_train(x, w, b, rm, rv, 0.1, 1e-5)
    dev = omt_ops.bn_relu_train(*(t.to(D) for t in (x, w, b, rm, rv)), 0.1, 1e-5)
    for r, d in zip(ref, dev):
        assert e(d, r) <= TOL
    assert len({t.untyped_storage().data_ptr() for t in dev}) == 5  # no two outputs alias (the schema declares none)
    g = torch.randn_like(x)
    rb = omt_ops.bn_relu_backward(g, x, ref[0], w, ref[1], ref[2], [True, True, True])
    db = omt_ops.bn_relu_backward(g.to(D), x.to(D), dev[0], w.to(D), dev[1], dev[2], [True, True, True])
    for r, d in zip(rb, db):
        assert e(d, r) <= TOL
    # the residual-block variants, in NCHW and (8 channels) channels-last
    for xs, cl in ((x, False), (torch.randn(4, 8, 6, 5) * 2 + 1, True)):
        c = xs.shape[1]
        w_, b_, rm_, rv_ = torch.randn(c), torch.randn(c), torch.randn(c), torch.rand(c) + 0.5
        res, g_ = torch.randn_like(xs), torch.randn_like(xs)
        fmt = torch.channels_last if cl else torch.contiguous_format
        xd, resd, gd = (t.to(D).contiguous(memory_format=fmt) for t in (xs, res, g_))
        ref = omt_ops.bn_add_relu_train(xs, res, w_, b_, rm_, rv_, 0.1, 1e-5)
        dev = omt_ops.bn_add_relu_train(xd, resd, *(t.to(D) for t in (w_, b_, rm_, rv_)), 0.1, 1e-5)
        for r, d in zip(ref, dev):
            assert e(d, r) <= TOL
        rb = omt_ops.bn_add_relu_backward(g_, xs, ref[0], w_, ref[1], ref[2], [True, True, True])
        db = omt_ops.bn_add_relu_backward(gd, xd, dev[0], w_.to(D), dev[1], dev[2], [True, True, True])
        assert len(db) == 4
        for r, d in zip(rb, db):
            assert e(d, r) <= TOL
    # input gradient accumulated into an existing gradient: tensor-core geometry (channels-last) and a fallback one (ci = 6)
    for ci_, co_, cl in ((16, 24, True), (6, 5, False)):
        xa, wa = torch.randn(3, ci_, 9, 9), torch.randn(co_, ci_, 3, 3) * 0.2
        ga, acc0 = torch.randn(3, co_, 9, 9), torch.randn(3, ci_, 9, 9)
        fmt = torch.channels_last if cl else torch.contiguous_format
        r_acc, r_w = omt_ops.conv_backward_acc(ga, xa, wa, acc0.clone(), [1, 1], [1, 1], True)
        accd = acc0.to(D).contiguous(memory_format=fmt)
        d_acc, d_w = omt_ops.conv_backward_acc(ga.to(D).contiguous(memory_format=fmt), xa.to(D).contiguous(memory_format=fmt), wa.to(D), accd,
                                               [1, 1], [1, 1], True)
        assert d_acc.untyped_storage().data_ptr() == accd.untyped_storage().data_ptr()
        assert e(d_acc, r_acc) <= TOL and e(d_w, r_w) <= TOL
    # conv feeding a training BatchNorm (+ identity)(+ ReLU): statistics from the conv epilogue on tensor-core geometries
    # (16 -> 32 channels, channels-last), from a separate pass otherwise (6 -> 5 channels)
    from omarchy_mac_torch_b200.native import core
    for ci_, co_, cl, bias_, with_res, act_ in ((16, 32, True, False, False, 1), (16, 32, True, True, True, 1), (16, 32, True, False, False, 0),
                                                 (3, 32, False, True, False, 1), (6, 5, False, True, True, 1)):
        xa, wa = torch.randn(32, ci_, 20, 20), torch.randn(co_, ci_, 3, 3) * 0.2  # 100 row tiles: no reduction split over CTAs
        ba = torch.randn(co_) if bias_ else None
        ra = torch.randn(32, co_, 20, 20) if with_res else None
        g_, b_, rm_, rv_ = torch.randn(co_), torch.randn(co_), torch.randn(co_), torch.rand(co_) + 0.5
        fmt = torch.channels_last if cl else torch.contiguous_format
        ref = omt_ops.conv_bn_train(xa, wa, ba, [1, 1], [1, 1], ra, g_, b_, rm_, rv_, 0.1, 1e-5, act_)
        core.kernel_counts(True)
        dev = omt_ops.conv_bn_train(xa.to(D).contiguous(memory_format=fmt), wa.to(D), None if ba is None else ba.to(D), [1, 1], [1, 1],
                                    None if ra is None else ra.to(D).contiguous(memory_format=fmt), g_.to(D), b_.to(D), rm_.to(D), rv_.to(D), 0.1, 1e-5, act_)
        kc = core.kernel_counts(True)
        assert (kc.get("bn_stats_from_partials", 0) == 1) == (co_ % 4 == 0), kc
        assert len(dev) == 6 and len({t.untyped_storage().data_ptr() for t in dev}) == 6
        for r, d in zip(ref, dev):
            assert e(d, r) <= TOL
    cw, cb = torch.randn(5, 6, 3, 3) * 0.2, torch.randn(5)
    assert e(omt_ops.conv_act(x.to(D), cw.to(D), cb.to(D), [1, 1], [1, 1], 1), omt_ops.conv_act(x, cw, cb, [1, 1], [1, 1], 1)) <= TOL
    w5, b5, rm5, rv5 = torch.randn(5), torch.randn(5), torch.randn(5), torch.rand(5) + 0.5
    r = omt_ops.conv_bn_act_eval(x, cw, cb, w5, b5, rm5, rv5, 1e-5, [2, 2], [1, 1], 1)
    d = omt_ops.conv_bn_act_eval(*(t.to(D) for t in (x, cw, cb, w5, b5, rm5, rv5)), 1e-5, [2, 2], [1, 1], 1)
    assert e(d, r) <= TOL
    assert not omt.FALLBACKS, dict(omt.FALLBACKS)


def test_linear_layers_run_on_the_conv_gemm_kernels(omt):
    """aten::mm / aten::addmm on the device (csrc/linalg.cpp:62-92 of the reference): nn.Linear forward, input gradient and
    weight gradient are the three layouts omt_gemm maps onto the forward / input-gradient / weight-gradient kernels;
    against float64 on the CPU. Sizes: the AlexNet classifier's first layer at batch 16, the MobileNetV3 head, ragged
    sizes that leave the tensor-core path (exact-fp32 kernels), and operand layouts that need a copy."""
    from omarchy_mac_torch_b200.native import core
    torch.manual_seed(0)
    omt.FALLBACKS.clear()
    core.bridge_counts(True)
    for batch, fin, fout in ((16, 9216, 4096), (32, 576, 1024), (32, 1024, 1000), (256, 2048, 1000), (7, 37, 11), (64, 64, 8)):
        lin = nn.Linear(fin, fout)
        x = torch.randn(batch, fin)
        gy = torch.randn(batch, fout)
        x64 = x.double().requires_grad_()
        lin64 = copy.deepcopy(lin).double()
        y64 = lin64(x64)
        y64.backward(gy.double())
        lind = copy.deepcopy(lin).to(D)
        xd = x.to(D).requires_grad_()
        core.kernel_counts(True)
        yd = lind(xd)
        yd.backward(gy.to(D))
        kc = core.kernel_counts(True)
        assert e(yd, y64.float()) <= TOL and e(xd.grad, x64.grad.float()) <= TOL, (batch, fin, fout)
        assert e(lind.weight.grad, lin64.weight.grad.float()) <= TOL and e(lind.bias.grad, lin64.bias.grad.float()) <= TOL, (batch, fin, fout)
        if fin % 32 == 0 and fout % 8 == 0:  # tensor-core geometries: forward, input gradient and weight gradient kernels all ran
            assert sum(v for k, v in kc.items() if k.startswith(("conv_tc_1", "conv_tc_2"))) >= 2 and sum(v for k, v in kc.items() if k.startswith(("wgrad_tc_1", "wgrad_tc_2"))) >= 1, kc
    # plain products in every combination of operand layouts, and addmm forms outside the nn.Linear case (served by the bridge)
    a, b = torch.randn(48, 40), torch.randn(40, 24)
    want = (a.double() @ b.double()).float()
    ad, bd = a.to(D), b.to(D)
    for aa in (ad, ad.t().contiguous().t()):
        for bb in (bd, bd.t().contiguous().t()):
            assert e(aa @ bb, want) <= TOL
    assert e(torch.mm(ad[:, ::2], bd[::2]), (a[:, ::2].double() @ b[::2].double()).float()) <= TOL  # strided: copied
    bias = torch.randn(48, 24)
    assert e(torch.addmm(bias.to(D), ad, bd, beta=0.5, alpha=2.0), torch.addmm(bias, a, b, beta=0.5, alpha=2.0)) <= TOL
    bc = core.bridge_counts(True)
    assert not any(k.startswith("aten::mm") for k in bc), bc
    assert all("mm" not in k or "addmm" in k for k in omt.FALLBACKS), dict(omt.FALLBACKS)
    omt.FALLBACKS.clear()


def test_cross_entropy_on_the_device_eager_and_compiled(omt):
    """F.cross_entropy lowers to _log_softmax + nll_loss_forward (+ their backward ops): all four run on the library's kernels
    (reference csrc/reduce.cpp:141-201), and the compile backend fuses each pair into one launch; losses and gradients
    against the CPU, bridge untouched. Also bmm on the GEMM kernels (csrc/linalg.cpp:81-92)."""
    from omarchy_mac_torch_b200.native import core
    torch.manual_seed(0)
    omt.FALLBACKS.clear()
    core.bridge_counts(True)
    for rows, cols, kw in ((256, 1000, {}), (32, 10, dict(reduction="sum", ignore_index=3)), (7, 5, dict(reduction="none")),
                           (64, 100, dict(weight=torch.rand(100) + 0.5))):
        x = torch.randn(rows, cols) * 2
        t = torch.randint(0, cols, (rows,))
        t[1] = 3
        xc = x.clone().requires_grad_()
        ref = F.cross_entropy(xc, t, **kw)
        ref.sum().backward()
        kwd = {k: (v.to(D) if torch.is_tensor(v) else v) for k, v in kw.items()}
        for compiled in (False, True):
            xd = x.to(D).requires_grad_()
            fn = (lambda a, b: F.cross_entropy(a, b, **kwd))
            if compiled:
                fn = torch.compile(fn, backend="omarchy_mac_torch")
            core.kernel_counts(True)
            out = fn(xd, t.to(D))
            out.sum().backward()
            kc = core.kernel_counts(True)
            assert e(out, ref.detach()) <= 1e-5 and e(xd.grad, xc.grad) <= 1e-5, (rows, cols, kw, compiled)
            if compiled:
                assert kc.get("softmax_nll_fwd") == 1 and kc.get("softmax_nll_bwd") == 1 and "nll_fwd" not in kc and "log_softmax" not in kc, kc
            else:
                assert kc.get("log_softmax") == 1 and kc.get("nll_fwd") == 1 and kc.get("nll_bwd") == 1 and kc.get("log_softmax_bwd") == 1, kc
    bc = core.bridge_counts(True)
    assert not any("softmax" in k or "nll" in k for k in bc), bc
    assert not any("softmax" in k or "nll" in k for k in omt.FALLBACKS), dict(omt.FALLBACKS)
    a, b = torch.randn(3, 130, 70), torch.randn(3, 70, 160)
    core.kernel_counts(True)
    got = torch.bmm(a.to(D), b.to(D))
    kc = core.kernel_counts(True)
    assert e(got, torch.bmm(a.double(), b.double()).float()) <= TOL
    assert sum(kc.values()) >= 3, kc   # one GEMM per matrix of the batch
    assert not any("bmm" in k for k in core.bridge_counts(True))
    omt.FALLBACKS.clear()


def test_side_stream_producer_and_default_stream_consumer(omt):
    """Events and record_stream act on the stream they are given, not on the calling thread's current stream: a tensor
    produced on a side stream, handed over by an event recorded and waited for from the default stream's thread state.
    (The device's streams are PyTorch's CUDA streams under the same ids.)"""
    cside, cmain = torch.cuda.Stream(), torch.cuda.current_stream()
    private_use_1 = 20  # c10::DeviceType::PrivateUse1
    handle = lambda cs: torch.Stream(stream_id=cs.stream_id, device_index=0, device_type=private_use_1)
    side, main = handle(cside), handle(cmain)
    base = torch.randn(1 << 22).to(D)
    omt.synchronize()
    with torch.cuda.stream(cside):
        t = base
        for _ in range(20):   # enough queued work that the consumer would run ahead without the event
            t = t * 1.0001 + 1.0
    ev = torch.Event(D)
    ev.record(side)           # current stream here: the default one
    t.record_stream(main)
    ev.wait(main)
    got = (t * 2).cpu()
    want = base.cpu()
    for _ in range(20):
        want = want * 1.0001 + 1.0
    assert torch.allclose(got, want * 2, rtol=1e-5, atol=1e-5)
    side.synchronize()
    assert side.query()


def test_kernel_times_reports_device_time_per_kernel(omt):
    """debug_time_kernels / kernel_times (csrc/module.cpp:30-33 of the reference): per-kernel device time from CUDA events."""
    from omarchy_mac_torch_b200.native import core
    conv = nn.Conv2d(16, 32, 3, padding=1).to(D)
    x = torch.randn(8, 16, 32, 32).to(D).contiguous(memory_format=torch.channels_last)
    conv(x)
    core.kernel_times(True)
    core.debug_time_kernels(True)
    try:
        for _ in range(3):
            conv(x)
        omt.synchronize()
        times = core.kernel_times(True)
    finally:
        core.debug_time_kernels(False)
    conv_ms = sum(v for k, v in times.items() if k.startswith(("conv_tc_1", "conv_tc_2")))
    assert conv_ms > 0 and all(0 <= v < 50 for v in times.values()), times
    assert "conv_tc_weight_split" in times
    assert core.kernel_times(True) == {}


def test_fused_pointwise_programs_on_the_device(omt):
    """omt::fused_pointwise: the interpreter kernel against the composite definition on the CPU, for every op of the table,
    with broadcast and scalar operands, channels-last inputs (the output keeps that layout) and a maximal-length chain."""
    fp = torch.ops.omt.fused_pointwise
    h = lambda *v: ",".join("nan" if x != x else ("inf" if x == float("inf") else ("-inf" if x == float("-inf") else float(x).hex())) for x in v)
    torch.manual_seed(0)
    a, b = torch.randn(3, 8, 5, 7), torch.randn(3, 8, 5, 7)
    pos = a.abs() + 0.1
    one = lambda op, second="v1", third="v0": f"pw1|2|{op},v0,{second},{third};mul,t0,#0,t0|{h(1.0, 0.5, 0.0, 2.0)}"
    cases = [(one(op), (a, b)) for op in ("mul", "div", "max", "min", "sigmoid_bwd", "tanh_bwd", "silu_bwd", "gelu_bwd", "gelu_tanh_bwd",
                                           "hardswish_bwd", "hardsigmoid_bwd")]
    cases += [(one(op, "v0"), (a, b)) for op in ("neg", "relu", "exp", "abs", "tanh", "sigmoid", "silu", "gelu", "gelu_tanh", "hardswish", "hardsigmoid")]
    cases += [(one(op, "v0"), (pos, b)) for op in ("log", "sqrt", "rsqrt", "recip")]
    cases += [(one("add", "v1", "#1"), (a, b)), (one("sub", "v1", "#3"), (a, b)), (one("rsub", "#3", "#1"), (a, b)), (one("pow", "#3"), (a, b)),
              (one("pow", "#1"), (pos, b)), (one("threshold_bwd", "v1", "#2"), (a, b)), (one("clamp", "#1", "#3"), (a, b))]
    # broadcasting: a per-channel [1,8,1,1] operand and a [7] operand; a scalar-only second operand
    cases.append((f"pw1|3|mul,v0,v1,v0;add,t0,v2,#0;hardswish,t1,t1,t1|{h(1.0)}", (a, torch.randn(1, 8, 1, 1), torch.randn(7))))
    # a 24-instruction chain
    chain = ";".join(["add,v0,v1,#0"] + [f"{'tanh' if j % 2 else 'add'},t{j - 1},v1,#0" for j in range(1, 24)])
    cases.append((f"pw1|2|{chain}|{h(0.25)}", (a, b)))
    for prog, ins in cases:
        want = fp(prog, list(ins))
        got = fp(prog, [t.to(D) for t in ins])
        assert got.device.type == D and got.shape == want.shape
        assert e(got, want) <= 1e-5, prog
    # channels-last inputs: the output keeps the layout, and the kernel walks memory linearly
    acl, bcl = (t.to(D).contiguous(memory_format=torch.channels_last) for t in (a, b))
    got = fp(cases[0][0], [acl, bcl])
    assert got.is_contiguous(memory_format=torch.channels_last) and e(got, fp(cases[0][0], [a, b])) <= 1e-5
    mixed = fp(cases[0][0], [acl, b.to(D)])   # one NHWC, one NCHW operand: general indexing
    assert e(mixed, fp(cases[0][0], [a, b])) <= 1e-5
    # NaN handling follows aten: maximum / minimum propagate, clamp keeps NaN
    n1 = torch.tensor([float("nan"), 1.0, -2.0, float("nan")])
    n2 = torch.tensor([0.0, float("nan"), 3.0, float("nan")])
    for op in ("max", "min"):
        prog = f"pw1|2|{op},v0,v1,v0;add,t0,#0,#1|{h(0.0, 1.0)}"
        got, want = fp(prog, [n1.to(D), n2.to(D)]).cpu(), fp(prog, [n1, n2])
        assert torch.equal(torch.isnan(got), torch.isnan(want)) and torch.equal(got[~torch.isnan(got)], want[~torch.isnan(want)])
    with pytest.raises(RuntimeError, match="pointwise"):
        fp("pw1|1|frobnicate,v0,v0,v0|", [a.to(D)])
    assert not omt.FALLBACKS, dict(omt.FALLBACKS)


def test_compile_backend_fuses_pointwise_chains_on_the_device(omt):
    """Pass 4 end to end: a squeeze-excite style block (global pool, two 1x1 convs, hard-sigmoid gate, scale, residual add,
    hard-swish) compiled for the device; outputs and gradients against the eager CPU model."""
    from omarchy_mac_torch_b200.native import core

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.fc1, self.fc2 = nn.Conv2d(16, 8, 1), nn.Conv2d(8, 16, 1)

        def forward(self, x):
            g = F.hardsigmoid(self.fc2(F.relu(self.fc1(F.adaptive_avg_pool2d(x, 1)))))
            return F.hardswish(x * g + x) * 0.5 + torch.tanh(x)

    torch.manual_seed(0)
    ref = Block()
    mod = copy.deepcopy(ref).to(D)
    x = torch.randn(4, 16, 12, 12)
    x1, x2 = x.clone().requires_grad_(), x.to(D).requires_grad_()
    omt.FALLBACKS.clear()
    core.kernel_counts(True)
    ref(x1).square().sum().backward()
    out = torch.compile(mod, backend="omarchy_mac_torch")(x2)
    out.square().sum().backward()
    kc = core.kernel_counts(True)
    assert kc.get("pointwise_program", 0) >= 2, kc
    assert e(out, ref(x)) <= TOL and e(x2.grad, x1.grad) <= TOL
    for a_, b_ in zip(ref.parameters(), mod.parameters()):
        assert e(b_.grad, a_.grad) <= TOL
    assert not omt.FALLBACKS, dict(omt.FALLBACKS)


def test_step_graph_replays_match_eager_steps(omt):
    """graphs.capture: the whole training step (zero_grad, fused-stack forward/backward, fused SGD) recorded once and
    replayed; every replay has to do exactly what an eager step does, also after the static batch tensors are refilled."""
    from omarchy_mac_torch_b200 import graphs, models
    torch.manual_seed(0)
    ref = models.ResNet18(num_classes=10)
    a, b = copy.deepcopy(ref).to(D), copy.deepcopy(ref).to(D)
    oa = torch.optim.SGD(a.parameters(), lr=0.01, momentum=0.9, weight_decay=1e-4)
    ob = torch.optim.SGD(b.parameters(), lr=0.01, momentum=0.9, weight_decay=1e-4)
    x, y = torch.randn(8, 3, 32, 32).to(D), torch.randint(0, 10, (8,)).to(D)

    def step(m, o):
        o.zero_grad(set_to_none=True)
        loss = F.cross_entropy(m(x), y)
        loss.backward()
        o.step()
        return loss

    g = graphs.capture(lambda: step(b, ob), warmup=3)  # three real steps; the recorded run itself executes nothing
    assert g.kernels > 50
    for _ in range(3):
        step(a, oa)
    for it in range(3):
        if it == 2:  # a new batch through the static tensors
            x.copy_(torch.randn(8, 3, 32, 32))
            y.copy_(torch.randint(0, 10, (8,)))
        lb = g().item()
        la = step(a, oa).item()
        assert abs(la - lb) <= 1e-6 * abs(la)
        for p, q in zip(a.parameters(), b.parameters()):
            assert e(q, p.detach().cpu()) <= 1e-6
    for p, q in zip(a.buffers(), b.buffers()):
        assert e(q.float(), p.float().cpu()) <= 1e-6
    assert not omt.FALLBACKS, dict(omt.FALLBACKS)


def test_compile_backend_residual_blocks(omt):
    """torch.compile(backend="omarchy_mac_torch") on a residual network: the BatchNorm -> + identity -> ReLU tails and their
    backward run as the fused device ops, and one training step's gradients match the CPU's eager run."""
    from omarchy_mac_torch_b200 import models
    from omarchy_mac_torch_b200.native import core
    torch.manual_seed(0)
    ref = models.ResNet18(num_classes=10)
    mod = copy.deepcopy(ref).to(D)
    cmod = torch.compile(mod, backend="omarchy_mac_torch")
    x, y = torch.randn(8, 3, 64, 64), torch.randint(0, 10, (8,))
    omt.FALLBACKS.clear()
    core.kernel_counts(True)
    core.bridge_counts(True)
    l1 = F.cross_entropy(ref(x), y); l1.backward()
    l2 = F.cross_entropy(cmod(x.to(D)), y.to(D)); l2.backward()
    kc, bc = core.kernel_counts(True), core.bridge_counts(True)
    assert kc.get("bn_apply_add", 0) == 8 and kc.get("bn_bwd_apply_add", 0) == 8
    assert not any(k.startswith(("relu", "threshold_backward")) for k in bc), bc  # no separate ReLU kernels left
    assert abs(l1.item() - l2.item()) <= 1e-4 * abs(l1.item())
    # Gradients against the same model run eagerly on the device (whose ops the other tests hold against the CPU): a
    # whole-network comparison with the CPU is at the mercy of single ReLU inputs that sit within rounding of zero (one
    # flipped mask among a layer's 32 values per channel moves that layer's BatchNorm gradients by 10 %).
    eager = copy.deepcopy(ref).to(D)
    eager.zero_grad()
    F.cross_entropy(eager(x.to(D)), y.to(D)).backward()
    for a, b in zip(eager.parameters(), mod.parameters()):
        assert e(b.grad, a.grad) <= 1e-4
    for a, b in zip(ref.buffers(), mod.buffers()):
        assert e(b.float(), a.float()) <= 1e-4
    assert not omt.FALLBACKS, dict(omt.FALLBACKS)


def test_resnet50_compile_path_matches_cpu(omt, capsys):
    """The benchmarked code path at a size the CPU finishes in seconds: ResNet-50 (Bottleneck [3,4,6,3]) called through
    torch.compile(backend="omarchy_mac_torch"), SGD momentum 0.9 nesterov weight decay 1e-4, batch 8 at 112x112,
    1 warm-up + 5 steps, against the same run on the CPU (tools/acceptance.py:51-98).

    Run A, the benchmark's exact configuration (default initialisation, lr 0.1). At this batch size that run is chaotic from
    the third step on: the CPU on 1 thread and on 8 threads differ by 4e-2 at step 2 and by 50 % at step 3, and CPU fp32
    differs from CPU float64 by 10 % at step 2. What can be held to a bound is held: step 0's loss to 1e-5; every parameter's
    gradients at step 0 and the parameters after the first optimizer step (nesterov momentum + weight decay through the
    fused kernel) against a CPU float64 run, measured the way the CPU's own fp32 run can be measured: over all tensors
    together (relative L2 distance: at most max(1e-3, 4 x the CPU's), and per tensor (max norm: at most max(1e-3, 4 x the
    CPU's error on that tensor, 2 x the CPU's worst tensor): single ReLU inputs within rounding of zero flip their mask in
    one fp32 run and not in another, which moves a 4x4-pixel layer's gradients by 10-20 %, on the CPU as well); the losses
    of steps 0-2 within max(1e-3, 10 x the CPU fp32 run's distance from float64). All six losses and distances are printed.

    Run B, the same network, optimizer and code path made well conditioned (the last BatchNorm scale of every block starts at
    zero, the usual ResNet-50 recipe, and lr 0.02; CPU fp32 then tracks float64 to 3e-7): all six losses within the plain
    1e-3 of the CPU's, and the final parameters within 5e-3 (all tensors together, L2)."""
    from omarchy_mac_torch_b200 import models
    from omarchy_mac_torch_b200.native import core
    x, y = torch.randn(8, 3, 112, 112), torch.randint(0, 1000, (8,))

    def run(call, model, xx, yy, lr):
        opt = torch.optim.SGD(model.parameters(), lr=lr, momentum=0.9, nesterov=True, weight_decay=1e-4)
        losses, grads, after = [], None, None
        for it in range(6):
            loss = F.cross_entropy(call(xx), yy)
            opt.zero_grad()
            loss.backward()
            if it == 0:
                grads = [p.grad.detach().double().cpu().clone() for p in model.parameters()]
            opt.step()
            if it == 0:
                after = [p.detach().double().cpu().clone() for p in model.parameters()]
            losses.append(loss.item())
        return losses, grads, after

    def err(a, b):
        return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))

    rel = lambda a, b: [abs(p - q) / max(abs(p), 1e-6) for p, q in zip(a, b)]

    # ---- run A: the benchmark's configuration
    torch.manual_seed(0)
    ref = models.ResNet50()
    ref64, mod = copy.deepcopy(ref).double(), copy.deepcopy(ref).to(D)
    cmod = torch.compile(mod, backend="omarchy_mac_torch")
    omt.FALLBACKS.clear()
    core.kernel_counts(True)
    l_cpu, g_cpu, p_cpu = run(ref, ref, x, y, 0.1)
    l_64, g_64, p_64 = run(ref64, ref64, x.double(), y, 0.1)
    l_dev, g_dev, p_dev = run(cmod, mod, x.to(D), y.to(D), 0.1)
    kc = core.kernel_counts(True)
    assert not omt.FALLBACKS, dict(omt.FALLBACKS)
    assert kc.get("bn_apply_add", 0) >= 16 * 6 and kc.get("sgd_multi", 0) == 6, kc  # the fused residual tails and one optimizer launch per step
    assert kc.get("bn_stats_from_partials", 0) >= 6, kc  # at this small batch only the stem is long and wide enough for statistics in the conv epilogue
    assert sum(v for k, v in kc.items() if k.startswith(("conv_tc_1", "conv_tc_2", "wgrad_tc_1", "wgrad_tc_2"))) >= 150 * 6, kc  # the convs ran on the tensor cores
    assert abs(l_dev[0] - l_cpu[0]) <= 1e-5 * abs(l_cpu[0])
    names = [n for n, _ in ref.named_parameters()]

    def l2_all(a, b):
        return (sum(float(((u - v) ** 2).sum()) for u, v in zip(a, b)) / sum(float((v ** 2).sum()) for v in b)) ** 0.5

    assert l2_all(g_dev, g_64) <= max(1e-3, 4 * l2_all(g_cpu, g_64)), (l2_all(g_dev, g_64), l2_all(g_cpu, g_64))
    assert l2_all(p_dev, p_64) <= max(1e-3, 4 * l2_all(p_cpu, p_64)), (l2_all(p_dev, p_64), l2_all(p_cpu, p_64))
    cpu_g = max(err(gc, g6) for gc, g6 in zip(g_cpu, g_64))
    cpu_p = max(err(pc, p6) for pc, p6 in zip(p_cpu, p_64))
    worst_g = worst_p = 0.0
    for n, gd, gc, g6, pd, pc, p6 in zip(names, g_dev, g_cpu, g_64, p_dev, p_cpu, p_64):
        eg, ep = err(gd, g6), err(pd, p6)
        assert eg <= max(1e-3, 4 * err(gc, g6), 2 * cpu_g), ("gradient", n, eg, err(gc, g6), cpu_g)
        assert ep <= max(1e-3, 4 * err(pc, p6), 2 * cpu_p), ("parameter after one step", n, ep, err(pc, p6), cpu_p)
        worst_g, worst_p = max(worst_g, eg), max(worst_p, ep)
    d_cpu, d_64, noise = rel(l_cpu, l_dev), rel(l_64, l_dev), rel(l_64, l_cpu)
    with capsys.disabled():
        print(f"\nresnet50 compile path, lr 0.1: gradients vs float64, all tensors (L2) {l2_all(g_dev, g_64):.2e} (the CPU's own: {l2_all(g_cpu, g_64):.2e}), "
              f"worst tensor (max norm) {worst_g:.2e} (the CPU's own: {cpu_g:.2e}), worst parameter error {worst_p:.2e}")
        print("  device vs CPU fp32 :", [f"{v:.1e}" for v in d_cpu])
        print("  device vs CPU fp64 :", [f"{v:.1e}" for v in d_64])
        print("  CPU fp32 vs fp64   :", [f"{v:.1e}" for v in noise])
    _assert_losses_track(l_dev[:3], l_cpu[:3], l_64[:3], "resnet50 through the compile backend")

    # ---- run B: well conditioned
    torch._dynamo.reset()
    torch.manual_seed(0)
    ref = models.ResNet50()
    for m in ref.modules():
        if isinstance(m, models._Bottleneck):
            nn.init.zeros_(m.b3.weight)
    mod = copy.deepcopy(ref).to(D)
    cmod = torch.compile(mod, backend="omarchy_mac_torch")
    l_cpu, _, _ = run(ref, ref, x, y, 0.02)
    l_dev, _, _ = run(cmod, mod, x.to(D), y.to(D), 0.02)
    assert not omt.FALLBACKS, dict(omt.FALLBACKS)
    with capsys.disabled():
        print("  well-conditioned run, device vs CPU fp32:", [f"{v:.1e}" for v in rel(l_cpu, l_dev)], "losses", [f"{v:.4f}" for v in l_dev])
    assert max(rel(l_cpu, l_dev)) <= 1e-3, (l_cpu, l_dev)
    # the parameters after the six steps: all together to 5e-3 (L2). (Single small tensors, BatchNorm biases of 1e-7 in size, carry
    # the rounding noise of gradients that are zero in exact arithmetic at the first step, amplified by five more steps.)
    p_ref = [p.detach().double() for p in ref.parameters()]
    p_got = [p.detach().double().cpu() for p in mod.parameters()]
    assert l2_all(p_got, p_ref) <= 5e-3, l2_all(p_got, p_ref)


def test_compile_backend(omt):
    """notes/scripts/compile_check.py: torch.compile(backend="omarchy_mac_torch") gradients and eval output vs CPU."""
    from omarchy_mac_torch_b200 import models
    from omarchy_mac_torch_b200.native import core
    torch.manual_seed(0)
    ref = models.PlainCNN3(bias=False)
    mod = copy.deepcopy(ref).to(D)
    cmod = torch.compile(mod, backend="omarchy_mac_torch")
    x, y = torch.randn(16, 3, 32, 32), torch.randint(0, 10, (16,))
    core.kernel_counts(True)
    F.cross_entropy(ref(x), y).backward()
    F.cross_entropy(cmod(x.to(D)), y.to(D)).backward()
    assert max(e(b.grad, a.grad) for a, b in zip(ref.parameters(), mod.parameters())) <= 1e-3
    ref.eval(); mod.eval()
    with torch.no_grad():
        assert e(torch.compile(mod, backend="omarchy_mac_torch")(x.to(D)), ref(x)) <= 1e-3


def test_tuning_pass_through_the_device_ops(omt):
    """set_tuning(True): the first dense convolution of a (pass, geometry) runs the library's timing pass; results are those of
    the CPU, later calls reuse the choice, and tune_dump / tune_load carry the choices in the reference's key format."""
    from omarchy_mac_torch_b200.native import core
    torch.manual_seed(3)
    conv = torch.nn.Conv2d(64, 192, 3, padding=1, bias=False)
    x = torch.randn(16, 64, 28, 28, requires_grad=True)
    y = conv(x)
    y.square().sum().backward()
    want = (y.detach(), x.grad.clone(), conv.weight.grad.clone())
    before = dict(core.tune_dump())
    core.set_tuning(True, 4)
    try:
        dconv = copy.deepcopy(conv).to(omt.DEVICE)
        dconv.weight.grad = None
        for _ in range(2):  # the second pass finds every geometry tuned
            xd = x.detach().to(omt.DEVICE).requires_grad_(True)
            yd = dconv(xd)
            yd.square().sum().backward()
        assert e(yd, want[0]) <= TOL and e(xd.grad, want[1]) <= TOL
        assert e(dconv.weight.grad / 2, want[2]) <= TOL
        dump = core.tune_dump()
        for k, (tile, mult) in dump.items():
            f = [int(v) for v in k.split(",")]
            assert len(f) == 11 and f[0] in (0, 1, 2) and tile in (0, 64, 128, 192, 256) and mult > 0
        assert core.tune_load(dict(dump)) == len(dump)
        assert set(core.tuned_plans()) == set(dump)
    finally:
        core.set_tuning(False, 4)
        for k in set(core.tune_dump()) - set(before):
            core.tune_load({k: (0, 1.0)})

