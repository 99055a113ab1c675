"""Host-side logic that needs no GPU: stack eligibility rules and layer specs (omarchy_mac_torch/stacks.py:41-94), the
fused-optimizer constructor rule (optim.py:15-31), the FX rewrite passes (compile.py:69-161) exercised on CPU graphs
through the ops' composite definitions, and the workload model definitions against the golden loss curves."""
import copy

import pytest
import torch
import torch.nn.functional as F
from torch import nn


@pytest.fixture(scope="module")
def pkg():
    import omarchy_mac_torch_b200 as m
    m.DEVICE  # loads the extension and registers the device (no CUDA call happens until a tensor is allocated)
    return m


def test_device_is_registered_and_fails_loudly_without_a_gpu(pkg):
    assert pkg.DEVICE == "omarchy_mac_torch" and hasattr(torch, "omarchy_mac_torch") and torch.omarchy_mac_torch.device_count() == 1
    import omarchy_mac_torch  # the reference's import name resolves to this package
    assert omarchy_mac_torch is pkg
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="no CUDA device"):
            torch.empty(2, device=pkg.DEVICE)
    assert pkg.validate_kernels() == [] and pkg.tune_cpu() is None and len(pkg.FALLBACKS) == 0


def test_fusable_rules(pkg):
    from omarchy_mac_torch_b200 import models, stacks
    cbr = lambda ci, co, **kw: [nn.Conv2d(ci, co, 3, padding=1, bias=False, **kw), nn.BatchNorm2d(co), nn.ReLU()]
    assert stacks.fusable(nn.Sequential(*cbr(3, 8), nn.MaxPool2d(2)))
    assert stacks.fusable(nn.Sequential(*cbr(3, 8), *cbr(8, 8, groups=8), nn.AvgPool2d(2), nn.AdaptiveAvgPool2d(1)))
    assert stacks.fusable(nn.Sequential(nn.Conv2d(3, 8, 3, padding=1, bias=True), nn.BatchNorm2d(8), nn.ReLU()))  # bias accepted here
    assert not stacks.fusable(nn.Sequential())
    assert not stacks.fusable(nn.Sequential(nn.BatchNorm2d(3), nn.ReLU()))                                # must start with a conv
    assert not stacks.fusable(nn.Sequential(nn.Conv2d(3, 8, 3, padding=1), nn.BatchNorm2d(8)))             # BN without ReLU
    assert not stacks.fusable(nn.Sequential(nn.Conv2d(3, 8, 3, padding=1), nn.BatchNorm2d(8, eps=1e-3), nn.ReLU()))
    assert not stacks.fusable(nn.Sequential(nn.Conv2d(3, 8, 3, stride=2, padding=1)))                      # strided
    assert not stacks.fusable(nn.Sequential(nn.Conv2d(3, 8, 7, padding=3)))                                # dense 7x7 not in a plan
    assert not stacks.fusable(nn.Sequential(nn.Conv2d(3, 8, 3, padding=1), nn.MaxPool2d(3, 2)))
    assert not stacks.fusable(nn.Sequential(nn.Conv2d(3, 8, 3, padding=1), nn.AdaptiveAvgPool2d(2)))
    assert not stacks.fusable(nn.Sequential(nn.Conv2d(4, 8, 3, padding=1, groups=2)))                      # grouped, not depthwise
    assert not stacks.fusable(nn.Sequential(nn.Conv2d(3, 8, 3, padding=1), nn.Hardswish()))
    m = models.PlainCNN3()
    assert stacks.layer_specs(m.features)[:3] == [("convb", 3, 32, 3, 0.0), ("bn", 32, 32, 0, 0.1), ("pool", 0, 0, 0, 0.0)]
    assert [tuple(p.shape) for p in stacks._params(m.features)][:4] == [(32, 3, 3, 3), (32,), (32,), (32,)]
    sep = models.SeparableCNN()
    kinds = [s[0] for s in stacks.layer_specs(sep.features)]
    assert kinds.count("dw") == 4 and kinds[-1] == "gap" and kinds.count("pool") == 2
    assert not stacks.fusable(models.ResNet18().stem)  # 7x7 stride-2 stem stays eager


def test_optimizer_constructor_rule(pkg):
    from omarchy_mac_torch_b200 import optim

    class P:  # stands in for a parameter on the device
        def __init__(self, dev):
            self.device = torch.device(dev)
    on, off = [P("omarchy_mac_torch:0")], [P("cpu")]
    assert optim.wants_fused(on, {})
    assert optim.wants_fused([{"params": on}], {"lr": 0.1})
    assert not optim.wants_fused(off, {}) and not optim.wants_fused(on + off, {}) and not optim.wants_fused([], {})
    assert not optim.wants_fused(on, {"fused": False}) and not optim.wants_fused(on, {"foreach": True})
    assert not optim.wants_fused(on, {"differentiable": True}) and not optim.wants_fused(on, {"lr": torch.tensor(0.1)})
    assert torch.optim.SGD([nn.Parameter(torch.zeros(2))], lr=0.1).defaults.get("fused") in (None, False)  # CPU params untouched


def test_fx_passes_rewrite_and_preserve_results(pkg, monkeypatch):
    """Passes 1-3 on CPU graphs (the omt:: ops' composite definitions run anywhere), compared with the unrewritten graph."""
    from torch._dynamo.backends.common import aot_autograd
    from functorch.compile import make_boxed_func
    from omarchy_mac_torch_b200 import compile as C, models
    monkeypatch.setattr(C, "_ANY_DEVICE", True)
    seen = []

    def compiler(gm, _inputs):
        seen.append(C.rewrite(gm))
        return make_boxed_func(gm.forward)

    backend = aot_autograd(fw_compiler=compiler, bw_compiler=compiler, inference_compiler=compiler)
    torch.manual_seed(0)
    ref = models.PlainCNN3(bias=False)
    mod = copy.deepcopy(ref)
    x, y = torch.randn(8, 3, 32, 32), torch.randint(0, 10, (8,))
    F.cross_entropy(ref(x), y).backward()
    F.cross_entropy(torch.compile(mod, backend=backend)(x), y).backward()
    assert sum(s["bn_relu"] for s in seen) == 3 and sum(s["bn_relu_backward"] for s in seen) == 3
    assert sum(s["conv_bn_train"] for s in seen) == 3  # each conv + BatchNorm + ReLU became one op
    for a, b in zip(ref.parameters(), mod.parameters()):
        assert torch.allclose(a.grad, b.grad, rtol=1e-4, atol=1e-6)
    for a, b in zip(ref.buffers(), mod.buffers()):
        assert torch.allclose(a.float(), b.float(), rtol=1e-5, atol=1e-6)
    seen.clear()
    ref.eval(); mod.eval()
    torch._dynamo.reset()
    with torch.no_grad():
        out = torch.compile(mod, backend=backend)(x)
        assert torch.allclose(out, ref(x), rtol=1e-4, atol=1e-5)
    assert sum(s["conv_epilogue"] for s in seen) == 3  # conv -> eval BN -> ReLU folded three times
    # residual blocks: BatchNorm -> + identity -> ReLU (with and without a downsample branch) and its backward
    seen.clear()
    torch._dynamo.reset()
    torch.manual_seed(1)
    ref = models.ResNet18(num_classes=10)
    mod = copy.deepcopy(ref)
    x, y = torch.randn(4, 3, 32, 32), torch.randint(0, 10, (4,))
    F.cross_entropy(ref(x), y).backward()
    F.cross_entropy(torch.compile(mod, backend=backend)(x), y).backward()
    assert sum(s["bn_add_relu"] for s in seen) == 8 and sum(s["bn_add_relu_backward"] for s in seen) == 8
    assert sum(s["bn_relu"] for s in seen) == 9 and sum(s["bn_relu_backward"] for s in seen) == 9
    assert sum(s["dgrad_accumulate"] for s in seen) == 8  # the backward joins of the 8 residual blocks
    assert sum(s["conv_bn_train"] for s in seen) == 20    # every conv feeds a BatchNorm: 9 + ReLU, 8 + identity + ReLU, 3 downsample (plain)
    for a, b in zip(ref.parameters(), mod.parameters()):
        assert (a.grad - b.grad).abs().max() <= 1e-4 * a.grad.abs().max() + 1e-7
    for a, b in zip(ref.buffers(), mod.buffers()):
        assert torch.allclose(a.float(), b.float(), rtol=1e-5, atol=1e-6)


def test_model_definitions_reproduce_reference_curves(pkg, golden_losses):
    """This package's PlainCNN / SeparableCNN register parameters in the reference's order: same seed, same CPU loss curve."""
    from omarchy_mac_torch_b200 import models
    for name, cls in (("plaincnn", models.PlainCNN), ("separablecnn", models.SeparableCNN)):
        g = golden_losses[name]
        torch.manual_seed(0)
        m = cls()
        x, y = torch.randn(*g["shape"]), torch.randint(0, g["classes"], (g["shape"][0],))
        opt = torch.optim.SGD(m.parameters(), lr=0.01, momentum=0.9)
        out = []
        for _ in range(3):
            loss = F.cross_entropy(m(x), y); opt.zero_grad(); loss.backward(); opt.step(); out.append(loss.item())
        assert max(abs(a - b) / abs(b) for a, b in zip(out, g["losses"][:3])) < 1e-5
    assert sum(p.numel() for p in models.ResNet50().parameters()) == 25557032


def test_compile_regions_matches_eager_and_delivers_gradients_region_by_region(pkg):
    """compile.compile_regions: the stem and every block become separate compiled graphs; results equal the eager model's,
    and parameter gradients arrive region by region during backward (last block first), which is what lets a data-parallel
    wrapper start reducing the last layers' buckets while the earlier layers' backward still runs."""
    from omarchy_mac_torch_b200 import compile as C, models
    torch.manual_seed(0)
    ref = models.ResNet50(num_classes=10, layers=(1, 1, 1, 1))
    mod = copy.deepcopy(ref)
    assert [n for _, n in mod.compile_regions()] == ["stem", (0, 2), (2, 3), (3, 4)]
    assert [n for _, n in models.ResNet50().compile_regions()] == ["stem", (0, 6), (6, 11), (11, 16)]
    C.compile_regions(mod)
    order = []
    for name, p in mod.named_parameters():
        p.register_post_accumulate_grad_hook(lambda _p, name=name: order.append(name))
    x, y = torch.randn(2, 3, 32, 32), torch.randint(0, 10, (2,))
    F.cross_entropy(ref(x), y).backward()
    F.cross_entropy(mod(x), y).backward()
    for (n, a), b in zip(ref.named_parameters(), mod.parameters()):
        assert torch.allclose(a.grad, b.grad, rtol=1e-4, atol=1e-6), n
    region = lambda n: {"0": "a", "1": "a", "2": "b", "3": "c"}[n.split(".")[1]] if n.startswith("layers.") else n.split(".")[0]
    seen = []
    for n in order:
        if not seen or seen[-1] != region(n):
            seen.append(region(n))
    assert seen == ["head", "c", "b", "a", "stem"], seen  # each region's gradients arrive together, in backward order
    assert [n for n, _ in mod.named_parameters()] == [n for n, _ in ref.named_parameters()]


def test_pointwise_chains_become_one_op_and_keep_their_results(pkg, monkeypatch):
    """Pass 4 on CPU graphs: chains of elementwise ops (forward and the backward forms autograd derives from them) collapse
    into omt.fused_pointwise programs; outputs and gradients equal the unfused model's."""
    from torch._dynamo.backends.common import aot_autograd
    from functorch.compile import make_boxed_func
    from omarchy_mac_torch_b200 import compile as C
    monkeypatch.setattr(C, "_ANY_DEVICE", True)
    seen, programs = [], []

    def compiler(gm, _inputs):
        seen.append(C.rewrite(gm))
        programs.extend(n.args[0] for n in gm.graph.nodes if n.op == "call_function" and n.target is torch.ops.omt.fused_pointwise.default)
        return make_boxed_func(gm.forward)

    backend = aot_autograd(fw_compiler=compiler, bw_compiler=compiler, inference_compiler=compiler)

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.scale = torch.nn.Parameter(torch.randn(1, 6, 1, 1))

        def forward(self, x, r):
            y = F.hardswish(x * self.scale + 0.5)                  # broadcast of a [1,6,1,1] parameter, a scalar folded in
            y = torch.sigmoid(y) * torch.tanh(r) - 2.0 * r       # two inputs, alpha
            y = F.gelu(y, approximate="tanh").clamp(min=-0.1) ** 2
            return F.silu(y).relu()

    torch.manual_seed(0)
    ref = Net()
    mod = copy.deepcopy(ref)
    x, r = torch.randn(4, 6, 5, 5), torch.randn(4, 6, 5, 5)
    x1, x2 = x.clone().requires_grad_(), x.clone().requires_grad_()
    ref(x1, r).square().sum().backward()
    out = torch.compile(mod, backend=backend)(x2, r)
    out.square().sum().backward()
    assert torch.allclose(out, ref(x, r), rtol=1e-5, atol=1e-6)
    assert torch.allclose(x1.grad, x2.grad, rtol=1e-4, atol=1e-6) and torch.allclose(ref.scale.grad, mod.scale.grad, rtol=1e-4, atol=1e-5)
    assert sum(s["pointwise"] for s in seen) >= 2 and programs, seen   # at least one chain in the forward and one in the backward graph
    assert all(p.startswith("pw1|") and 2 <= len(p.split("|")[2].split(";")) <= 24 for p in programs), programs
    assert any("hardswish" in p for p in programs) and any("_bwd" in p for p in programs), programs


@pytest.mark.parametrize("reduction,weighted", [("mean", False), ("sum", True), ("none", False)])
def test_cross_entropy_becomes_the_fused_pair(pkg, monkeypatch, reduction, weighted):
    """Pass 5 on CPU graphs: log_softmax + nll_loss (what F.cross_entropy lowers to) become omt.softmax_nll in the forward
    graph and omt.softmax_nll_backward in the backward graph; loss and gradient equal the unfused ones (ignore_index too)."""
    from torch._dynamo.backends.common import aot_autograd
    from functorch.compile import make_boxed_func
    from omarchy_mac_torch_b200 import compile as C
    monkeypatch.setattr(C, "_ANY_DEVICE", True)
    seen, targets = [], []

    def compiler(gm, _inputs):
        seen.append(C.rewrite(gm))
        targets.extend(str(n.target) for n in gm.graph.nodes if n.op == "call_function")
        return make_boxed_func(gm.forward)

    backend = aot_autograd(fw_compiler=compiler, bw_compiler=compiler, inference_compiler=compiler)
    torch.manual_seed(0)
    w = torch.rand(7) + 0.5 if weighted else None

    def loss_fn(x, t):
        out = F.cross_entropy(x * 1.5, t, weight=w, reduction=reduction, ignore_index=3)
        return out.sum() if reduction == "none" else out

    x = torch.randn(9, 7)
    t = torch.randint(0, 7, (9,))
    t[2] = 3
    x1, x2 = x.clone().requires_grad_(), x.clone().requires_grad_()
    ref = loss_fn(x1, t)
    ref.backward()
    out = torch.compile(loss_fn, backend=backend)(x2, t)
    out.backward()
    assert torch.allclose(out, ref, rtol=1e-6, atol=1e-7) and torch.allclose(x1.grad, x2.grad, rtol=1e-5, atol=1e-7)
    assert sum(s["softmax_nll"] for s in seen) == 2, seen
    assert "omt.softmax_nll.default" in targets and "omt.softmax_nll_backward.default" in targets
    assert not any("nll_loss" in s or "_log_softmax" in s for s in targets), targets


def test_step_counters_of_all_batch_norm_layers_advance_in_one_op(pkg, monkeypatch):
    """Pass 6 on a CPU graph: the `num_batches_tracked + 1` of every BatchNorm layer become one aten._foreach_add; the counters
    and the outputs equal the unfused model's, also over a second step."""
    from torch._dynamo.backends.common import aot_autograd
    from functorch.compile import make_boxed_func
    from omarchy_mac_torch_b200 import compile as C
    monkeypatch.setattr(C, "_ANY_DEVICE", True)
    seen, targets = [], []

    def compiler(gm, _inputs):
        seen.append(C.rewrite(gm))
        targets.extend(str(n.target) for n in gm.graph.nodes if n.op == "call_function")
        return make_boxed_func(gm.forward)

    backend = aot_autograd(fw_compiler=compiler, bw_compiler=compiler, inference_compiler=compiler)
    torch.manual_seed(0)
    ref = torch.nn.Sequential(torch.nn.Conv2d(3, 8, 3, padding=1, bias=False), torch.nn.BatchNorm2d(8), torch.nn.ReLU(),
                              torch.nn.Conv2d(8, 8, 3, padding=1, bias=False), torch.nn.BatchNorm2d(8), torch.nn.ReLU(),
                              torch.nn.Conv2d(8, 4, 1), torch.nn.BatchNorm2d(4))
    mod = copy.deepcopy(ref)
    fn = torch.compile(mod, backend=backend)
    x = torch.randn(2, 3, 8, 8)
    for _ in range(2):
        assert torch.allclose(fn(x), ref(x), rtol=1e-5, atol=1e-6)
    assert seen[0]["step_counters"] == 3 and "aten._foreach_add.Scalar" in targets
    assert [int(v) for k, v in mod.state_dict().items() if "num_batches" in k] == [2, 2, 2]
    assert all(torch.allclose(a, b, rtol=1e-5, atol=1e-6) for a, b in zip(mod.state_dict().values(), ref.state_dict().values()))


def test_bench_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` needs no GPU: it times the CPU implementation of the workload and prints one JSON line with the
    same metric, unit and config as the GPU arm, `impl`, a `cpu_baseline` describing the run and an `e2e` that repeats it."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--workload", "plaincnn", "--steps", "2", "--warmup", "3"],
                         capture_output=True, text=True, timeout=600, cwd=root)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "train_ms_per_step" and line["unit"] == "ms/step"
    assert line["higher_is_better"] is False and line["n_gpus"] == 1 and line["steps"] == 2 and line["vs_baseline"] is None
    assert line["config"]["workload"] == "plaincnn_b128_train" and line["data"] == "synthetic"
    assert line["value"] > 0 and line["value"] == line["ms_per_step"]
    cb = line["cpu_baseline"]
    assert cb["kind"] == "reference" and cb["cores"] >= 1 and cb["value"] == line["value"] and "PyTorch CPU" in cb["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "ms/step", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_conv_plan_overrides_round_trip_without_a_gpu():
    """The per-geometry plan table behind the tuning pass (set / get / dump / load) is host-side state of the library: stored
    overrides come back, the text form round-trips, entries naming a tile width this build does not have are skipped, and
    clearing leaves the table empty."""
    from omarchy_mac_torch_b200 import capi
    lib = capi.lib()
    g1 = capi.geo(256, 128, 128, 28, 28, 3, 1, 1)
    g2 = capi.geo(256, 64, 256, 56, 56, 1, 1, 0)
    assert capi.conv_plan_get(2, g1) is None
    capi.call("omt_conv_plan_set", 2, g1, 192, 0.5)
    capi.call("omt_conv_plan_set", 0, g2, 128, 1.0)
    assert capi.conv_plan_get(2, g1) == (192, 0.5) and capi.conv_plan_get(0, g2) == (128, 1.0) and capi.conv_plan_get(1, g2) is None
    dump = capi.conv_plans_dump()
    assert dump == {"2,256,128,128,28,28,28,28,3,1,1": (192, 0.5), "0,256,64,256,56,56,56,56,1,1,0": (128, 1.0)}
    with pytest.raises(capi.OmtError):
        capi.call("omt_conv_plan_set", 0, g2, 192, 1.0)   # 192 columns exist for the weight gradient only
    with pytest.raises(capi.OmtError):
        capi.call("omt_conv_plan_set", 1, g2, 256, 2.0)   # the slice factor belongs to the weight gradient
    capi.call("omt_conv_plan_set", 2, g1, 0, 1.0)
    capi.call("omt_conv_plan_set", 0, g2, 0, 0.0)
    assert capi.conv_plans_dump() == {}
    took = capi.conv_plans_load({**dump, "1,8,32,32,9,9,9,9,3,1,1": (96, 1.0), "not a key": (64, 1.0)})
    assert took == 2 and capi.conv_plans_dump() == dump
    assert lib.omt_conv_plans_load(b"") == 0
    for k in dump:  # leave the process as it was found
        f = [int(v) for v in k.split(",")]
        capi.call("omt_conv_plan_set", f[0], capi.geo(f[1], f[2], f[3], f[4], f[5], f[8], f[9], f[10]), 0, 1.0)
    assert capi.conv_plans_dump() == {}
