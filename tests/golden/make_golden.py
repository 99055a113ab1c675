"""Generates the golden fixtures in this directory. Run where a checkout of the reference is available:

    python tests/golden/make_golden.py <path to the omarchy-mac-torch checkout>

The reference ships no stored vectors; its checks compare the device with PyTorch's CPU aten on shape lists written in
its scripts (notes/scripts/conv_kinds_check.py:5, notes/scripts/alexnet_ops_check.py:6,12,16, tools/gemm_bench.py:8-9)
and on loss curves of its own model definitions (tools/acceptance.py:37-98, omarchy_mac_torch/models.py). This script
replays exactly that on the CPU and stores the expected outputs:

  ops.npz     per-op expected outputs (aten CPU) for those shape lists; inputs are regenerated from numpy PCG64 seeds
              (stable across platforms), so only outputs are stored
  losses.json 1 warm-up + 5 step loss curves of the reference's ResNet18 / MobileNetV3Small / PlainCNN / SeparableCNN
              classes, imported from the reference checkout, trained on the CPU as tools/acceptance.py does
"""
import importlib.util
import json
import pathlib
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
from cases import ADAPOOL, BN, MAXPOOL, conv_cases, conv_inputs, rnd  # noqa: E402

def conv_case(seed, n, ci, co, ks, stride, pad, hw, groups, bias):
    x, w, b, gy = conv_inputs(seed, n, ci, co, ks, stride, pad, hw, groups, bias)
    y = F.conv2d(x, w, b, stride=stride, padding=pad, groups=groups)
    dx, dw, db = torch.ops.aten.convolution_backward(gy, x, w, [co] if bias else None, [stride] * 2, [pad] * 2, [1, 1], False, [0, 0],
                                                     groups, [True, True, bias])
    out = {"y": y, "dx": dx, "dw": dw}
    if bias:
        out["db"] = db
    return out


def make_ops():
    out = {}
    for name, args in conv_cases().items():
        for k, v in conv_case(*args).items():
            out[f"{name}_{k}"] = v.numpy()
    for i, (k, s, p, hw) in enumerate(MAXPOOL):
        x = rnd(700 + i, 2, 4, hw, hw).requires_grad_()
        y, idx = F.max_pool2d(x, k, s, p, return_indices=True)
        g = rnd(720 + i, *y.shape)
        y.backward(g)
        out[f"maxpool{i}_y"], out[f"maxpool{i}_idx"], out[f"maxpool{i}_gx"] = y.detach().numpy(), idx.numpy(), x.grad.numpy()
    for i, (hw, o) in enumerate(ADAPOOL):
        x = rnd(800 + i, 2, 5, hw, hw).requires_grad_()
        y = F.adaptive_avg_pool2d(x, o)
        g = rnd(820 + i, *y.shape)
        y.backward(g)
        out[f"adapool{i}_y"], out[f"adapool{i}_gx"] = y.detach().numpy(), x.grad.numpy()
    for i, (n, c, h, w) in enumerate(BN):
        x = (rnd(900 + i, n, c, h, w) * 2 + 3).requires_grad_()
        gamma, beta = rnd(910 + i, c).requires_grad_(), rnd(920 + i, c).requires_grad_()
        rm, rv = rnd(930 + i, c), rnd(940 + i, c).abs() + 0.5
        rm2, rv2 = rm.clone(), rv.clone()
        y, mean, invstd = torch.native_batch_norm(x, gamma, beta, rm2, rv2, True, 0.1, 1e-5)
        g = rnd(950 + i, n, c, h, w)
        y.backward(g)
        ye = torch.native_batch_norm(x, gamma, beta, rm, rv, False, 0.1, 1e-5)[0]
        # BN+ReLU and its masked backward: the composite the omt:: ops are defined by (csrc/fused.cpp:19-28)
        yr = torch.relu(y.detach())
        gz = torch.ops.aten.threshold_backward(g, yr, 0)
        dxr, dgr, dbr = torch.ops.aten.native_batch_norm_backward(gz, x.detach(), gamma.detach(), None, None, mean, invstd, True, 1e-5,
                                                                 [True, True, True])
        for k, v in dict(y=y, mean=mean, invstd=invstd, rm=rm2, rv=rv2, dx=x.grad, dgamma=gamma.grad, dbeta=beta.grad, yeval=ye,
                         relu_dx=dxr, relu_dgamma=dgr, relu_dbeta=dbr).items():
            out[f"bn{i}_{k}"] = v.detach().numpy()
    # optimizers: torch.optim non-fused CPU path, 3 steps, per-step parameters
    for name, mk in [("sgd_nesterov_wd", lambda p: torch.optim.SGD(p, lr=0.1, momentum=0.9, nesterov=True, weight_decay=1e-4)),
                     ("sgd_plain", lambda p: torch.optim.SGD(p, lr=0.05)),
                     ("sgd_damp_max", lambda p: torch.optim.SGD(p, lr=0.05, momentum=0.8, dampening=0.3, maximize=True)),
                     ("adam_wd", lambda p: torch.optim.Adam(p, lr=1e-3, weight_decay=0.01)),
                     ("adamw", lambda p: torch.optim.AdamW(p, lr=1e-3, weight_decay=0.01))]:
        p = torch.nn.Parameter(rnd(1000, 37, 11))
        opt = mk([p])
        for step in range(3):
            p.grad = rnd(1001 + step, 37, 11)
            opt.step()
            out[f"optim_{name}_p{step}"] = p.detach().numpy().copy()
    np.savez_compressed(HERE / "ops.npz", **out)
    print("ops.npz:", len(out), "arrays,", (HERE / "ops.npz").stat().st_size, "bytes")


def train_losses(model, x, y, kind, steps=5):
    # tools/acceptance.py:43-72 (make_opt + train)
    if kind == "sgd":
        opt = torch.optim.SGD(model.parameters(), lr=0.01, momentum=0.9)
    elif kind == "adam":
        opt = torch.optim.Adam(model.parameters(), lr=1e-3)
    else:
        opt = torch.optim.AdamW(model.parameters(), lr=1e-3, weight_decay=0.01)
    losses = []
    for _ in range(steps + 1):
        out = model(x)
        loss = F.cross_entropy(out, y)
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(float(loss))
    return losses


def make_losses(ref_root):
    spec = importlib.util.spec_from_file_location("ref_models", pathlib.Path(ref_root) / "omarchy_mac_torch" / "models.py")
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    cases = {  # tools/acceptance.py:37-45
        "resnet18": (ref.ResNet18, (32, 3, 64, 64), 10, "sgd"),
        "mobilenetv3": (ref.MobileNetV3Small, (32, 3, 96, 96), 10, "adam"),
        "plaincnn": (ref.PlainCNN, (128, 1, 28, 28), 10, "sgd"),
        "separablecnn": (ref.SeparableCNN, (128, 1, 28, 28), 10, "sgd"),
    }
    out = {}
    torch.set_num_threads(8)
    for name, (cls, shape, classes, kind) in cases.items():
        torch.manual_seed(0)
        model = cls()
        for m in model.modules():
            if isinstance(m, torch.nn.Dropout):
                m.p = 0.0
        x, y = torch.randn(*shape), torch.randint(0, classes, (shape[0],))
        out[name] = {"shape": list(shape), "classes": classes, "optimizer": kind, "losses": train_losses(model, x, y, kind),
                     "params": sum(p.numel() for p in model.parameters())}
        print(name, out[name]["losses"])
    rec = pathlib.Path(ref_root) / "results" / "acceptance.json"
    if rec.exists():  # the reference's own recorded CPU curves (torch 2.15, aarch64): indicative cross-check
        for row in json.loads(rec.read_text()):
            if row["model"] in out:
                out[row["model"]]["recorded_reference_cpu"] = row["losses_cpu"]
    out["_meta"] = {"torch": torch.__version__, "note": "torch.manual_seed(0); model(); x=randn; y=randint; CPU aten"}
    (HERE / "losses.json").write_text(json.dumps(out, indent=1))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__.split("\n\n")[1])
    make_ops()
    make_losses(sys.argv[1])
