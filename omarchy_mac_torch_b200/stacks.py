"""Fused conv / BatchNorm+ReLU / pool stacks.

`accelerate(model)` (and, automatically, the first forward of any nn.Sequential on a device tensor) swaps every
nn.Sequential made only of supported layers for a FusedSequential: same modules, parameters and state_dict, but run from
a native plan (one C++ call for the whole forward, one for the backward, gradients delivered as views of one slab).

Same entry points and eligibility rules as the reference's omarchy_mac_torch/stacks.py (fusable, FusedSequential,
accelerate, the global forward pre-hook, OMARCHY_MAC_TORCH_AUTO_FUSE), with one extension: convolutions may carry a
bias (the reference rejects them); the bias is added in the conv epilogue and its gradient lands in the slab too."""

import os
import weakref

import torch
from torch import nn

from omarchy_mac_torch_b200.native import DEVICE, core


def _two(v):
    return tuple(v) if isinstance(v, (tuple, list)) else (v, v)


def _is_max2(m):
    return (type(m) is nn.MaxPool2d and _two(m.kernel_size) == (2, 2) and _two(m.stride) == (2, 2) and _two(m.padding) == (0, 0)
            and _two(m.dilation) == (1, 1) and not m.ceil_mode and not m.return_indices)


def _is_avg2(m):
    return (type(m) is nn.AvgPool2d and _two(m.kernel_size) == (2, 2) and _two(m.stride) == (2, 2) and _two(m.padding) == (0, 0)
            and not m.ceil_mode and m.divisor_override is None)


def _same_square_conv(m, sizes):
    k = m.kernel_size
    return (type(m) is nn.Conv2d and k[0] == k[1] and k[0] in sizes and m.stride == (1, 1) and m.dilation == (1, 1)
            and m.padding == (k[0] // 2, k[0] // 2) and m.padding_mode == "zeros" and m.weight.dtype == torch.float32)


def _is_dense(m):
    return _same_square_conv(m, (1, 3, 5)) and m.groups == 1


def _is_depthwise(m):
    return _same_square_conv(m, (3, 5, 7)) and m.groups == m.in_channels == m.out_channels > 1


def _bn_relu_pair(mods, i):
    m = mods[i]
    return (type(m) is nn.BatchNorm2d and m.affine and m.track_running_stats and m.momentum is not None and m.eps == 1e-5
            and i + 1 < len(mods) and type(mods[i + 1]) is nn.ReLU)


def layer_specs(seq):
    """[(kind, ci, co, ks, momentum)] for a Sequential, or None when some layer has no fused-plan implementation.
    Kinds: conv / convb (with bias), dw / dwb, bn (BatchNorm2d + the ReLU that follows), pool, apool, gap."""
    mods = list(seq)
    if not mods or not isinstance(mods[0], nn.Conv2d):
        return None
    specs, i = [], 0
    while i < len(mods):
        m = mods[i]
        if isinstance(m, nn.Conv2d):
            if _is_dense(m):
                kind = "conv"
            elif _is_depthwise(m):
                kind = "dw"
            else:
                return None
            specs.append((kind + ("b" if m.bias is not None else ""), m.in_channels, m.out_channels, m.kernel_size[0], 0.0))
        elif type(m) is nn.BatchNorm2d:
            if not _bn_relu_pair(mods, i):
                return None
            specs.append(("bn", m.num_features, m.num_features, 0, float(m.momentum)))
            i += 1  # the ReLU belongs to the BN step
        elif type(m) is nn.AdaptiveAvgPool2d:
            if m.output_size not in (1, (1, 1)):
                return None
            specs.append(("gap", 0, 0, 0, 0.0))
        elif _is_max2(m):
            specs.append(("pool", 0, 0, 0, 0.0))
        elif _is_avg2(m):
            specs.append(("apool", 0, 0, 0, 0.0))
        else:
            return None
        i += 1
    return specs


def fusable(seq):
    """Whether every layer of nn.Sequential `seq` has a fused-plan implementation."""
    return layer_specs(seq) is not None


def _layer_specs(seq):
    return layer_specs(seq)


def _params(seq):
    out = []
    for m in seq:
        if isinstance(m, nn.Conv2d):
            out.append(m.weight)
            if m.bias is not None:
                out.append(m.bias)
        elif isinstance(m, nn.BatchNorm2d):
            out += [m.weight, m.bias]
    return out


_plans = weakref.WeakKeyDictionary()  # Sequential -> {(shape, train, input_grad): Plan}


def _plan(seq, shape, train, input_grad):
    cache = _plans.setdefault(seq, {})
    key = (tuple(shape), bool(train), bool(input_grad))
    plan = cache.get(key)
    if plan is None or plan.busy:  # busy: a forward of this plan still awaits its backward (re-entrant use)
        bns = [m for m in seq if isinstance(m, nn.BatchNorm2d)]
        plan = core.make_plan(layer_specs(seq), list(shape), train, input_grad, list(_params(seq)), [m.running_mean for m in bns],
                              [m.running_var for m in bns])
        cache.setdefault(key, plan)
    return plan


class _StackFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, seq, *params):
        plan = _plan(seq, x.shape, True, ctx.needs_input_grad[0])
        out = plan.forward(x)
        plan.busy = True
        ctx.plan = plan
        return out

    @staticmethod
    def backward(ctx, gout):
        plan = ctx.plan
        gx, grads = plan.backward(gout)
        plan.busy = False
        return (gx, None, *grads)


class FusedSequential(nn.Sequential):
    """The nn.Sequential it replaces (same modules and state_dict), run from a prebuilt native plan."""

    def _count_batches(self):
        for m in self:  # what nn.BatchNorm2d.forward would have done
            if isinstance(m, nn.BatchNorm2d) and m.num_batches_tracked is not None:
                m.num_batches_tracked.add_(1)

    def forward(self, x):
        if x.device.type == DEVICE and x.dtype == torch.float32 and x.dim() == 4:
            grad = torch.is_grad_enabled()
            if self.training and grad:
                self._count_batches()
                return _StackFn.apply(x, self, *_params(self))
            if not self.training and not grad:
                return _plan(self, x.shape, False, False).forward(x)
        return super().forward(x)


def accelerate(model):
    """Swap every fusable nn.Sequential of `model` for a FusedSequential, in place. Returns a short description."""
    count = 0
    for m in model.modules():
        if type(m) is nn.Sequential and fusable(m):
            m.__class__ = FusedSequential
            count += 1
    return f"{count} fused stacks on {core.adapter_name()}"


_seen = weakref.WeakSet()


def _auto_fuse(module, args):
    # global forward pre-hook: the first time a plain nn.Sequential sees a device tensor, decide once whether to fuse it
    if type(module) is not nn.Sequential or module in _seen:
        return None
    x = args[0] if args else None
    if isinstance(x, torch.Tensor) and x.device.type == DEVICE:
        _seen.add(module)
        if fusable(module):
            module.__class__ = FusedSequential
    return None


if os.environ.get("OMARCHY_MAC_TORCH_AUTO_FUSE", "1") != "0":
    nn.modules.module.register_module_forward_pre_hook(_auto_fuse)
