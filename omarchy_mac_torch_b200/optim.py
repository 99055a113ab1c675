"""torch.optim.SGD / Adam / AdamW pick their fused implementation by default when every parameter lives on the device.

PyTorch offers no hook for a backend to prefer its fused optimizers (left alone it takes the foreach path: several
launches per parameter), so the constructors are wrapped, as the reference's omarchy_mac_torch/optim.py does. An
explicit fused= or foreach= is respected; OMARCHY_MAC_TORCH_FUSED_OPTIM=0 disables the default."""

import functools
import os

import torch

from omarchy_mac_torch_b200.native import DEVICE


def _flat_params(params):
    for group in params:
        if isinstance(group, dict):
            yield from group["params"]
        else:
            yield group


def wants_fused(params, kwargs):
    """Whether the wrapped constructor should add fused=True (host-side rule; unit-tested without a device)."""
    flat = list(_flat_params(params))
    if not flat or any(p.device.type != DEVICE for p in flat):
        return False
    if kwargs.get("fused") is not None or kwargs.get("foreach") is not None or kwargs.get("differentiable"):
        return False
    return not isinstance(kwargs.get("lr", 0.0), torch.Tensor)  # only the float-lr overloads are registered


def _patch(cls):
    original = cls.__init__
    if getattr(original, "_omt_wrapped", False):
        return

    @functools.wraps(original)
    def init(self, params, *args, **kwargs):
        params = list(params)
        if wants_fused(params, kwargs):
            kwargs["fused"] = True
        original(self, params, *args, **kwargs)

    init._omt_wrapped = True
    cls.__init__ = init


if os.environ.get("OMARCHY_MAC_TORCH_FUSED_OPTIM", "1") != "0":
    for _c in (torch.optim.SGD, torch.optim.Adam, torch.optim.AdamW):
        _patch(_c)
