"""Shadow mode: run every op on the CPU as well and report where the device result differs (a debugging aid with the
same entry points as the reference's omarchy_mac_torch/debug.py: `shadow()` context manager, OMARCHY_MAC_TORCH_SHADOW=1)."""

import contextlib
import os

import torch
from torch.utils._python_dispatch import TorchDispatchMode
from torch.utils._pytree import tree_map

from omarchy_mac_torch_b200.native import DEVICE


class _Shadow(TorchDispatchMode):
    def __init__(self, tol=1e-3, verbose=False):
        super().__init__()
        self.tol, self.verbose, self.mismatches = tol, verbose, []

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        to_cpu = lambda t: t.detach().cpu() if isinstance(t, torch.Tensor) and t.device.type == DEVICE else t
        ref_args, ref_kwargs = tree_map(to_cpu, args), tree_map(to_cpu, kwargs)
        out = func(*args, **kwargs)
        name = str(func)
        if any(s in name for s in ("empty", "_copy_from", "random", "normal", "uniform", "dropout", "bernoulli")):
            return out
        try:
            ref = func(*ref_args, **ref_kwargs)
        except Exception:
            return out
        flat_o = out if isinstance(out, (tuple, list)) else (out,)
        flat_r = ref if isinstance(ref, (tuple, list)) else (ref,)
        for o, r in zip(flat_o, flat_r):
            if isinstance(o, torch.Tensor) and isinstance(r, torch.Tensor) and o.is_floating_point() and o.numel():
                err = ((o.detach().cpu() - r).abs().max() / r.abs().max().clamp_min(1e-12)).item()
                if err > self.tol:
                    self.mismatches.append((name, err))
                    if self.verbose:
                        print(f"[shadow] {name}: relative error {err:.2e}")
        return out


@contextlib.contextmanager
def shadow(tol=1e-3, verbose=True):
    mode = _Shadow(tol, verbose)
    with mode:
        yield mode


if os.environ.get("OMARCHY_MAC_TORCH_SHADOW", "0") == "1":
    _global = _Shadow(verbose=True)
    _global.__enter__()
