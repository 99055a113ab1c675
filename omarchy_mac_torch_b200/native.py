"""Loads the C++ device extension and registers the "omarchy_mac_torch" PrivateUse1 device with PyTorch (the public
out-of-tree backend route: rename_privateuse1_backend + generated tensor/module methods + a device module).

Same Python surface as the reference's omarchy_mac_torch/native.py (DEVICE, FALLBACKS, synchronize, empty_cache,
memory_*, set_queue_depth, validate_kernels, the torch.omarchy_mac_torch device module); the WGSL kernel generator
hand-off and the on-disk tuning cache of the reference have no counterpart because the CUDA kernels are prebuilt."""

import ctypes
import json
import os
import pathlib
import types

import torch

_HERE = pathlib.Path(__file__).resolve().parent
DEVICE = "omarchy_mac_torch"


def _require_build():
    so, lib, info = _HERE / "_native.so", _HERE / "lib" / "libomt_b200.so", _HERE / "_build_info.json"
    if not (so.exists() and lib.exists() and info.exists()):
        raise ImportError("omarchy-mac-torch: the native backend is not built; run `python -m omarchy_mac_torch_b200.build`")
    built = json.loads(info.read_text())["torch"].split("+")[0]
    if built != torch.__version__.split("+")[0]:
        raise ImportError(f"omarchy-mac-torch was built against torch {built} but torch {torch.__version__} is installed; rebuild")
    return lib


ctypes.CDLL(str(_require_build()), mode=ctypes.RTLD_GLOBAL)
from omarchy_mac_torch_b200 import _native as core  # noqa: E402

torch.utils.rename_privateuse1_backend(DEVICE)
torch.utils.generate_methods_for_privateuse1_backend(for_tensor=True, for_module=True, for_packed_sequence=True, for_storage=True)

core.set_fold(int(os.environ.get("OMARCHY_MAC_TORCH_FOLD", "1")))
# OMARCHY_MAC_TORCH_TUNE=1: the first use of a convolution (pass, geometry) times the library's candidate tile plans and keeps
# the winner (the reference tunes by default, omarchy_mac_torch/native.py:75; here the built-in rules are the default and
# the timing pass is opt-in, because it synchronises the stream and a step may be under CUDA-graph capture).
TUNING = os.environ.get("OMARCHY_MAC_TORCH_TUNE", "0") == "1"
core.set_tuning(TUNING, 4)
core.set_debug(os.environ.get("OMARCHY_MAC_TORCH_DEBUG", "0") == "1")
# conv outputs are produced channels-last (the layout the tensor-core kernels read) unless this is set to 0
core.set_channels_last(int(os.environ.get("OMARCHY_MAC_TORCH_CHANNELS_LAST", "1")))


def synchronize():
    """Wait for all queued device work; raises if a kernel failed asynchronously."""
    core.sync()


def empty_cache():
    core.empty_cache()


def memory_allocated():
    return core.memory_allocated()


def memory_reserved():
    return core.memory_reserved()


def set_queue_depth(depth=3, chunk=64):
    """Kept for API parity. The reference bounded its wgpu queue so a desktop compositor sharing the GPU stayed
    responsive; CUDA streams on a compute-only B200 need no such throttle, so this records nothing."""
    core.set_queue(chunk, depth)


def validate_kernels():
    """Kernels are compiled ahead of time for sm_100a, so there is nothing to compile at run time: no failures."""
    return core.validate_kernels()


class _DeviceContext:
    def __init__(self, device=None):
        self.device = device

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


def _device_module():
    m = types.ModuleType("torch." + DEVICE)
    const = lambda v: (lambda *a, **k: v)
    m.is_available, m.is_initialized, m._is_in_bad_fork = const(True), const(True), const(False)
    m._lazy_init, m.set_device = const(None), const(None)
    m.device_count, m.current_device = const(1), const(0)
    m.get_amp_supported_dtype = const([torch.float32])
    m.synchronize = lambda device=None: core.sync()
    m.empty_cache = core.empty_cache
    m.memory_allocated = lambda device=None: core.memory_allocated()
    m.memory_reserved = lambda device=None: core.memory_reserved()
    m.manual_seed = m.manual_seed_all = lambda seed: core.manual_seed(int(seed) & 0xFFFFFFFFFFFFFFFF)
    m.seed = m.seed_all = core.seed
    m.initial_seed = core.initial_seed
    m.get_rng_state = lambda device=None: core.get_rng_state()
    m.set_rng_state = lambda state, device=None: core.set_rng_state(state)
    m.device = _DeviceContext
    return m


torch._register_device_module(DEVICE, _device_module())


class _Fallbacks:
    """Read-only view of the ops that did not run on this library's kernels, with why: {"op (reason)": count}.
    An entry means the call was served by ATen's CUDA kernel (or, if ATen has none, on the host)."""

    def _d(self):
        return core.fallback_counts()

    def keys(self):
        return self._d().keys()

    def items(self):
        return self._d().items()

    def values(self):
        return self._d().values()

    def __getitem__(self, k):
        return self._d()[k]

    def __contains__(self, k):
        return k in self._d()

    def __iter__(self):
        return iter(self._d())

    def __len__(self):
        return len(self._d())

    def __bool__(self):
        return bool(self._d())

    def clear(self):
        core.reset_fallbacks()

    def __repr__(self):
        return repr(self._d())


FALLBACKS = _Fallbacks()


# ---- on-disk cache of the convolution tuning (omarchy_mac_torch/native.py:182-206): read at import and written at exit, only
# when tuning is on, so that a default run never depends on what an earlier process measured ----
_TUNE_FILE = os.path.expanduser(os.environ.get("OMARCHY_MAC_TORCH_TUNE_FILE", "~/.cache/omarchy-mac-torch-b200/tuning.json"))


def load_tuning(path=None):
    """Install the plan overrides stored in a tuning file ({"pass,n,ci,co,ih,iw,oh,ow,ks,stride,pad": [tile, mult]}); returns
    how many the library took."""
    import json
    with open(path or _TUNE_FILE) as f:
        return core.tune_load({k: (int(v[0]), float(v[1])) for k, v in json.load(f).items()})


def save_tuning(path=None):
    """Merge the current plan overrides into the tuning file."""
    import json
    path = path or _TUNE_FILE
    os.makedirs(os.path.dirname(path), exist_ok=True)
    old = {}
    try:
        with open(path) as f:
            old = json.load(f)
    except (OSError, ValueError):
        pass
    old.update({k: list(v) for k, v in core.tune_dump().items()})
    with open(path, "w") as f:
        json.dump(old, f)


if TUNING:
    import atexit

    try:
        load_tuning()
    except (OSError, ValueError, TypeError):
        pass

    def _save_tuning_at_exit():
        try:
            save_tuning()
        except Exception:
            pass

    atexit.register(_save_tuning_at_exit)

