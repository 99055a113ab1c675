"""B200-native hot path of omarchy-mac-torch: fp32 conv fwd/dgrad/wgrad, fused conv+BN+ReLU(+pool) stacks, depthwise
conv, BatchNorm, fused SGD/Adam/AdamW, behind the "omarchy_mac_torch" PyTorch device.

    import omarchy_mac_torch_b200 as omt   # registers the "omarchy_mac_torch" device
    model = model.to(omt.DEVICE)
    omt.accelerate(model)                  # optional: fused conv/BN/ReLU/pool stacks

The device registration loads on first attribute access, so `omarchy_mac_torch_b200.capi` (ctypes binding of the C
ABI) and `omarchy_mac_torch_b200.build` can be imported where the torch extension has not been built."""

__version__ = "0.1.0"

_PUBLIC = ["DEVICE", "FALLBACKS", "FusedSequential", "accelerate", "debug", "empty_cache", "memory_allocated", "memory_reserved",
           "set_queue_depth", "synchronize", "tune_cpu", "validate_kernels"]
__all__ = list(_PUBLIC)


def _load():
    import importlib
    import sys
    me = sys.modules[__name__]
    native = importlib.import_module(__name__ + ".native")      # registers the device (C++ backend)
    importlib.import_module(__name__ + ".optim")                 # fused optimizers by default
    debug = importlib.import_module(__name__ + ".debug")
    importlib.import_module(__name__ + ".compile")               # torch.compile(model, backend="omarchy_mac_torch")
    stacks = importlib.import_module(__name__ + ".stacks")
    utils = importlib.import_module(__name__ + ".utils")
    for k in ("DEVICE", "FALLBACKS", "empty_cache", "memory_allocated", "memory_reserved", "set_queue_depth", "synchronize",
              "validate_kernels"):
        setattr(me, k, getattr(native, k))
    me.FusedSequential, me.accelerate, me.debug, me.tune_cpu = stacks.FusedSequential, stacks.accelerate, debug, utils.tune_cpu
    sys.modules.setdefault("omarchy_mac_torch", me)              # code written for the reference imports this name
    me._loaded = True


def __getattr__(name):
    if name in _PUBLIC and not globals().get("_loaded"):
        _load()
        return globals()[name]
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
