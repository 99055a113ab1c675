"""B200-native hot path of omarchy-mac-torch: fp32 conv fwd/dgrad/wgrad, fused conv+BN+ReLU(+pool) plans, depthwise
conv, BatchNorm, fused SGD/Adam/AdamW, behind the "omarchy_mac_torch" PyTorch device.

    import omarchy_mac_torch_b200 as omt   # registers the "omarchy_mac_torch" device (needs a B200)
    model = model.to(omt.DEVICE)

Importing this package never touches the GPU by itself unless the device extension is present; `capi` (the ctypes
binding of the C ABI) and `build` can be imported on a machine without one."""

__version__ = "0.1.0"


def __getattr__(name):
    # the device registration (and everything that needs it) loads on first use, so that `import
    # omarchy_mac_torch_b200.capi` / `.build` work where the torch extension has not been built
    if name in {"DEVICE", "FALLBACKS", "FusedSequential", "accelerate", "debug", "empty_cache", "memory_allocated",
                "memory_reserved", "set_queue_depth", "synchronize", "tune_cpu", "validate_kernels", "native", "stacks",
                "optim", "compile", "dp"}:
        from omarchy_mac_torch_b200 import _api
        return getattr(_api, name)
    raise AttributeError(name)
