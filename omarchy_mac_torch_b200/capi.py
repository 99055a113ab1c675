"""ctypes binding of libomt_b200.so (the C ABI declared in include/omt_b200.h).

Used by the parity tests and bench to call the kernels directly on device memory owned by torch CUDA tensors, without
going through the PyTorch device extension. Every call raises OmtError on a non-zero status; there is no fallback."""

import ctypes as C
import pathlib

_HERE = pathlib.Path(__file__).resolve().parent
LIB_PATH = _HERE / "lib" / "libomt_b200.so"

# flags (include/omt_b200.h)
EPI_BIAS, EPI_RELU, EPI_BNSTATS, EPI_ACCUM, FORCE_SIMT, FORCE_TC, PRECISE_ACCUM = 1, 2, 4, 8, 0x100, 0x200, 0x400
BN_RELU, BN_FUNCTIONAL, BN_MASKBITS = 1, 2, 4


class OmtError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"libomt_b200 error {code}: {msg}")
        self.code = code


class ConvGeo(C.Structure):
    _fields_ = [(k, C.c_int32) for k in ("n", "ci", "co", "ih", "iw", "oh", "ow", "ks", "stride", "pad", "groups")]


class Act(C.Structure):
    _fields_ = [("p", C.c_void_p), ("sn", C.c_int64), ("sc", C.c_int64), ("sh", C.c_int64), ("sw", C.c_int64)]


class Pool(C.Structure):
    _fields_ = [(k, C.c_int32) for k in ("kh", "kw", "sh", "sw", "ph", "pw", "dh", "dw")]


class Param(C.Structure):
    _fields_ = [("p", C.c_void_p), ("g", C.c_void_p), ("m", C.c_void_p), ("v", C.c_void_p), ("step", C.c_void_p),
                ("numel", C.c_int64)]


_P, _I, _U, _F, _SZ, _I64 = C.c_void_p, C.c_int32, C.c_uint32, C.c_float, C.c_size_t, C.c_int64
_G, _A, _PL = C.POINTER(ConvGeo), C.POINTER(Act), C.POINTER(Pool)

# name -> (restype, argtypes); status-returning functions are checked automatically
SIGNATURES = {
    "omt_init": (_I, [_I]),
    "omt_device": (_I, []),
    "omt_last_error": (_I, [C.c_char_p, _SZ]),
    "omt_check_errors": (_I, []),
    "omt_sync": (_I, []),
    "omt_malloc": (_P, [_SZ, _P]),
    "omt_free": (None, [_P]),
    "omt_record_stream": (_I, [_P, _P]),
    "omt_empty_cache": (None, []),
    "omt_memory_allocated": (_SZ, []),
    "omt_memory_reserved": (_SZ, []),
    "omt_stream_create": (_P, [_I]),
    "omt_stream_destroy": (_I, [_P]),
    "omt_stream_sync": (_I, [_P]),
    "omt_stream_query": (_I, [_P]),
    "omt_event_create": (_P, [_I]),
    "omt_event_destroy": (_I, [_P]),
    "omt_event_record": (_I, [_P, _P]),
    "omt_event_query": (_I, [_P]),
    "omt_event_sync": (_I, [_P]),
    "omt_stream_wait_event": (_I, [_P, _P]),
    "omt_event_elapsed_ms": (_I, [_P, _P, C.POINTER(C.c_float)]),
    "omt_memcpy_h2d": (_I, [_P, _P, _SZ, _P]),
    "omt_memcpy_d2h": (_I, [_P, _P, _SZ, _P]),
    "omt_memcpy_d2d": (_I, [_P, _P, _SZ, _P]),
    "omt_memset": (_I, [_P, _I, _SZ, _P]),
    "omt_launch_count": (C.c_uint64, []),
    "omt_kernel_counts": (_SZ, [C.c_char_p, _SZ, _I]),
    "omt_conv_workspace_bytes": (_SZ, [_I, _G, _U]),
    "omt_conv_fwd": (_I, [_G, _A, _P, _P, _A, _P, _U, _P, _SZ, _P]),
    "omt_conv_plan_set": (_I, [_I, _G, C.c_int32, C.c_double]),
    "omt_conv_plan_get": (_I, [_I, _G, C.POINTER(C.c_int32), C.POINTER(C.c_double)]),
    "omt_conv_autotune": (_I, [_I, _G, C.POINTER(C.c_int32), C.POINTER(C.c_double), C.POINTER(C.c_float), C.POINTER(C.c_float), _P]),
    "omt_conv_plans_dump": (_SZ, [C.c_char_p, _SZ]),
    "omt_conv_plans_load": (_I, [C.c_char_p]),
    "omt_conv_dgrad": (_I, [_G, _A, _P, _A, _U, _P, _SZ, _P]),
    "omt_conv_wgrad": (_I, [_G, _A, _A, _P, _F, _U, _P, _SZ, _P]),
    "omt_conv_wgrad_noalloc_capacity": (_SZ, []),
    "omt_conv_wgrad_noalloc": (_I, [_G, _A, _A, _P, _F, _P]),
    "omt_conv_bias_grad": (_I, [_A, _I, _I, _I, _I, _P, _F, _P]),
    "omt_kernel_timing": (_I, [_I]),
    "omt_kernel_times": (_SZ, [C.c_char_p, _SZ, _I]),
    "omt_gemm": (_I, [_P, _I64, _I64, _P, _I64, _I64, _P, _P, _I, _I, _I, _P]),
    "omt_pointwise": (_I, [_P, _I, _P, _P, _P, _P, _I, _P, _P]),
    "omt_log_softmax": (_I, [_P, _P, _I64, _I, _P]),
    "omt_log_softmax_backward": (_I, [_P, _P, _P, _I64, _I, _P]),
    "omt_nll_loss": (_I, [_P, _P, _P, _P, _P, _I64, _I, _I64, _I, _P]),
    "omt_nll_loss_backward": (_I, [_P, _P, _P, _P, _P, _I64, _I, _I64, _I, _P]),
    "omt_softmax_nll": (_I, [_P, _P, _P, _P, _P, _P, _I64, _I, _I64, _I, _P]),
    "omt_softmax_nll_backward": (_I, [_P, _P, _P, _P, _P, _P, _I64, _I, _I64, _I, _P]),
    "omt_conv_timing": (_I, [_I]),
    "omt_conv_timing_read": (_I, [C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_int64), _I]),
    "omt_conv_timing_bytes": (_I, [C.POINTER(C.c_double)]),
    "omt_dw_fwd": (_I, [_G, _A, _P, _P, _A, _U, _P]),
    "omt_dw_dgrad": (_I, [_G, _A, _P, _A, _P]),
    "omt_dw_wgrad": (_I, [_G, _A, _A, _P, _F, _P]),
    "omt_bn_stats": (_I, [_A, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P, _F, _F, _U, _P]),
    "omt_bn_stats_from_partials": (_I, [_P, _I, _I, _P, _P, _P, _P, _P, _P, _P, _F, _F, _U, _P]),
    "omt_conv_bnstats_groups": (C.c_int32, [_G, _A, _A]),
    "omt_conv_bnstats_floats": (_SZ, [C.c_int32, C.c_int32]),
    "omt_bn_apply": (_I, [_A, _A, _I, _I, _I, _I, _P, _P, _P, _P, _U, _P]),
    "omt_bn_apply_add": (_I, [_A, _A, _A, _I, _I, _I, _I, _P, _P, _P, _P, _U, _P]),
    "omt_bn_apply_pool2": (_I, [_A, _A, _A, _P, _I, _I, _I, _I, _P, _P, _P, _P, _U, _P]),
    "omt_bn_eval": (_I, [_A, _A, _I, _I, _I, _I, _P, _P, _P, _P, _F, _U, _P]),
    "omt_bn_backward": (_I, [_A, _A, _A, _A, _I, _I, _I, _I, _P, _P, _P, _P, _F, _U, _P]),
    "omt_bn_backward_add": (_I, [_A, _A, _A, _A, _A, _I, _I, _I, _I, _P, _P, _P, _P, _F, _U, _P]),
    "omt_pool2_fwd": (_I, [_A, _A, _P, _I, _I, _I, _I, _P]),
    "omt_pool2_bwd": (_I, [_A, _P, _A, _I, _I, _I, _I, _P]),
    "omt_avgpool2_fwd": (_I, [_A, _A, _I, _I, _I, _I, _P]),
    "omt_avgpool2_bwd": (_I, [_A, _A, _I, _I, _I, _I, _P]),
    "omt_maxpool_fwd": (_I, [_A, _A, _P, _I, _I, _I, _I, _I, _I, _PL, _P]),
    "omt_maxpool_bwd": (_I, [_A, _P, _A, _I, _I, _I, _I, _I, _I, _PL, _P]),
    "omt_avgpool_fwd": (_I, [_A, _A, _I, _I, _I, _I, _I, _I, _PL, _I, _I, _P]),
    "omt_avgpool_bwd": (_I, [_A, _A, _I, _I, _I, _I, _I, _I, _PL, _I, _I, _P]),
    "omt_adaptive_avgpool_fwd": (_I, [_A, _A, _I, _I, _I, _I, _I, _I, _P]),
    "omt_adaptive_avgpool_bwd": (_I, [_A, _A, _I, _I, _I, _I, _I, _I, _P]),
    "omt_sgd": (_I, [C.POINTER(Param), _I, _F, _F, _F, _F, _I, _I, _I, _P]),
    "omt_adam": (_I, [C.POINTER(Param), _I, _F, _F, _F, _F, _F, _I, _I, _P]),
    "omt_scale_copy": (_I, [_P, _P, _I64, _F, _P]),
    "omt_act_copy": (_I, [_A, _A, _I, _I, _I, _I, _P]),
}
# these return a status that is not an error code convention (counts, booleans)
_UNCHECKED = {"omt_device", "omt_last_error", "omt_stream_query", "omt_event_query"}

_lib = None


def lib():
    """The loaded library (loads on first use; raises if it has not been built)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m omarchy_mac_torch_b200.build`")
        l = C.CDLL(str(LIB_PATH), mode=C.RTLD_GLOBAL)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(l, name)
            fn.restype, fn.argtypes = res, args
        _lib = l
    return _lib


def last_error():
    buf = C.create_string_buffer(512)
    lib().omt_last_error(buf, 512)
    return buf.value.decode(errors="replace")


def call(name, *args):
    """Call a status-returning entry point; raise OmtError on failure."""
    r = getattr(lib(), name)(*args)
    if SIGNATURES[name][0] is _I and name not in _UNCHECKED and r != 0:
        raise OmtError(r, last_error())
    return r


# ---- helpers for torch CUDA tensors ----

def ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


def act(t):
    """OmtAct for a 4-D float32 CUDA tensor (any strides)."""
    assert t.dim() == 4 and t.dtype.is_floating_point and t.element_size() == 4
    sn, sc, sh, sw = t.stride()
    return Act(t.data_ptr(), sn, sc, sh, sw)


def null_act():
    return Act(0, 0, 0, 0, 0)


def geo(n, ci, co, ih, iw, ks, stride, pad, groups=1):
    oh = (ih + 2 * pad - ks) // stride + 1
    ow = (iw + 2 * pad - ks) // stride + 1
    return ConvGeo(n, ci, co, ih, iw, oh, ow, ks, stride, pad, groups)


def stream_handle(stream=None):
    """cudaStream_t of a torch.cuda.Stream (default: torch's current stream)."""
    import torch
    s = stream if stream is not None else torch.cuda.current_stream()
    return C.c_void_p(s.cuda_stream)


def conv_timing(enable):
    call("omt_conv_timing", int(enable))


def conv_timing_read(reset=True):
    """{pass: (flops, ms, calls, algorithmic bytes)} for fwd / dgrad / wgrad since the last reset."""
    f, m, c, b = (C.c_double * 3)(), (C.c_double * 3)(), (C.c_int64 * 3)(), (C.c_double * 3)()
    call("omt_conv_timing_bytes", b)
    call("omt_conv_timing_read", f, m, c, int(reset))
    return {k: (f[i], m[i], c[i], b[i]) for i, k in enumerate(("fwd", "dgrad", "wgrad"))}


def conv_autotune(kind, g, stream=None):
    """Time the planner's rules and every candidate plan for pass `kind` (0 forward, 1 input gradient, 2 weight gradient) of
    geometry `g`; the fastest becomes the stored override when it beats the rules by more than 3 %. Returns
    (tile, mult, best_ms, rule_ms); tile 0 and mult 1.0 mean the rules stay."""
    tile, mult, best, rule = C.c_int32(0), C.c_double(1.0), C.c_float(0), C.c_float(0)
    call("omt_conv_autotune", int(kind), g, C.byref(tile), C.byref(mult), C.byref(best), C.byref(rule), stream_handle(stream))
    return tile.value, mult.value, best.value, rule.value


def conv_plan_get(kind, g):
    """(tile, mult) of the stored override for (kind, g), or None."""
    tile, mult = C.c_int32(0), C.c_double(1.0)
    have = lib().omt_conv_plan_get(int(kind), g, C.byref(tile), C.byref(mult))
    return (tile.value, mult.value) if have == 1 else None


def conv_plans_dump():
    """All stored overrides as {"pass,n,ci,co,ih,iw,oh,ow,ks,stride,pad": (tile, mult)}."""
    n = lib().omt_conv_plans_dump(None, 0)
    buf = C.create_string_buffer(n + 1)
    lib().omt_conv_plans_dump(buf, n + 1)
    out = {}
    for line in buf.value.decode().splitlines():
        k, _, v = line.partition("=")
        t, _, m = v.partition(",")
        out[k] = (int(t), float(m))
    return out


def conv_plans_load(entries):
    """Store overrides from a {key: (tile, mult)} mapping as conv_plans_dump returns it; returns how many were taken."""
    text = "".join(f"{k}={int(v[0])},{float(v[1])!r}\n" for k, v in entries.items())
    return lib().omt_conv_plans_load(text.encode())


def kernel_counts(reset=False):
    n = lib().omt_kernel_counts(None, 0, 0)
    buf = C.create_string_buffer(n + 1)
    lib().omt_kernel_counts(buf, n + 1, 1 if reset else 0)
    out = {}
    for line in buf.value.decode().splitlines():
        k, _, v = line.partition("=")
        out[k] = int(v)
    return out


# ---- convenience wrappers on torch CUDA tensors (tests, bench, smoke) ---------------------------------------------------
# Each allocates its outputs with torch, runs on torch's current stream and returns tensors. `cl=True` makes the
# outputs channels-last.

def _empty(shape, like, cl=False):
    import torch
    fmt = torch.channels_last if cl and len(shape) == 4 else torch.contiguous_format
    return torch.empty(shape, device=like.device, dtype=torch.float32, memory_format=fmt)


def conv_fwd(x, w, bias=None, stride=1, pad=0, flags=0, cl=False, stats=None):
    n, ci, ih, iw = x.shape
    co, _, ks, _ = w.shape
    g = geo(n, ci, co, ih, iw, ks, stride, pad)
    y = _empty((n, co, g.oh, g.ow), x, cl)
    if bias is not None:
        flags |= EPI_BIAS
    call("omt_conv_fwd", g, act(x), ptr(w), ptr(bias), act(y), ptr(stats), flags, None, 0, stream_handle())
    return y


def conv_dgrad(gy, w, in_hw, stride=1, pad=0, flags=0, cl=False, acc=None):
    """acc: a tensor to accumulate into (EPI_ACCUM) instead of a fresh output"""
    n, co = gy.shape[:2]
    _, ci, ks, _ = w.shape
    g = geo(n, ci, co, in_hw[0], in_hw[1], ks, stride, pad)
    dx = acc if acc is not None else _empty((n, ci, in_hw[0], in_hw[1]), gy, cl)
    if acc is not None:
        flags |= EPI_ACCUM
    call("omt_conv_dgrad", g, act(gy), ptr(w), act(dx), flags, None, 0, stream_handle())
    return dx


def conv_wgrad(x, gy, ks, stride=1, pad=0, flags=0, scale=1.0):
    n, ci, ih, iw = x.shape
    co = gy.shape[1]
    g = geo(n, ci, co, ih, iw, ks, stride, pad)
    dw = _empty((co, ci, ks, ks), x)
    call("omt_conv_wgrad", g, act(x), act(gy), ptr(dw), scale, flags, None, 0, stream_handle())
    return dw


def conv_bias_grad(gy, scale=1.0):
    n, c, h, w = gy.shape
    db = _empty((c,), gy)
    call("omt_conv_bias_grad", act(gy), n, c, h, w, ptr(db), scale, stream_handle())
    return db


def dw_fwd(x, w, bias=None, stride=1, pad=0, flags=0, cl=False):
    n, c, ih, iw = x.shape
    ks = w.shape[-1]
    g = geo(n, c, c, ih, iw, ks, stride, pad, groups=c)
    y = _empty((n, c, g.oh, g.ow), x, cl)
    if bias is not None:
        flags |= EPI_BIAS
    call("omt_dw_fwd", g, act(x), ptr(w), ptr(bias), act(y), flags, stream_handle())
    return y


def dw_dgrad(gy, w, in_hw, stride=1, pad=0, cl=False):
    n, c = gy.shape[:2]
    ks = w.shape[-1]
    g = geo(n, c, c, in_hw[0], in_hw[1], ks, stride, pad, groups=c)
    dx = _empty((n, c, in_hw[0], in_hw[1]), gy, cl)
    call("omt_dw_dgrad", g, act(gy), ptr(w), act(dx), stream_handle())
    return dx


def dw_wgrad(x, gy, ks, stride=1, pad=0, scale=1.0):
    n, c, ih, iw = x.shape
    g = geo(n, c, c, ih, iw, ks, stride, pad, groups=c)
    dw = _empty((c, 1, ks, ks), x)
    call("omt_dw_wgrad", g, act(x), act(gy), ptr(dw), scale, stream_handle())
    return dw


def bn_train(x, gamma, beta, rm, rv, momentum=0.1, eps=1e-5, relu=False, functional=False):
    """-> y, mean, invstd (and new_rm, new_rv when functional). rm/rv are updated in place otherwise."""
    import torch
    n, c, h, w = x.shape
    mean, var, invstd = (_empty((c,), x) for _ in range(3))
    nrm, nrv = (_empty((c,), x), _empty((c,), x)) if functional else (None, None)
    call("omt_bn_stats", act(x), n, c, h, w, ptr(mean), ptr(var), ptr(invstd), ptr(rm), ptr(rv), ptr(nrm), ptr(nrv), momentum, eps,
         BN_FUNCTIONAL if functional else 0, stream_handle())
    y = torch.empty_like(x)
    call("omt_bn_apply", act(x), act(y), n, c, h, w, ptr(mean), ptr(invstd), ptr(gamma), ptr(beta), BN_RELU if relu else 0, stream_handle())
    return (y, mean, invstd, nrm, nrv) if functional else (y, mean, invstd)


def conv_fwd_bnstats(x, w, bias=None, stride=1, pad=0, flags=0):
    """Forward convolution into a channels-last y with the batch-norm partial statistics of y taken in the epilogue.
    -> y, partials, groups; groups == 0 (and partials None) when this call cannot produce them."""
    import torch
    n, ci, ih, iw = x.shape
    co, _, ks, _ = w.shape
    g = geo(n, ci, co, ih, iw, ks, stride, pad)
    y = _empty((n, co, g.oh, g.ow), x, True)
    groups = lib().omt_conv_bnstats_groups(g, act(x), act(y))
    if groups == 0:
        return conv_fwd(x, w, bias, stride, pad, flags, cl=True), None, 0
    part = torch.full((lib().omt_conv_bnstats_floats(groups, co),), float("nan"), device=x.device, dtype=torch.float32)
    call("omt_conv_fwd", g, act(x), ptr(w), ptr(bias), act(y), ptr(part), flags | EPI_BNSTATS | (EPI_BIAS if bias is not None else 0), None, 0,
         stream_handle())
    return y, part, groups


def bn_stats_from_partials(part, groups, c, rm=None, rv=None, momentum=0.1, eps=1e-5, functional=False):
    """-> mean, var, invstd (and new_rm, new_rv when functional) from what conv_fwd_bnstats wrote."""
    mean, var, invstd = (_empty((c,), part) for _ in range(3))
    nrm, nrv = (_empty((c,), part), _empty((c,), part)) if functional else (None, None)
    call("omt_bn_stats_from_partials", ptr(part), groups, c, ptr(mean), ptr(var), ptr(invstd), ptr(rm), ptr(rv), ptr(nrm), ptr(nrv), momentum, eps,
         BN_FUNCTIONAL if functional else 0, stream_handle())
    return (mean, var, invstd, nrm, nrv) if functional else (mean, var, invstd)


def bn_eval(x, gamma, beta, rm, rv, eps=1e-5, relu=False):
    import torch
    n, c, h, w = x.shape
    y = torch.empty_like(x)
    call("omt_bn_eval", act(x), act(y), n, c, h, w, ptr(rm), ptr(rv), ptr(gamma), ptr(beta), eps, BN_RELU if relu else 0, stream_handle())
    return y


def bn_backward(gy, x, y, mean, invstd, gamma, relu=False, need_dx=True, scale=1.0):
    import torch
    n, c, h, w = x.shape
    dx = torch.empty_like(x) if need_dx else None
    dgb = _empty((2, c), x)
    call("omt_bn_backward", act(gy), act(x), act(y) if y is not None else null_act(), act(dx) if need_dx else null_act(), n, c, h, w,
         ptr(mean), ptr(invstd), ptr(gamma), ptr(dgb), scale, BN_RELU if relu else 0, stream_handle())
    return dx, dgb[0], dgb[1]


def pool2_fwd(x):
    import torch
    n, c, h, w = x.shape
    cl = x.stride(1) == 1 and c > 1
    y = _empty((n, c, h // 2, w // 2), x, cl)
    idx = torch.empty_strided(y.shape, y.stride(), device=x.device, dtype=torch.uint8)
    call("omt_pool2_fwd", act(x), act(y), ptr(idx), n, c, h, w, stream_handle())
    return y, idx


def pool2_bwd(gy, idx, hw):
    n, c = gy.shape[:2]
    gx = _empty((n, c, hw[0], hw[1]), gy, gy.stride(1) == 1 and c > 1)
    call("omt_pool2_bwd", act(gy), ptr(idx), act(gx), n, c, hw[0], hw[1], stream_handle())
    return gx


def maxpool_fwd(x, k, s, p, d=1):
    import torch
    n, c, ih, iw = x.shape
    oh = (ih + 2 * p - d * (k - 1) - 1) // s + 1
    ow = (iw + 2 * p - d * (k - 1) - 1) // s + 1
    cl = x.stride(1) == 1 and c > 1
    y = _empty((n, c, oh, ow), x, cl)
    idx = torch.empty_strided(y.shape, y.stride(), device=x.device, dtype=torch.int64)
    call("omt_maxpool_fwd", act(x), act(y), ptr(idx), n, c, ih, iw, oh, ow, Pool(k, k, s, s, p, p, d, d), stream_handle())
    return y, idx


def maxpool_bwd(gy, idx, in_hw, k, s, p, d=1):
    n, c, oh, ow = gy.shape
    gx = _empty((n, c, in_hw[0], in_hw[1]), gy, gy.stride(1) == 1 and c > 1)
    call("omt_maxpool_bwd", act(gy), ptr(idx), act(gx), n, c, in_hw[0], in_hw[1], oh, ow, Pool(k, k, s, s, p, p, d, d), stream_handle())
    return gx


def adaptive_avgpool_fwd(x, o):
    n, c, ih, iw = x.shape
    y = _empty((n, c, o, o), x, x.stride(1) == 1 and c > 1 and o > 1)
    call("omt_adaptive_avgpool_fwd", act(x), act(y), n, c, ih, iw, o, o, stream_handle())
    return y


def adaptive_avgpool_bwd(gy, in_hw):
    n, c, oh, ow = gy.shape
    gx = _empty((n, c, in_hw[0], in_hw[1]), gy)
    call("omt_adaptive_avgpool_bwd", act(gy), act(gx), n, c, in_hw[0], in_hw[1], oh, ow, stream_handle())
    return gx


def param_table(params, grads, ms=None, vs=None, steps=None):
    n = len(params)
    tab = (Param * n)()
    for i in range(n):
        tab[i] = Param(params[i].data_ptr(), grads[i].data_ptr(), ms[i].data_ptr() if ms and ms[i] is not None else 0,
                       vs[i].data_ptr() if vs else 0, steps[i].data_ptr() if steps else 0, params[i].numel())
    return tab


def sgd(params, grads, ms, lr, momentum=0.0, dampening=0.0, weight_decay=0.0, nesterov=False, first=False, maximize=False):
    tab = param_table(params, grads, ms)
    call("omt_sgd", tab, len(params), lr, momentum, dampening, weight_decay, int(nesterov), int(first), int(maximize), stream_handle())


def adam(params, grads, ms, vs, steps, lr, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, decoupled=False, maximize=False):
    tab = param_table(params, grads, ms, vs, steps)
    call("omt_adam", tab, len(params), lr, beta1, beta2, eps, weight_decay, int(decoupled), int(maximize), stream_handle())
