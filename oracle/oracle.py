"""Python face of the CPU oracle. TEST INFRASTRUCTURE ONLY (see oracle.c's header).

Two independent statements of the path's arithmetic live here:

  * `c.*`   numpy wrappers over oracle.c (plain loops, double accumulation), compiled to oracle/liboracle.so;
  * `aten_*` the reference's own oracle: PyTorch CPU aten ops called exactly as the reference's check scripts call
             them (tools/gemm_bench.py:26-38, notes/scripts/conv_kinds_check.py, tools/acceptance.py:51-98).

tests/test_oracle.py holds the two to each other and to the fixtures in tests/golden/."""

import ctypes as C
import pathlib
import subprocess

import numpy as np

_HERE = pathlib.Path(__file__).resolve().parent
_LIB = _HERE / "liboracle.so"


def build():
    """Compile oracle.c (gcc) if the shared object is missing or older than the source."""
    src = _HERE / "oracle.c"
    if not _LIB.exists() or _LIB.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["gcc", "-O2", "-fPIC", "-std=c11", "-shared", "-o", str(_LIB), str(src), "-lm"], check=True)
    return _LIB


_lib = None


def _l():
    global _lib
    if _lib is None:
        _lib = C.CDLL(str(build()))
    return _lib


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(C.c_void_p)


def _opt(a):
    if a is None:
        return None, C.c_void_p(0)
    return _f(a)


def out_hw(ih, iw, ks, stride, pad):
    return (ih + 2 * pad - ks) // stride + 1, (iw + 2 * pad - ks) // stride + 1


def rel_err(a, ref):
    """max|a-ref| / max|ref|: the metric of tools/gemm_bench.py:37."""
    a = np.asarray(a, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(a - ref).max() / max(np.abs(ref).max(), 1e-30)) if ref.size else 0.0


class c:
    """numpy wrappers over oracle.c"""

    @staticmethod
    def conv_fwd(x, w, bias=None, stride=1, pad=0, relu=False):
        x, xp = _f(x); w, wp = _f(w); b, bp = _opt(bias)
        n, ci, ih, iw = x.shape
        co, _, ks, _ = w.shape
        oh, ow = out_hw(ih, iw, ks, stride, pad)
        y = np.empty((n, co, oh, ow), np.float32)
        _l().orc_conv_fwd(xp, wp, bp, y.ctypes.data_as(C.c_void_p), n, ci, co, ih, iw, ks, stride, pad, int(relu))
        return y

    @staticmethod
    def conv_dgrad(gy, w, in_hw, stride=1, pad=0, phases=False):
        gy, gp = _f(gy); w, wp = _f(w)
        n, co = gy.shape[:2]
        _, ci, ks, _ = w.shape
        ih, iw = in_hw
        dx = np.zeros((n, ci, ih, iw), np.float32)
        fn = _l().orc_conv_dgrad_phases if phases else _l().orc_conv_dgrad
        fn(gp, wp, dx.ctypes.data_as(C.c_void_p), n, ci, co, ih, iw, ks, stride, pad)
        return dx

    @staticmethod
    def conv_wgrad(x, gy, ks, stride=1, pad=0):
        x, xp = _f(x); gy, gp = _f(gy)
        n, ci, ih, iw = x.shape
        co = gy.shape[1]
        dw = np.empty((co, ci, ks, ks), np.float32)
        _l().orc_conv_wgrad(xp, gp, dw.ctypes.data_as(C.c_void_p), n, ci, co, ih, iw, ks, stride, pad)
        return dw

    @staticmethod
    def wgrad_slices(M, N, K, bm, bn, mult=1.0):
        ks = C.c_int64(0)
        fn = _l().orc_wgrad_slices
        fn.argtypes = [C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_double, C.POINTER(C.c_int64)]
        s = fn(M, N, K, bm, bn, mult, C.byref(ks))
        return s, ks.value

    @staticmethod
    def bias_grad(gy):
        gy, gp = _f(gy)
        n, ch = gy.shape[:2]
        db = np.empty((ch,), np.float32)
        _l().orc_bias_grad(gp, db.ctypes.data_as(C.c_void_p), n, ch, int(np.prod(gy.shape[2:])))
        return db

    @staticmethod
    def dw_fwd(x, w, bias=None, stride=1, pad=0):
        x, xp = _f(x); w, wp = _f(w); b, bp = _opt(bias)
        n, ch, ih, iw = x.shape
        ks = w.shape[-1]
        oh, ow = out_hw(ih, iw, ks, stride, pad)
        y = np.empty((n, ch, oh, ow), np.float32)
        _l().orc_dw_fwd(xp, wp, bp, y.ctypes.data_as(C.c_void_p), n, ch, ih, iw, ks, stride, pad)
        return y

    @staticmethod
    def dw_dgrad(gy, w, in_hw, stride=1, pad=0):
        gy, gp = _f(gy); w, wp = _f(w)
        n, ch = gy.shape[:2]
        ks = w.shape[-1]
        dx = np.empty((n, ch, in_hw[0], in_hw[1]), np.float32)
        _l().orc_dw_dgrad(gp, wp, dx.ctypes.data_as(C.c_void_p), n, ch, in_hw[0], in_hw[1], ks, stride, pad)
        return dx

    @staticmethod
    def dw_wgrad(x, gy, ks, stride=1, pad=0):
        x, xp = _f(x); gy, gp = _f(gy)
        n, ch, ih, iw = x.shape
        dw = np.empty((ch, 1, ks, ks), np.float32)
        _l().orc_dw_wgrad(xp, gp, dw.ctypes.data_as(C.c_void_p), n, ch, ih, iw, ks, stride, pad)
        return dw

    @staticmethod
    def bn_stats(x, momentum=0.1, rm=None, rv=None):
        """-> mean, var(biased); rm/rv (float32 arrays) are updated in place when given."""
        x, xp = _f(x)
        n, ch = x.shape[:2]
        hw = int(np.prod(x.shape[2:]))
        mean = np.empty((ch,), np.float32); var = np.empty((ch,), np.float32)
        fn = _l().orc_bn_stats
        fn.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        fn(xp, n, ch, hw, momentum, mean.ctypes.data_as(C.c_void_p), var.ctypes.data_as(C.c_void_p),
           rm.ctypes.data_as(C.c_void_p) if rm is not None else None, rv.ctypes.data_as(C.c_void_p) if rv is not None else None)
        return mean, var

    @staticmethod
    def bn_apply(x, mean, invstd, gamma, beta, relu=False):
        x, xp = _f(x)
        n, ch = x.shape[:2]
        y = np.empty_like(x)
        args = [_f(a) for a in (mean, invstd, gamma, beta)]
        _l().orc_bn_apply(xp, y.ctypes.data_as(C.c_void_p), n, ch, int(np.prod(x.shape[2:])), *[a[1] for a in args], int(relu))
        return y

    @staticmethod
    def bn_backward(g, x, y, mean, invstd, gamma, relu=False, need_dx=True):
        g, gp = _f(g); x, xp = _f(x); y_, yp = _opt(y)
        n, ch = x.shape[:2]
        dx = np.empty_like(x) if need_dx else None
        dgb = np.empty((2, ch), np.float32)
        args = [_f(a) for a in (mean, invstd, gamma)]
        _l().orc_bn_backward(gp, xp, yp, dx.ctypes.data_as(C.c_void_p) if need_dx else None, n, ch, int(np.prod(x.shape[2:])),
                             *[a[1] for a in args], dgb.ctypes.data_as(C.c_void_p), int(relu))
        return dx, dgb[0].copy(), dgb[1].copy()

    @staticmethod
    def fold_bn(cw, cb, gamma, beta, rm, rv, eps):
        cw, cwp = _f(cw); cb_, cbp = _opt(cb)
        co = cw.shape[0]
        per = int(np.prod(cw.shape[1:]))
        fw = np.empty_like(cw); fb = np.empty((co,), np.float32)
        args = [_f(a) for a in (gamma, beta, rm, rv)]
        fn = _l().orc_fold_bn
        fn.argtypes = [C.c_void_p] * 6 + [C.c_float, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        fn(cwp, cbp, *[a[1] for a in args], eps, co, per, fw.ctypes.data_as(C.c_void_p), fb.ctypes.data_as(C.c_void_p))
        return fw, fb

    @staticmethod
    def pool2_fwd(x):
        x, xp = _f(x)
        n, ch, h, w = x.shape
        y = np.empty((n, ch, h // 2, w // 2), np.float32); idx = np.empty(y.shape, np.uint8)
        _l().orc_pool2_fwd(xp, y.ctypes.data_as(C.c_void_p), idx.ctypes.data_as(C.c_void_p), n * ch, h, w)
        return y, idx

    @staticmethod
    def pool2_bwd(g, idx, hw):
        g, gp = _f(g)
        idx = np.ascontiguousarray(idx, np.uint8)
        n, ch = g.shape[:2]
        gx = np.empty((n, ch, hw[0], hw[1]), np.float32)
        _l().orc_pool2_bwd(gp, idx.ctypes.data_as(C.c_void_p), gx.ctypes.data_as(C.c_void_p), n * ch, hw[0], hw[1])
        return gx

    @staticmethod
    def maxpool_fwd(x, k, s, p, d=1, ceil=False):
        x, xp = _f(x)
        n, ch, ih, iw = x.shape

        def osz(i):
            num = i + 2 * p - d * (k - 1) - 1 + (s - 1 if ceil else 0)
            o = num // s + 1
            if ceil and (o - 1) * s >= i + p:
                o -= 1
            return o
        oh, ow = osz(ih), osz(iw)
        y = np.empty((n, ch, oh, ow), np.float32); idx = np.empty(y.shape, np.int64)
        _l().orc_maxpool_fwd(xp, y.ctypes.data_as(C.c_void_p), idx.ctypes.data_as(C.c_void_p), n * ch, ih, iw, oh, ow, k, k, s, s, p, p, d, d)
        return y, idx

    @staticmethod
    def maxpool_bwd(g, idx, in_hw):
        g, gp = _f(g)
        idx = np.ascontiguousarray(idx, np.int64)
        n, ch, oh, ow = g.shape
        gx = np.empty((n, ch, in_hw[0], in_hw[1]), np.float32)
        _l().orc_maxpool_bwd(gp, idx.ctypes.data_as(C.c_void_p), gx.ctypes.data_as(C.c_void_p), n * ch, in_hw[0], in_hw[1], oh, ow)
        return gx

    @staticmethod
    def adapool_fwd(x, o):
        x, xp = _f(x)
        n, ch, ih, iw = x.shape
        y = np.empty((n, ch, o, o), np.float32)
        _l().orc_adapool_fwd(xp, y.ctypes.data_as(C.c_void_p), n * ch, ih, iw, o, o)
        return y

    @staticmethod
    def sgd(p, g, m, lr, mom=0.0, damp=0.0, wd=0.0, nesterov=False, first=False, maximize=False):
        """In place on float32 arrays p and m."""
        fn = _l().orc_sgd
        fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64] + [C.c_float] * 4 + [C.c_int] * 3
        g, gp = _f(g)
        fn(p.ctypes.data_as(C.c_void_p), gp, m.ctypes.data_as(C.c_void_p) if m is not None else None, p.size, lr, mom, damp, wd,
           int(nesterov), int(first), int(maximize))

    @staticmethod
    def adam(p, g, m, v, step, lr, b1=0.9, b2=0.999, eps=1e-8, wd=0.0, decoupled=False, maximize=False):
        fn = _l().orc_adam
        fn.argtypes = [C.c_void_p] * 4 + [C.c_int64] + [C.c_float] * 6 + [C.c_int] * 2
        g, gp = _f(g)
        fn(p.ctypes.data_as(C.c_void_p), gp, m.ctypes.data_as(C.c_void_p), v.ctypes.data_as(C.c_void_p), p.size, float(step), lr, b1, b2,
           eps, wd, int(decoupled), int(maximize))


# ---- the reference's own oracle: PyTorch CPU aten ------------------------------------------------------------------------

def aten_conv(x, w, bias, stride, pad, gy, groups=1, mask=(True, True, True)):
    """y, dx, dw, db exactly as tools/gemm_bench.py:26-38 obtains them (F.conv2d + aten.convolution_backward)."""
    import torch
    import torch.nn.functional as F
    y = F.conv2d(x, w, bias, stride=stride, padding=pad, groups=groups)
    dx, dw, db = torch.ops.aten.convolution_backward(gy, x, w, [w.shape[0]] if bias is not None else None, [stride, stride],
                                                     [pad, pad], [1, 1], False, [0, 0], groups, list(mask))
    return y, dx, dw, db
