"""ctypes front end of the CPU oracle (test infrastructure, not product code).

Loads ``libthnn_ref.so`` built from ``thnn_ref.c`` by the Makefile in this
folder and exposes each routine on numpy arrays.  ``Ref("ref64_")`` is the
fp64-accumulating oracle, ``Ref("ref32_")`` the fp32 port that the benchmark
times as its CPU baseline.  Only tests, the smoke check and the benchmark's
CPU legs may import this module.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libthnn_ref.so")


def build(force=False):
    """Compile the oracle library if it is missing or older than its source."""
    src = os.path.join(_HERE, "thnn_ref.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE])
    return _SO


_DTYPE = [np.float32]          # element type of the library prefix in use (set by Ref methods; the fp64 build is "refd_")


def _f(a):
    return np.ascontiguousarray(a, dtype=_DTYPE[0])


def _p(a):
    if a is None:
        return None
    return a.ctypes.data_as(ctypes.c_void_p)


def conv_out(size, k, d, pad):
    return (size + 2 * pad - k) // d + 1


class Ref:
    def __init__(self, prefix="ref64_"):
        build()
        self.lib = ctypes.CDLL(_SO)
        self.prefix = prefix
        self.dtype = np.float64 if prefix == "refd_" else np.float32
        self.creal = ctypes.c_double if prefix == "refd_" else ctypes.c_float
        self.index_base = self._fn("index_base", ctypes.c_int)()

    def __getattribute__(self, name):
        # looking up a routine selects this instance's element type for the array conversions of the call
        if not name.startswith("_"):
            d = object.__getattribute__(self, "__dict__").get("dtype")
            if d is not None:
                _DTYPE[0] = d
        return object.__getattribute__(self, name)

    def set_threads(self, n):
        """Fixes the OpenMP thread count of this library (both prefixes share one runtime); returns the count in use."""
        self._fn("set_threads")(int(n))
        return self._fn("max_threads", ctypes.c_int)()

    def _fn(self, name, restype=None):
        f = getattr(self.lib, self.prefix + name)
        f.restype = restype
        return f

    # -- depthwise ---------------------------------------------------------
    def dwconv_forward(self, x, w, b, dH, dW, padH, padW):
        x, w = _f(x), _f(w)
        b = None if b is None else _f(b)
        N, C, H, W = x.shape
        M, _, kH, kW = w.shape
        y = np.empty((N, C * M, conv_out(H, kH, dH, padH), conv_out(W, kW, dW, padW)), self.dtype)
        self._fn("dwconv_forward")(_p(x), _p(w), _p(b), _p(y), N, C, H, W, M, kH, kW, dH, dW, padH, padW)
        return y

    def dwconv_grad_input(self, gy, w, H, W, dH, dW, padH, padW):
        gy, w = _f(gy), _f(w)
        M, C, kH, kW = w.shape
        N = gy.shape[0]
        gx = np.empty((N, C, H, W), self.dtype)
        self._fn("dwconv_grad_input")(_p(gy), _p(w), _p(gx), N, C, H, W, M, kH, kW, dH, dW, padH, padW)
        return gx

    def dwconv_acc_grad(self, x, gy, gw, gb, dH, dW, padH, padW, scale):
        """Returns updated copies of gw [M,C,kH,kW] and gb [M,C] (or None)."""
        x, gy = _f(x), _f(gy)
        gw = _f(gw).copy()
        gb = None if gb is None else _f(gb).copy()
        N, C, H, W = x.shape
        M, _, kH, kW = gw.shape
        self._fn("dwconv_acc_grad")(_p(x), _p(gy), _p(gw), _p(gb), N, C, H, W, M, kH, kW, dH, dW, padH, padW,
                                    self.creal(scale))
        return gw, gb

    # -- im2col + GEMM convolution ----------------------------------------------
    def convmm_forward(self, x, w, b, dH, dW, padH, padW):
        x, w = _f(x), _f(w)
        b = None if b is None else _f(b)
        N, C, H, W = x.shape
        K, _, kH, kW = w.shape
        y = np.empty((N, K, conv_out(H, kH, dH, padH), conv_out(W, kW, dW, padW)), self.dtype)
        self._fn("convmm_forward")(_p(x), _p(w), _p(b), _p(y), N, C, H, W, K, kH, kW, dH, dW, padH, padW)
        return y

    def convmm_grad_input(self, gy, w, H, W, dH, dW, padH, padW):
        gy, w = _f(gy), _f(w)
        K, C, kH, kW = w.shape
        N = gy.shape[0]
        gx = np.empty((N, C, H, W), self.dtype)
        self._fn("convmm_grad_input")(_p(gy), _p(w), _p(gx), N, C, H, W, K, kH, kW, dH, dW, padH, padW)
        return gx

    def convmm_acc_grad(self, x, gy, gw, gb, dH, dW, padH, padW, scale):
        x, gy = _f(x), _f(gy)
        gw = _f(gw).copy()
        gb = None if gb is None else _f(gb).copy()
        N, C, H, W = x.shape
        K, _, kH, kW = gw.shape
        self._fn("convmm_acc_grad")(_p(x), _p(gy), _p(gw), _p(gb), N, C, H, W, K, kH, kW, dH, dW, padH, padW,
                                    self.creal(scale))
        return gw, gb

    # -- dilated convolution (SpatialDilatedConvolution; dilation 1 is SpatialConvolutionMM) -------
    def dilconv_forward(self, x, w, b, dH, dW, padH, padW, dilH, dilW):
        x, w = _f(x), _f(w)
        b = None if b is None else _f(b)
        N, C, H, W = x.shape
        K, _, kH, kW = w.shape
        oH = (H + 2 * padH - (dilH * (kH - 1) + 1)) // dH + 1
        oW = (W + 2 * padW - (dilW * (kW - 1) + 1)) // dW + 1
        y = np.empty((N, K, oH, oW), self.dtype)
        self._fn("dilconv_forward")(_p(x), _p(w), _p(b), _p(y), N, C, H, W, K, kH, kW, dH, dW, padH, padW, dilH, dilW)
        return y

    def dilconv_grad_input(self, gy, w, H, W, dH, dW, padH, padW, dilH, dilW):
        gy, w = _f(gy), _f(w)
        K, C, kH, kW = w.shape
        N = gy.shape[0]
        gx = np.empty((N, C, H, W), self.dtype)
        self._fn("dilconv_grad_input")(_p(gy), _p(w), _p(gx), N, C, H, W, K, kH, kW, dH, dW, padH, padW, dilH, dilW)
        return gx

    def dilconv_acc_grad(self, x, gy, gw, gb, dH, dW, padH, padW, dilH, dilW, scale):
        x, gy = _f(x), _f(gy)
        gw = _f(gw).copy()
        gb = None if gb is None else _f(gb).copy()
        N, C, H, W = x.shape
        K, _, kH, kW = gw.shape
        self._fn("dilconv_acc_grad")(_p(x), _p(gy), _p(gw), _p(gb), N, C, H, W, K, kH, kW, dH, dW, padH, padW,
                                     dilH, dilW, self.creal(scale))
        return gw, gb

    # -- transposed convolution (SpatialFullDilatedConvolution; weight [P, Q, kH, kW]) -------------
    @staticmethod
    def fullconv_out_size(H, W, kH, kW, dH, dW, padH, padW, dilH, dilW, adjH, adjW):
        return ((H - 1) * dH - 2 * padH + dilH * (kH - 1) + 1 + adjH,
                (W - 1) * dW - 2 * padW + dilW * (kW - 1) + 1 + adjW)

    def fullconv_forward(self, x, w, b, dH, dW, padH, padW, dilH=1, dilW=1, adjH=0, adjW=0):
        x, w = _f(x), _f(w)
        b = None if b is None else _f(b)
        N, P, H, W = x.shape
        _, Q, kH, kW = w.shape
        OH, OW = self.fullconv_out_size(H, W, kH, kW, dH, dW, padH, padW, dilH, dilW, adjH, adjW)
        y = np.empty((N, Q, OH, OW), self.dtype)
        self._fn("fullconv_forward")(_p(x), _p(w), _p(b), _p(y), N, P, H, W, Q, kH, kW, dH, dW, padH, padW,
                                     dilH, dilW, adjH, adjW)
        return y

    def fullconv_grad_input(self, gy, w, H, W, dH, dW, padH, padW, dilH=1, dilW=1, adjH=0, adjW=0):
        gy, w = _f(gy), _f(w)
        P, Q, kH, kW = w.shape
        N = gy.shape[0]
        gx = np.empty((N, P, H, W), self.dtype)
        self._fn("fullconv_grad_input")(_p(gy), _p(w), _p(gx), N, P, H, W, Q, kH, kW, dH, dW, padH, padW,
                                        dilH, dilW, adjH, adjW)
        return gx

    def fullconv_acc_grad(self, x, gy, gw, gb, dH, dW, padH, padW, dilH=1, dilW=1, adjH=0, adjW=0, scale=1.0):
        x, gy = _f(x), _f(gy)
        gw = _f(gw).copy()
        gb = None if gb is None else _f(gb).copy()
        N, P, H, W = x.shape
        _, Q, kH, kW = gw.shape
        self._fn("fullconv_acc_grad")(_p(x), _p(gy), _p(gw), _p(gb), N, P, H, W, Q, kH, kW, dH, dW, padH, padW,
                                      dilH, dilW, adjH, adjW, self.creal(scale))
        return gw, gb

    # -- batch norm --------------------------------------------------------------
    def bn_forward(self, x, weight, bias, running_mean, running_var, train, momentum, eps):
        """Returns y, running_mean', running_var', save_mean, save_std."""
        x = _f(x)
        N, C = x.shape[:2]
        S = int(np.prod(x.shape[2:])) if x.ndim > 2 else 1
        y = np.empty_like(x)
        rm, rv = _f(running_mean).copy(), _f(running_var).copy()
        sm, ss = np.zeros(C, self.dtype), np.zeros(C, self.dtype)
        weight = None if weight is None else _f(weight)
        bias = None if bias is None else _f(bias)
        self._fn("bn_forward")(_p(x), _p(y), _p(weight), _p(bias), _p(rm), _p(rv), _p(sm), _p(ss),
                               N, C, S, int(train), ctypes.c_double(momentum), ctypes.c_double(eps))
        return y, rm, rv, sm, ss

    def bn_backward(self, x, gy, weight, running_mean, running_var, save_mean, save_std, train, scale, eps,
                    gw=None, gb=None, want_gx=True):
        x, gy = _f(x), _f(gy)
        N, C = x.shape[:2]
        S = int(np.prod(x.shape[2:])) if x.ndim > 2 else 1
        gx = np.empty_like(x) if want_gx else None
        gw = None if gw is None else _f(gw).copy()
        gb = None if gb is None else _f(gb).copy()
        weight = None if weight is None else _f(weight)
        self._fn("bn_backward")(_p(x), _p(gy), _p(gx), _p(gw), _p(gb), _p(weight),
                                _p(_f(running_mean)), _p(_f(running_var)), _p(_f(save_mean)), _p(_f(save_std)),
                                N, C, S, int(train), ctypes.c_double(scale), ctypes.c_double(eps))
        return gx, gw, gb

    # -- max pooling ---------------------------------------------------------------
    def pool_out_size(self, size, k, d, pad, dil, ceil_mode):
        return self._fn("pool_out_size", ctypes.c_int)(size, k, d, pad, dil, int(ceil_mode))

    def maxpool_forward(self, x, kH, kW, dH, dW, padH, padW, ceil_mode, dilH=1, dilW=1):
        x = _f(x)
        N, C, H, W = x.shape
        oH = self.pool_out_size(H, kH, dH, padH, dilH, ceil_mode)
        oW = self.pool_out_size(W, kW, dW, padW, dilW, ceil_mode)
        y = np.empty((N, C, oH, oW), self.dtype)
        ind = np.empty((N, C, oH, oW), np.int64)
        self._fn("maxpool_forward")(_p(x), _p(y), _p(ind), N, C, H, W, oH, oW, kH, kW, dH, dW, padH, padW,
                                    dilH, dilW)
        return y, ind

    def maxpool_backward(self, gy, ind, H, W, kH, kW, dH, dW, padH, padW, dilH=1, dilW=1):
        gy = _f(gy)
        ind = np.ascontiguousarray(ind, dtype=np.int64)
        N, C, oH, oW = gy.shape
        gx = np.empty((N, C, H, W), self.dtype)
        self._fn("maxpool_backward")(_p(gy), _p(ind), _p(gx), N, C, H, W, oH, oW, kH, kW, dH, dW, padH, padW,
                                     dilH, dilW)
        return gx

    # -- support ops --------------------------------------------------------------
    def threshold_forward(self, x, th=0.0, val=0.0):
        x = _f(x)
        y = np.empty_like(x)
        self._fn("threshold_forward")(_p(x), _p(y), ctypes.c_size_t(x.size), self.creal(th), self.creal(val))
        return y

    def threshold_backward(self, x, gy, th=0.0):
        x, gy = _f(x), _f(gy)
        gx = np.empty_like(x)
        self._fn("threshold_backward")(_p(x), _p(gy), _p(gx), ctypes.c_size_t(x.size), self.creal(th))
        return gx

    def avgpool_forward(self, x, kH, kW, dH, dW, padH, padW, ceil_mode=False, count_include_pad=True):
        x = _f(x)
        N, C, H, W = x.shape
        oH = self.pool_out_size(H, kH, dH, padH, 1, ceil_mode)
        oW = self.pool_out_size(W, kW, dW, padW, 1, ceil_mode)
        y = np.empty((N, C, oH, oW), self.dtype)
        self._fn("avgpool_forward")(_p(x), _p(y), N, C, H, W, oH, oW, kH, kW, dH, dW, padH, padW,
                                    int(count_include_pad))
        return y

    def avgpool_backward(self, gy, H, W, kH, kW, dH, dW, padH, padW, count_include_pad=True):
        gy = _f(gy)
        N, C, oH, oW = gy.shape
        gx = np.empty((N, C, H, W), self.dtype)
        self._fn("avgpool_backward")(_p(gy), _p(gx), N, C, H, W, oH, oW, kH, kW, dH, dW, padH, padW,
                                     int(count_include_pad))
        return gx

    def logsoftmax_forward(self, x):
        x = _f(x)
        y = np.empty_like(x)
        self._fn("logsoftmax_forward")(_p(x), _p(y), x.shape[0], x.shape[1])
        return y

    def logsoftmax_backward(self, y, gy):
        y, gy = _f(y), _f(gy)
        gx = np.empty_like(y)
        self._fn("logsoftmax_backward")(_p(y), _p(gy), _p(gx), y.shape[0], y.shape[1])
        return gx

    def classnll_forward(self, lp, target, weights=None, size_average=True, ignore_index=-100):
        lp = _f(lp)
        target = np.ascontiguousarray(target, dtype=np.int64)
        weights = None if weights is None else _f(weights)
        loss, tw = self.creal(), self.creal()
        self._fn("classnll_forward")(_p(lp), _p(target), _p(weights), ctypes.byref(loss), ctypes.byref(tw),
                                     lp.shape[0], lp.shape[1], int(size_average), ctypes.c_int64(ignore_index))
        return loss.value, tw.value

    def classnll_backward(self, target, total_weight, B, D, weights=None, size_average=True, ignore_index=-100):
        target = np.ascontiguousarray(target, dtype=np.int64)
        weights = None if weights is None else _f(weights)
        gx = np.zeros((B, D), self.dtype)
        self._fn("classnll_backward")(_p(target), _p(weights), self.creal(total_weight), _p(gx), B, D,
                                      int(size_average), ctypes.c_int64(ignore_index))
        return gx

    # -- SpatialConvolutionLocal (weight [oH*oW, K, C*kH*kW], bias [K, oH, oW]) -----------------
    def localconv_forward(self, x, w, b, kH, kW, dH, dW, padH, padW):
        x, w = _f(x), _f(w)
        b = None if b is None else _f(b)
        N, C, H, W = x.shape
        K = w.shape[1]
        oH, oW = conv_out(H, kH, dH, padH), conv_out(W, kW, dW, padW)
        y = np.empty((N, K, oH, oW), self.dtype)
        self._fn("localconv_forward")(_p(x), _p(w), _p(b), _p(y), N, C, H, W, K, kH, kW, dH, dW, padH, padW, oH, oW)
        return y

    def localconv_grad_input(self, gy, w, C, H, W, kH, kW, dH, dW, padH, padW):
        gy, w = _f(gy), _f(w)
        N, K, oH, oW = gy.shape
        gx = np.empty((N, C, H, W), self.dtype)
        self._fn("localconv_grad_input")(_p(gy), _p(w), _p(gx), N, C, H, W, K, kH, kW, dH, dW, padH, padW, oH, oW)
        return gx

    def localconv_acc_grad(self, x, gy, gw, gb, kH, kW, dH, dW, padH, padW, scale):
        x, gy = _f(x), _f(gy)
        gw = _f(gw).copy()
        gb = None if gb is None else _f(gb).copy()
        N, C, H, W = x.shape
        _, K, oH, oW = gy.shape
        self._fn("localconv_acc_grad")(_p(x), _p(gy), _p(gw), _p(gb), N, C, H, W, K, kH, kW, dH, dW, padH, padW, oH, oW,
                                       self.creal(scale))
        return gw, gb

    # -- adaptive pooling ------------------------------------------------------------------------
    def adaptive_maxpool_forward(self, x, oH, oW):
        """Returns y [N, C, oH, oW] and indices [2, N, C, oH, oW] (row, column offsets inside the window + base)."""
        x = _f(x)
        N, C, H, W = x.shape
        y = np.empty((N, C, oH, oW), self.dtype)
        ind = np.empty((2, N, C, oH, oW), np.int64)
        self._fn("adaptive_maxpool_forward")(_p(x), _p(y), _p(ind), N * C, H, W, oH, oW)
        return y, ind

    def adaptive_maxpool_backward(self, gy, ind, H, W):
        gy = _f(gy)
        ind = np.ascontiguousarray(ind, dtype=np.int64)
        N, C, oH, oW = gy.shape
        gx = np.empty((N, C, H, W), self.dtype)
        self._fn("adaptive_maxpool_backward")(_p(gy), _p(ind), _p(gx), N * C, H, W, oH, oW)
        return gx

    def adaptive_avgpool_forward(self, x, oH, oW):
        x = _f(x)
        N, C, H, W = x.shape
        y = np.empty((N, C, oH, oW), self.dtype)
        self._fn("adaptive_avgpool_forward")(_p(x), _p(y), N * C, H, W, oH, oW)
        return y

    def adaptive_avgpool_backward(self, gy, H, W):
        gy = _f(gy)
        N, C, oH, oW = gy.shape
        gx = np.empty((N, C, H, W), self.dtype)
        self._fn("adaptive_avgpool_backward")(_p(gy), _p(gx), N * C, H, W, oH, oW)
        return gx

    def slice_range(self, n, g, i):
        s, c = ctypes.c_long(), ctypes.c_long()
        self._fn("slice_range")(ctypes.c_long(n), g, i, ctypes.byref(s), ctypes.byref(c))
        return s.value, c.value
