"""ctypes front end of oracle/_ref: the reference's own device kernels (test infrastructure).

``make -C oracle ref`` compiles the kernel templates of the reference's
``lib/THCUNN/SpatialDilatedMaxPooling.cu``, ``SpatialAveragePooling.cu``,
``BatchNormalization.cu`` and ``im2col.h`` from where they lie in the reference tree
(behind the stand-in headers of ``oracle/ref_shim``) into

* ``_ref/librefk_cpu.so`` — the pooling kernels as host loops (``RefKernelsCPU``, numpy arrays);
* ``_ref/librefk_gpu.so`` — all of them for the GPU, the convolution ones inside the reference's
  per-image unfold + cuBLAS schedule (``RefKernelsGPU``, torch CUDA tensors).

The libraries are built where the reference tree exists and travel as built files; where they are
missing ``available_cpu()`` / ``available_gpu()`` say so and the tests that need them skip.
Only tests and the benchmark's reference legs import this module.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_CPU_SO = os.path.join(_HERE, "_ref", "librefk_cpu.so")
_GPU_SO = os.path.join(_HERE, "_ref", "librefk_gpu.so")
REFERENCE = os.environ.get("CUNN_REFERENCE_TREE", "/root/reference")


def build():
    """Compile oracle/_ref when the reference tree is present; a no-op elsewhere."""
    if os.path.isdir(os.path.join(REFERENCE, "lib", "THCUNN")):
        subprocess.check_call(["make", "-s", "-C", _HERE, "ref", "REFERENCE=" + REFERENCE])
    return available_cpu(), available_gpu()


def available_cpu():
    return os.path.exists(_CPU_SO)


def available_gpu():
    return os.path.exists(_GPU_SO)


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class RefKernelsCPU:
    """The reference's pooling kernels executed on the host, one loop iteration per CUDA thread."""

    def __init__(self):
        self.lib = ctypes.CDLL(_CPU_SO)
        self.index_base = self.lib.refk_cpu_index_base()

    def maxpool_forward(self, x, oH, oW, kH, kW, dH, dW, padH, padW, dilH=1, dilW=1):
        x = _f(x)
        N, C, H, W = x.shape
        y = np.empty((N, C, oH, oW), np.float32)
        ind = np.empty((N, C, oH, oW), np.int64)
        self.lib.refk_cpu_maxpool_forward(_p(x), _p(y), _p(ind), N, C, H, W, oH, oW, kH, kW, dH, dW, padH, padW, dilH, dilW)
        return y, ind

    def maxpool_backward(self, gy, ind, H, W, kH, kW, dH, dW, padH, padW, dilH=1, dilW=1):
        gy = _f(gy)
        ind = np.ascontiguousarray(ind, dtype=np.int64)
        N, C, oH, oW = gy.shape
        gx = np.empty((N, C, H, W), np.float32)
        self.lib.refk_cpu_maxpool_backward(_p(gy), _p(ind), _p(gx), N, C, H, W, oH, oW, kH, kW, dH, dW, padH, padW, dilH, dilW)
        return gx

    def avgpool_forward(self, x, oH, oW, kH, kW, dH, dW, padH, padW, count_include_pad=True):
        x = _f(x)
        N, C, H, W = x.shape
        y = np.empty((N, C, oH, oW), np.float32)
        self.lib.refk_cpu_avgpool_forward(_p(x), _p(y), N, C, H, W, oH, oW, kH, kW, dH, dW, padH, padW, int(count_include_pad))
        return y

    def avgpool_backward(self, gy, H, W, kH, kW, dH, dW, padH, padW, count_include_pad=True):
        gy = _f(gy)
        N, C, oH, oW = gy.shape
        gx = np.empty((N, C, H, W), np.float32)
        self.lib.refk_cpu_avgpool_backward(_p(gy), _p(gx), N, C, H, W, oH, oW, kH, kW, dH, dW, padH, padW, int(count_include_pad))
        return gx


    def adaptive_maxpool_forward(self, x, oH, oW):
        x = _f(x)
        N, C, H, W = x.shape
        y = np.empty((N, C, oH, oW), np.float32)
        ind = np.empty((2, N, C, oH, oW), np.int64)
        self.lib.refk_cpu_adaptive_maxpool_forward(_p(x), _p(y), _p(ind), N * C, H, W, oH, oW)
        return y, ind

    def adaptive_maxpool_backward(self, gy, ind, H, W):
        gy = _f(gy)
        ind = np.ascontiguousarray(ind, dtype=np.int64)
        N, C, oH, oW = gy.shape
        gx = np.zeros((N, C, H, W), np.float32)                       # the reference's wrapper zeroes gradInput first
        self.lib.refk_cpu_adaptive_maxpool_backward(_p(gx), _p(gy), _p(ind), N * C, H, W, oH, oW)
        return gx

    def adaptive_avgpool_forward(self, x, oH, oW):
        x = _f(x)
        N, C, H, W = x.shape
        y = np.empty((N, C, oH, oW), np.float32)
        self.lib.refk_cpu_adaptive_avgpool_forward(_p(x), _p(y), N * C, H, W, oH, oW)
        return y

    def adaptive_avgpool_backward(self, gy, H, W):
        gy = _f(gy)
        N, C, oH, oW = gy.shape
        gx = np.zeros((N, C, H, W), np.float32)
        self.lib.refk_cpu_adaptive_avgpool_backward(_p(gx), _p(gy), N * C, H, W, oH, oW)
        return gx


def _out(size, k, d, pad, dil=1):
    return (size + 2 * pad - (dil * (k - 1) + 1)) // d + 1


class RefKernelsGPU:
    """The reference's kernels on the current CUDA device.  Arguments and results are contiguous
    fp32 (int64 for indices) torch CUDA tensors; every call runs on the legacy default stream and
    synchronises before it returns."""

    def __init__(self):
        import torch
        self.torch = torch
        self.lib = ctypes.CDLL(_GPU_SO)
        self.lib.refk_conv_scratch_bytes.restype = ctypes.c_size_t
        self.lib.refk_dwconv_scratch_bytes.restype = ctypes.c_size_t
        self.index_base = self.lib.refk_index_base()

    @staticmethod
    def _d(t):
        return None if t is None else ctypes.c_void_p(t.data_ptr())

    def _sync(self):
        self.torch.cuda.synchronize()

    def _new(self, shape, dtype=None):
        return self.torch.empty(shape, device="cuda", dtype=dtype or self.torch.float32)

    # pooling -------------------------------------------------------------------------------
    def maxpool_forward(self, x, oH, oW, kH, kW, dH, dW, padH, padW, dilH=1, dilW=1):
        N, C, H, W = x.shape
        y, ind = self._new((N, C, oH, oW)), self._new((N, C, oH, oW), self.torch.int64)
        self._sync()
        self.lib.refk_maxpool_forward(self._d(x), self._d(y), self._d(ind), N, C, H, W, oH, oW, kH, kW, dH, dW, padH, padW, dilH, dilW)
        self._sync()
        return y, ind

    def maxpool_backward(self, gy, ind, H, W, kH, kW, dH, dW, padH, padW, dilH=1, dilW=1):
        N, C, oH, oW = gy.shape
        gx = self._new((N, C, H, W))
        self._sync()
        self.lib.refk_maxpool_backward(self._d(gy), self._d(ind), self._d(gx), N, C, H, W, oH, oW, kH, kW, dH, dW, padH, padW, dilH, dilW)
        self._sync()
        return gx

    def avgpool_forward(self, x, oH, oW, kH, kW, dH, dW, padH, padW, count_include_pad=True):
        N, C, H, W = x.shape
        y = self._new((N, C, oH, oW))
        self._sync()
        self.lib.refk_avgpool_forward(self._d(x), self._d(y), N, C, H, W, oH, oW, kH, kW, dH, dW, padH, padW, int(count_include_pad))
        self._sync()
        return y

    def avgpool_backward(self, gy, H, W, kH, kW, dH, dW, padH, padW, count_include_pad=True):
        N, C, oH, oW = gy.shape
        gx = self._new((N, C, H, W))
        self._sync()
        self.lib.refk_avgpool_backward(self._d(gy), self._d(gx), N, C, H, W, oH, oW, kH, kW, dH, dW, padH, padW, int(count_include_pad))
        self._sync()
        return gx

    # batch norm ----------------------------------------------------------------------------
    def bn_forward(self, x, weight, bias, running_mean, running_var, train, momentum, eps):
        """Returns y, running_mean', running_var', save_mean, save_std (running stats are copies)."""
        N, C = x.shape[:2]
        S = x.numel() // max(N * C, 1)
        y = self.torch.empty_like(x)
        rm, rv = running_mean.clone(), running_var.clone()
        sm, ss = self._new((C,)).zero_(), self._new((C,)).zero_()
        self._sync()
        self.lib.refk_bn_forward(self._d(x), self._d(y), self._d(weight), self._d(bias), self._d(rm), self._d(rv),
                                 self._d(sm), self._d(ss), N, C, S, int(train), ctypes.c_double(momentum), ctypes.c_double(eps))
        self._sync()
        return y, rm, rv, sm, ss

    def bn_backward(self, x, gy, weight, running_mean, running_var, save_mean, save_std, train, scale, eps,
                    gw=None, gb=None, want_gx=True):
        N, C = x.shape[:2]
        S = x.numel() // max(N * C, 1)
        gx = self.torch.empty_like(x) if want_gx else None
        gw = None if gw is None else gw.clone()
        gb = None if gb is None else gb.clone()
        self._sync()
        self.lib.refk_bn_backward(self._d(x), self._d(gy), self._d(gx), self._d(gw), self._d(gb), self._d(weight),
                                  self._d(running_mean), self._d(running_var), self._d(save_mean), self._d(save_std),
                                  N, C, S, int(train), ctypes.c_double(scale), ctypes.c_double(eps))
        self._sync()
        return gx, gw, gb

    # unfold / fold -------------------------------------------------------------------------
    def im2col(self, x, kH, kW, padH, padW, dH, dW, dilH=1, dilW=1):
        C, H, W = x.shape
        oH, oW = _out(H, kH, dH, padH, dilH), _out(W, kW, dW, padW, dilW)
        col = self._new((C * kH * kW, oH * oW))
        self._sync()
        self.lib.refk_im2col(self._d(x), C, H, W, kH, kW, padH, padW, dH, dW, dilH, dilW, self._d(col))
        self._sync()
        return col

    def col2im(self, col, C, H, W, kH, kW, padH, padW, dH, dW, dilH=1, dilW=1):
        x = self._new((C, H, W))
        self._sync()
        self.lib.refk_col2im(self._d(col), C, H, W, kH, kW, padH, padW, dH, dW, dilH, dilW, self._d(x))
        self._sync()
        return x

    # convolutions in the reference's schedule -------------------------------------------------
    def _conv_scratch(self, C, H, W, kH, kW, dH, dW, padH, padW):
        n = self.lib.refk_conv_scratch_bytes(C, H, W, kH, kW, dH, dW, padH, padW)
        return self._new((n // 4 + 1,))

    def convmm_forward(self, x, w, b, dH, dW, padH, padW):
        N, C, H, W = x.shape
        K, kH, kW = w.shape[0], w.shape[-2], w.shape[-1]
        y = self._new((N, K, _out(H, kH, dH, padH), _out(W, kW, dW, padW)))
        s = self._conv_scratch(C, H, W, kH, kW, dH, dW, padH, padW)
        self._sync()
        self.lib.refk_convmm_forward(self._d(x), self._d(w), self._d(b), self._d(y), N, C, H, W, K, kH, kW, dH, dW, padH, padW, self._d(s))
        self._sync()
        return y

    def convmm_grad_input(self, gy, w, H, W, dH, dW, padH, padW):
        N = gy.shape[0]
        K, C, kH, kW = w.shape
        gx = self._new((N, C, H, W))
        s = self._conv_scratch(C, H, W, kH, kW, dH, dW, padH, padW)
        self._sync()
        self.lib.refk_convmm_grad_input(self._d(gy), self._d(w), self._d(gx), N, C, H, W, K, kH, kW, dH, dW, padH, padW, self._d(s))
        self._sync()
        return gx

    def convmm_acc_grad(self, x, gy, gw, gb, dH, dW, padH, padW, scale):
        N, C, H, W = x.shape
        K, _, kH, kW = gw.shape
        gw = gw.clone()
        gb = None if gb is None else gb.clone()
        s = self._conv_scratch(C, H, W, kH, kW, dH, dW, padH, padW)
        self._sync()
        self.lib.refk_convmm_acc_grad(self._d(x), self._d(gy), self._d(gw), self._d(gb), N, C, H, W, K, kH, kW, dH, dW, padH, padW,
                                      ctypes.c_float(scale), self._d(s))
        self._sync()
        return gw, gb

    def _dw_scratch(self, C, H, W, M, kH, kW, dH, dW, padH, padW):
        n = self.lib.refk_dwconv_scratch_bytes(C, H, W, M, kH, kW, dH, dW, padH, padW)
        return self._new((n // 4 + 1,))

    def dwconv_forward(self, x, w, b, dH, dW, padH, padW):
        N, C, H, W = x.shape
        M, _, kH, kW = w.shape
        y = self._new((N, C * M, _out(H, kH, dH, padH), _out(W, kW, dW, padW)))
        s = self._dw_scratch(C, H, W, M, kH, kW, dH, dW, padH, padW)
        self._sync()
        self.lib.refk_dwconv_forward(self._d(x), self._d(w), self._d(b), self._d(y), N, C, H, W, M, kH, kW, dH, dW, padH, padW, self._d(s))
        self._sync()
        return y

    def dwconv_grad_input(self, gy, w, H, W, dH, dW, padH, padW):
        N = gy.shape[0]
        M, C, kH, kW = w.shape
        gx = self._new((N, C, H, W))
        s = self._dw_scratch(C, H, W, M, kH, kW, dH, dW, padH, padW)
        self._sync()
        self.lib.refk_dwconv_grad_input(self._d(gy), self._d(w), self._d(gx), N, C, H, W, M, kH, kW, dH, dW, padH, padW, self._d(s))
        self._sync()
        return gx

    def dwconv_acc_grad(self, x, gy, gw, gb, dH, dW, padH, padW, scale):
        N, C, H, W = x.shape
        M, _, kH, kW = gw.shape
        gw = gw.clone()
        gb = None if gb is None else gb.clone()
        s = self._dw_scratch(C, H, W, M, kH, kW, dH, dW, padH, padW)
        self._sync()
        self.lib.refk_dwconv_acc_grad(self._d(x), self._d(gy), self._d(gw), self._d(gb), N, C, H, W, M, kH, kW, dH, dW, padH, padW,
                                      ctypes.c_float(scale), self._d(s))
        self._sync()
        return gw, gb
