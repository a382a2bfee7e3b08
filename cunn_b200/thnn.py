"""Drives the THNN_Cuda* entry points of libTHCUNN.so the way the reference's FFI binding does
(THCUNN.lua:129-138): the state comes first, tensors are THCudaTensor structs, outputs are resized by the
callee, errors arrive through the state's error hook.  torch CUDA tensors provide the device memory.

    nnb = THNN()                       # one state (stream = torch's current stream at call time)
    y = nnb.SpatialDepthWiseConvolution_updateOutput(x, weight, bias, kW, kH, dW, dH, padW, padH)

Inputs may be non-contiguous (their strides are passed through); outputs come back as torch tensors of
the shape the callee chose.
"""
import ctypes

import torch

from ._lib import lib, CunnError

c_long, c_int, c_void_p, c_float, c_double, c_bool = (ctypes.c_long, ctypes.c_int, ctypes.c_void_p, ctypes.c_float,
                                                      ctypes.c_double, ctypes.c_bool)


class THCudaStorage(ctypes.Structure):
    _fields_ = [("data", c_void_p), ("size", ctypes.c_ssize_t), ("refcount", c_int), ("flag", ctypes.c_char),
                ("allocator", c_void_p), ("allocatorContext", c_void_p), ("view", c_void_p), ("device", c_int)]


class THCudaTensor(ctypes.Structure):
    _fields_ = [("size", ctypes.POINTER(c_long)), ("stride", ctypes.POINTER(c_long)), ("nDimension", c_int),
                ("storage", ctypes.POINTER(THCudaStorage)), ("storageOffset", ctypes.c_ssize_t), ("refcount", c_int),
                ("flag", ctypes.c_char)]


_TP = ctypes.POINTER(THCudaTensor)
_ERRFN = ctypes.CFUNCTYPE(None, ctypes.c_char_p, c_void_p)

lib.THCState_b200_new.restype = c_void_p
lib.THCState_b200_free.argtypes = [c_void_p]
lib.THCState_b200_setStream.argtypes = [c_void_p, c_void_p]
lib.THCState_b200_setErrorHandler.argtypes = [c_void_p, _ERRFN, c_void_p]
lib.THCudaTensor_b200_wrap.restype = _TP
lib.THCudaTensor_b200_wrap.argtypes = [c_void_p, c_void_p, ctypes.c_ssize_t, c_int, ctypes.POINTER(c_long),
                                       ctypes.POINTER(c_long), c_int, ctypes.c_ssize_t]
lib.THCudaTensor_b200_data.restype = c_void_p
lib.THCudaTensor_b200_data.argtypes = [c_void_p, _TP, c_int]
lib.THCudaTensor_b200_new.restype = _TP
lib.THCudaTensor_b200_new.argtypes = [c_void_p]
lib.THCudaTensor_b200_free.argtypes = [c_void_p, _TP]

_T, _I, _F, _D, _B, _L = _TP, c_int, c_float, c_double, c_bool, c_long
_CONV = [_I] * 6
_SIGS = {
    "SpatialDepthWiseConvolution_updateOutput": [_T] * 6 + _CONV,
    "SpatialDepthWiseConvolution_updateGradInput": [_T] * 6 + _CONV,
    "SpatialDepthWiseConvolution_accGradParameters": [_T] * 6 + _CONV + [_F],
    "SpatialConvolutionMM_updateOutput": [_T] * 6 + _CONV,
    "SpatialConvolutionMM_updateGradInput": [_T] * 6 + _CONV,
    "SpatialConvolutionMM_accGradParameters": [_T] * 6 + _CONV + [_F],
    "SpatialDilatedConvolution_updateOutput": [_T] * 6 + _CONV + [ctypes.c_int, ctypes.c_int],
    "SpatialDilatedConvolution_updateGradInput": [_T] * 5 + _CONV + [ctypes.c_int, ctypes.c_int],
    "SpatialDilatedConvolution_accGradParameters": [_T] * 6 + _CONV + [ctypes.c_int, ctypes.c_int, _F],
    "SpatialFullDilatedConvolution_updateOutput": [_T] * 6 + _CONV + [_I] * 4,
    "SpatialFullDilatedConvolution_updateGradInput": [_T] * 5 + _CONV + [_I] * 4,
    "SpatialFullDilatedConvolution_accGradParameters": [_T] * 6 + _CONV + [_I] * 4 + [_F],
    "SpatialFullConvolution_updateOutput": [_T] * 6 + _CONV + [_I] * 2,
    "SpatialFullConvolution_updateGradInput": [_T] * 5 + _CONV + [_I] * 2,
    "SpatialFullConvolution_accGradParameters": [_T] * 6 + _CONV + [_I] * 2 + [_F],
    "BatchNormalization_updateOutput": [_T] * 8 + [_B, _D, _D],
    "BatchNormalization_backward": [_T] * 10 + [_B, _D, _D],
    "SpatialMaxPooling_updateOutput": [_T] * 3 + _CONV + [_B],
    "SpatialMaxPooling_updateGradInput": [_T] * 4 + _CONV + [_B],
    "SpatialConvolutionLocal_updateOutput": [_T] * 6 + _CONV + [_L] * 4,
    "SpatialConvolutionLocal_updateGradInput": [_T] * 6 + _CONV + [_L] * 4,
    "SpatialConvolutionLocal_accGradParameters": [_T] * 6 + _CONV + [_L] * 4 + [_F],
    "SpatialAdaptiveMaxPooling_updateOutput": [_T, _T, _T, _I, _I],
    "SpatialAdaptiveMaxPooling_updateGradInput": [_T] * 4,
    "SpatialAdaptiveAveragePooling_updateOutput": [_T, _T, _I, _I],
    "SpatialAdaptiveAveragePooling_updateGradInput": [_T] * 3,
    "Threshold_updateOutput": [_T, _T, _F, _F, _B],
    "Threshold_updateGradInput": [_T, _T, _T, _F, _F, _B],
    "SpatialAveragePooling_updateOutput": [_T, _T] + _CONV + [_B, _B],
    "SpatialAveragePooling_updateGradInput": [_T, _T, _T] + _CONV + [_B, _B],
    "LogSoftMax_updateOutput": [_T, _T],
    "LogSoftMax_updateGradInput": [_T] * 4,
    "ClassNLLCriterion_updateOutput": [_T, _T, _T, _B, _T, _T, _L],
    "ClassNLLCriterion_updateGradInput": [_T, _T, _T, _B, _T, _T, _L],
}
for _name, _args in _SIGS.items():
    _f = getattr(lib, "THNN_Cuda" + _name)
    _f.restype = None
    _f.argtypes = [c_void_p] + _args

# the hot path also exists for double tensors (THNN_CudaDouble*): accreal, i.e. `scale`, is a double there
DOUBLE_ENTRY_POINTS = [n for n in _SIGS if n.split("_")[0] in ("SpatialDepthWiseConvolution", "SpatialConvolutionMM",
                                                                "BatchNormalization", "SpatialMaxPooling")]
for _name in DOUBLE_ENTRY_POINTS:
    _f = getattr(lib, "THNN_CudaDouble" + _name)
    _f.restype = None
    _f.argtypes = [c_void_p] + [c_double if a is _F else a for a in _SIGS[_name]]


class THNNError(CunnError):
    """An argument or launch error reported through the state's error hook (TH's THError)."""


class THNN:
    """Drives the THNN_Cuda* entry points (dtype=torch.float32) or the THNN_CudaDouble* ones (torch.float64)
    the way the LuaJIT binding does: a state first, tensor structs, outputs resized by the callee."""

    def __init__(self, dtype=torch.float32):
        self.real = dtype
        self.prefix = "THNN_CudaDouble" if dtype == torch.float64 else "THNN_Cuda"
        self.state = lib.THCState_b200_new()
        self.errors = []
        self._hook = _ERRFN(lambda msg, ctx: self.errors.append(msg.decode()))
        lib.THCState_b200_setErrorHandler(self.state, self._hook, None)
        self._keep = []

    def close(self):
        if self.state:
            lib.THCState_b200_free(self.state)
            self.state = None

    # -- tensor plumbing ------------------------------------------------------------------------------
    def wrap(self, t):
        """THCudaTensor over a torch tensor's memory, with its sizes and strides (None stays NULL)."""
        if t is None:
            return None
        nd = t.dim()
        sizes = (c_long * max(nd, 1))(*t.shape)
        strides = (c_long * max(nd, 1))(*t.stride())
        # the storage starts at the torch storage's base; a view keeps its offset, as a Lua tensor would
        st = t.untyped_storage()
        cap = st.nbytes() // t.element_size()
        h = lib.THCudaTensor_b200_wrap(self.state, st.data_ptr(), cap, nd, sizes, strides, t.element_size(),
                                       t.storage_offset())
        self._keep.append(t)
        return h

    def out(self, capacity, dtype=None, device="cuda"):
        """An output tensor with no shape yet over `capacity` elements of torch memory: the callee resizes it."""
        dtype = dtype or self.real
        buf = torch.empty(max(int(capacity), 1), dtype=dtype, device=device)
        sizes = (c_long * 1)(0)
        h = lib.THCudaTensor_b200_wrap(self.state, buf.data_ptr(), buf.numel(), 0, sizes, None, buf.element_size(), 0)
        return h, buf

    @staticmethod
    def shape_of(h):
        t = h.contents
        return tuple(int(t.size[i]) for i in range(t.nDimension))

    def view(self, h, buf):
        shape = self.shape_of(h)
        n = 1
        for s in shape:
            n *= s
        return buf[:n].view(shape) if shape else buf[:0]

    def call(self, name, *args):
        lib.THCState_b200_setStream(self.state, torch.cuda.current_stream().cuda_stream)
        n0 = len(self.errors)
        getattr(lib, self.prefix + name)(self.state, *args)
        if len(self.errors) > n0:
            raise THNNError(self.errors[-1])

    def free(self, *handles):
        for h in handles:
            if h:
                lib.THCudaTensor_b200_free(self.state, h)
        self._keep.clear()

    # -- the hot path, one method per reference entry point ------------------------------------------
    def _conv_out(self, x, k_out, kW, kH, dW, dH, padW, padH):
        H, W = x.shape[-2:]
        oH = max((H + 2 * padH - kH) // max(dH, 1) + 1, 1)
        oW = max((W + 2 * padW - kW) // max(dW, 1) + 1, 1)
        n = x.shape[0] if x.dim() == 4 else 1
        return n * k_out * oH * oW

    def SpatialDepthWiseConvolution_updateOutput(self, x, weight, bias, kW, kH, dW, dH, padW, padH):
        cap = self._conv_out(x, weight.shape[0] * (weight.shape[1] if weight.dim() == 4 else weight.shape[1] // (kH * kW)),
                             kW, kH, dW, dH, padW, padH)
        hx, hw, hb = self.wrap(x), self.wrap(weight), self.wrap(bias)
        ho, buf = self.out(cap)
        try:
            self.call("SpatialDepthWiseConvolution_updateOutput", hx, ho, hw, hb, None, None, kW, kH, dW, dH, padW, padH)
            return self.view(ho, buf)
        finally:
            self.free(hx, hw, hb, ho)

    def SpatialDepthWiseConvolution_updateGradInput(self, x, gy, weight, kW, kH, dW, dH, padW, padH):
        hx, hg, hw = self.wrap(x), self.wrap(gy), self.wrap(weight)
        ho, buf = self.out(x.numel())
        try:
            self.call("SpatialDepthWiseConvolution_updateGradInput", hx, hg, ho, hw, None, None, kW, kH, dW, dH, padW, padH)
            return self.view(ho, buf)
        finally:
            self.free(hx, hg, hw, ho)

    def SpatialDepthWiseConvolution_accGradParameters(self, x, gy, gw, gb, kW, kH, dW, dH, padW, padH, scale):
        hx, hg, hw, hb = self.wrap(x), self.wrap(gy), self.wrap(gw), self.wrap(gb)
        try:
            self.call("SpatialDepthWiseConvolution_accGradParameters", hx, hg, hw, hb, None, None, kW, kH, dW, dH, padW, padH, scale)
        finally:
            self.free(hx, hg, hw, hb)

    def SpatialConvolutionMM_updateOutput(self, x, weight, bias, kW, kH, dW, dH, padW, padH):
        cap = self._conv_out(x, weight.shape[0], kW, kH, dW, dH, padW, padH)
        hx, hw, hb = self.wrap(x), self.wrap(weight), self.wrap(bias)
        ho, buf = self.out(cap)
        try:
            self.call("SpatialConvolutionMM_updateOutput", hx, ho, hw, hb, None, None, kW, kH, dW, dH, padW, padH)
            return self.view(ho, buf)
        finally:
            self.free(hx, hw, hb, ho)

    def SpatialConvolutionMM_updateGradInput(self, x, gy, weight, kW, kH, dW, dH, padW, padH):
        hx, hg, hw = self.wrap(x), self.wrap(gy), self.wrap(weight)
        ho, buf = self.out(x.numel())
        try:
            self.call("SpatialConvolutionMM_updateGradInput", hx, hg, ho, hw, None, None, kW, kH, dW, dH, padW, padH)
            return self.view(ho, buf)
        finally:
            self.free(hx, hg, hw, ho)

    def SpatialConvolutionMM_accGradParameters(self, x, gy, gw, gb, kW, kH, dW, dH, padW, padH, scale):
        hx, hg, hw, hb = self.wrap(x), self.wrap(gy), self.wrap(gw), self.wrap(gb)
        try:
            self.call("SpatialConvolutionMM_accGradParameters", hx, hg, hw, hb, None, None, kW, kH, dW, dH, padW, padH, scale)
        finally:
            self.free(hx, hg, hw, hb)

    def SpatialDilatedConvolution_updateOutput(self, x, weight, bias, kW, kH, dW, dH, padW, padH, dilW, dilH):
        b = x.dim() == 4
        H, W = x.shape[b + 1], x.shape[b + 2]
        oH = (H + 2 * padH - (dilH * (kH - 1) + 1)) // dH + 1
        oW = (W + 2 * padW - (dilW * (kW - 1) + 1)) // dW + 1
        cap = max(1, (x.shape[0] if b else 1) * weight.shape[0] * max(oH, 1) * max(oW, 1))
        hx, hw, hb = self.wrap(x), self.wrap(weight), self.wrap(bias)
        ho, buf = self.out(cap)
        try:
            self.call("SpatialDilatedConvolution_updateOutput", hx, ho, hw, hb, None, None, kW, kH, dW, dH, padW, padH, dilW, dilH)
            return self.view(ho, buf)
        finally:
            self.free(hx, hw, hb, ho)

    def SpatialDilatedConvolution_updateGradInput(self, x, gy, weight, kW, kH, dW, dH, padW, padH, dilW, dilH):
        hx, hg, hw = self.wrap(x), self.wrap(gy), self.wrap(weight)
        ho, buf = self.out(x.numel())
        try:
            self.call("SpatialDilatedConvolution_updateGradInput", hx, hg, ho, hw, None, kW, kH, dW, dH, padW, padH, dilW, dilH)
            return self.view(ho, buf)
        finally:
            self.free(hx, hg, hw, ho)

    def SpatialDilatedConvolution_accGradParameters(self, x, gy, gw, gb, kW, kH, dW, dH, padW, padH, dilW, dilH, scale):
        hx, hg, hw, hb = self.wrap(x), self.wrap(gy), self.wrap(gw), self.wrap(gb)
        try:
            self.call("SpatialDilatedConvolution_accGradParameters", hx, hg, hw, hb, None, None, kW, kH, dW, dH, padW, padH,
                      dilW, dilH, scale)
        finally:
            self.free(hx, hg, hw, hb)

    def SpatialFullDilatedConvolution_updateOutput(self, x, weight, bias, kW, kH, dW, dH, padW, padH, dilW, dilH, adjW, adjH):
        b = x.dim() == 4
        H, W = x.shape[b + 1], x.shape[b + 2]
        OH = (H - 1) * dH - 2 * padH + dilH * (kH - 1) + 1 + adjH
        OW = (W - 1) * dW - 2 * padW + dilW * (kW - 1) + 1 + adjW
        cap = max(1, (x.shape[0] if b else 1) * weight.shape[1] * max(OH, 1) * max(OW, 1))
        hx, hw, hb = self.wrap(x), self.wrap(weight), self.wrap(bias)
        ho, buf = self.out(cap)
        try:
            self.call("SpatialFullDilatedConvolution_updateOutput", hx, ho, hw, hb, None, None, kW, kH, dW, dH, padW, padH,
                      dilW, dilH, adjW, adjH)
            return self.view(ho, buf)
        finally:
            self.free(hx, hw, hb, ho)

    def SpatialFullDilatedConvolution_updateGradInput(self, x, gy, weight, kW, kH, dW, dH, padW, padH, dilW, dilH, adjW, adjH):
        hx, hg, hw = self.wrap(x), self.wrap(gy), self.wrap(weight)
        ho, buf = self.out(x.numel())
        try:
            self.call("SpatialFullDilatedConvolution_updateGradInput", hx, hg, ho, hw, None, kW, kH, dW, dH, padW, padH,
                      dilW, dilH, adjW, adjH)
            return self.view(ho, buf)
        finally:
            self.free(hx, hg, hw, ho)

    def SpatialFullDilatedConvolution_accGradParameters(self, x, gy, gw, gb, kW, kH, dW, dH, padW, padH, dilW, dilH, adjW,
                                                        adjH, scale):
        hx, hg, hw, hb = self.wrap(x), self.wrap(gy), self.wrap(gw), self.wrap(gb)
        try:
            self.call("SpatialFullDilatedConvolution_accGradParameters", hx, hg, hw, hb, None, None, kW, kH, dW, dH, padW, padH,
                      dilW, dilH, adjW, adjH, scale)
        finally:
            self.free(hx, hg, hw, hb)

    def SpatialFullConvolution_updateOutput(self, x, weight, bias, kW, kH, dW, dH, padW, padH, adjW, adjH):
        b = x.dim() == 4
        OH = (x.shape[b + 1] - 1) * dH - 2 * padH + kH + adjH
        OW = (x.shape[b + 2] - 1) * dW - 2 * padW + kW + adjW
        cap = max(1, (x.shape[0] if b else 1) * weight.shape[1] * max(OH, 1) * max(OW, 1))
        hx, hw, hb = self.wrap(x), self.wrap(weight), self.wrap(bias)
        ho, buf = self.out(cap)
        try:
            self.call("SpatialFullConvolution_updateOutput", hx, ho, hw, hb, None, None, kW, kH, dW, dH, padW, padH, adjW, adjH)
            return self.view(ho, buf)
        finally:
            self.free(hx, hw, hb, ho)

    def SpatialConvolutionLocal_updateOutput(self, x, weight, bias, kW, kH, dW, dH, padW, padH, iW, iH, oW, oH):
        b = x.dim() == 4
        K = weight.shape[2] if weight.dim() == 6 else weight.shape[1]
        hx, hw, hb = self.wrap(x), self.wrap(weight), self.wrap(bias)
        ho, buf = self.out((x.shape[0] if b else 1) * K * oH * oW)
        try:
            self.call("SpatialConvolutionLocal_updateOutput", hx, ho, hw, hb, None, None, kW, kH, dW, dH, padW, padH, iW, iH, oW, oH)
            return self.view(ho, buf)
        finally:
            self.free(hx, hw, hb, ho)

    def SpatialConvolutionLocal_updateGradInput(self, x, gy, weight, kW, kH, dW, dH, padW, padH, iW, iH, oW, oH):
        hx, hg, hw = self.wrap(x), self.wrap(gy), self.wrap(weight)
        ho, buf = self.out(x.numel())
        try:
            self.call("SpatialConvolutionLocal_updateGradInput", hx, hg, ho, hw, None, None, kW, kH, dW, dH, padW, padH, iW, iH, oW, oH)
            return self.view(ho, buf)
        finally:
            self.free(hx, hg, hw, ho)

    def SpatialConvolutionLocal_accGradParameters(self, x, gy, gw, gb, kW, kH, dW, dH, padW, padH, iW, iH, oW, oH, scale):
        hx, hg, hw, hb = self.wrap(x), self.wrap(gy), self.wrap(gw), self.wrap(gb)
        try:
            self.call("SpatialConvolutionLocal_accGradParameters", hx, hg, hw, hb, None, None, kW, kH, dW, dH, padW, padH, iW, iH,
                      oW, oH, scale)
        finally:
            self.free(hx, hg, hw, hb)

    def SpatialAdaptiveMaxPooling_updateOutput(self, x, nOutputCols, nOutputRows):
        planes = x.numel() // (x.shape[-1] * x.shape[-2])
        hx = self.wrap(x)
        ho, buf = self.out(planes * nOutputCols * nOutputRows)
        hi, ibuf = self.out(2 * planes * nOutputCols * nOutputRows, torch.int64)
        try:
            self.call("SpatialAdaptiveMaxPooling_updateOutput", hx, ho, hi, nOutputCols, nOutputRows)
            return self.view(ho, buf), self.view(hi, ibuf)
        finally:
            self.free(hx, ho, hi)

    def SpatialAdaptiveMaxPooling_updateGradInput(self, x, gy, indices):
        hx, hg, hi = self.wrap(x), self.wrap(gy), self.wrap(indices)
        ho, buf = self.out(x.numel())
        try:
            self.call("SpatialAdaptiveMaxPooling_updateGradInput", hx, hg, ho, hi)
            return self.view(ho, buf)
        finally:
            self.free(hx, hg, hi, ho)

    def SpatialAdaptiveAveragePooling_updateOutput(self, x, nOutputCols, nOutputRows):
        planes = x.numel() // (x.shape[-1] * x.shape[-2])
        hx = self.wrap(x)
        ho, buf = self.out(planes * nOutputCols * nOutputRows)
        try:
            self.call("SpatialAdaptiveAveragePooling_updateOutput", hx, ho, nOutputCols, nOutputRows)
            return self.view(ho, buf)
        finally:
            self.free(hx, ho)

    def SpatialAdaptiveAveragePooling_updateGradInput(self, x, gy):
        hx, hg = self.wrap(x), self.wrap(gy)
        ho, buf = self.out(x.numel())
        try:
            self.call("SpatialAdaptiveAveragePooling_updateGradInput", hx, hg, ho)
            return self.view(ho, buf)
        finally:
            self.free(hx, hg, ho)

    def BatchNormalization_updateOutput(self, x, weight, bias, running_mean, running_var, train, momentum, eps):
        C = x.shape[1]
        hx, hw, hb, hrm, hrv = self.wrap(x), self.wrap(weight), self.wrap(bias), self.wrap(running_mean), self.wrap(running_var)
        ho, buf = self.out(x.numel())
        hsm, bsm = self.out(C)
        hss, bss = self.out(C)
        try:
            self.call("BatchNormalization_updateOutput", hx, ho, hw, hb, hrm, hrv, hsm, hss, train, momentum, eps)
            return self.view(ho, buf), (bsm[:C] if train else None), (bss[:C] if train else None)
        finally:
            self.free(hx, hw, hb, hrm, hrv, ho, hsm, hss)

    def BatchNormalization_backward(self, x, gy, gw, gb, weight, running_mean, running_var, save_mean, save_std, train,
                                    scale, eps, want_gx=True):
        hs = [self.wrap(t) for t in (x, gy, gw, gb, weight, running_mean, running_var, save_mean, save_std)]
        ho, buf = self.out(x.numel()) if want_gx else (None, None)
        try:
            self.call("BatchNormalization_backward", hs[0], hs[1], ho, hs[2], hs[3], hs[4], hs[5], hs[6], hs[7], hs[8], train, scale, eps)
            return self.view(ho, buf) if want_gx else None
        finally:
            self.free(ho, *hs)

    def SpatialMaxPooling_updateOutput(self, x, kW, kH, dW, dH, padW, padH, ceil_mode):
        hx = self.wrap(x)
        ho, buf = self.out(x.numel())
        hi, ibuf = self.out(x.numel(), torch.int64)
        try:
            self.call("SpatialMaxPooling_updateOutput", hx, ho, hi, kW, kH, dW, dH, padW, padH, ceil_mode)
            return self.view(ho, buf), self.view(hi, ibuf)
        finally:
            self.free(hx, ho, hi)

    def SpatialMaxPooling_updateGradInput(self, x, gy, indices, kW, kH, dW, dH, padW, padH, ceil_mode):
        hx, hg, hi = self.wrap(x), self.wrap(gy), self.wrap(indices)
        ho, buf = self.out(x.numel())
        try:
            self.call("SpatialMaxPooling_updateGradInput", hx, hg, ho, hi, kW, kH, dW, dH, padW, padH, ceil_mode)
            return self.view(ho, buf)
        finally:
            self.free(hx, hg, hi, ho)
