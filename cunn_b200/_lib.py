"""Loads libTHCUNN.so and declares the flat C ABI (include/cunn_b200.h) for ctypes.

There is no fallback: if the library has not been built, importing raises.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(_HERE, "lib", "libTHCUNN.so")

if not os.path.exists(SO_PATH):
    raise ImportError(
        "cunn_b200: %s is missing; build it with `python -m cunn_b200.build` "
        "(there is no CPU or PyTorch fallback)" % SO_PATH)

lib = ctypes.CDLL(SO_PATH)

c_int, c_float, c_double, c_void_p, c_size_t = ctypes.c_int, ctypes.c_float, ctypes.c_double, ctypes.c_void_p, ctypes.c_size_t


def _decl(name, restype, argtypes):
    f = getattr(lib, name)
    f.restype = restype
    f.argtypes = argtypes
    return f


_decl("cunn_b200_last_error", ctypes.c_char_p, [])
_decl("cunn_b200_device_status", c_int, [])

_CONV = [c_int] * 11  # N C H W M|K kH kW dH dW padH padW
_decl("cunn_b200_dwconv_forward", c_int, [c_void_p] * 4 + _CONV + [c_void_p])
_decl("cunn_b200_dwconv_grad_input", c_int, [c_void_p] * 3 + _CONV + [c_void_p])
_decl("cunn_b200_dwconv_acc_grad_workspace", c_size_t, _CONV)
_decl("cunn_b200_dwconv_acc_grad", c_int, [c_void_p] * 4 + _CONV + [c_float, c_void_p, c_size_t, c_void_p])
_decl("cunn_b200_dwconv_acc_grad_static", c_int, [c_void_p] * 4 + _CONV + [c_float, c_void_p])
_decl("cunn_b200_dwconv_acc_grad_static_capacity", c_size_t, [])
_decl("cunn_b200_convmm_forward", c_int, [c_void_p] * 4 + _CONV + [c_void_p])
_decl("cunn_b200_convmm_grad_input", c_int, [c_void_p] * 3 + _CONV + [c_void_p])
_decl("cunn_b200_convmm_acc_grad_workspace", c_size_t, _CONV)
_decl("cunn_b200_convmm_acc_grad", c_int, [c_void_p] * 4 + _CONV + [c_float, c_void_p, c_size_t, c_void_p])
_DCONV = _CONV + [c_int, c_int]  # ... dilH dilW
_decl("cunn_b200_dilated_conv_forward", c_int, [c_void_p] * 4 + _DCONV + [c_void_p])
_decl("cunn_b200_dilated_conv_grad_input", c_int, [c_void_p] * 3 + _DCONV + [c_void_p])
_decl("cunn_b200_dilated_conv_acc_grad_workspace", c_size_t, _DCONV)
_decl("cunn_b200_dilated_conv_acc_grad", c_int, [c_void_p] * 4 + _DCONV + [c_float, c_void_p, c_size_t, c_void_p])
_FCONV = _DCONV + [c_int, c_int]  # ... adjH adjW
_decl("cunn_b200_full_conv_forward", c_int, [c_void_p] * 4 + _FCONV + [c_void_p])
_decl("cunn_b200_full_conv_grad_input", c_int, [c_void_p] * 3 + _FCONV + [c_void_p])
_decl("cunn_b200_full_conv_acc_grad_workspace", c_size_t, _FCONV)
_decl("cunn_b200_full_conv_acc_grad", c_int, [c_void_p] * 4 + _FCONV + [c_float, c_void_p, c_size_t, c_void_p])
_LCONV = _CONV + [c_int, c_int]  # ... oH oW
_decl("cunn_b200_local_conv_forward", c_int, [c_void_p] * 4 + _LCONV + [c_void_p])
_decl("cunn_b200_local_conv_grad_input", c_int, [c_void_p] * 3 + _LCONV + [c_void_p])
_decl("cunn_b200_local_conv_acc_grad", c_int, [c_void_p] * 4 + _LCONV + [c_float, c_void_p])
_decl("cunn_b200_adaptive_maxpool_forward", c_int, [c_void_p] * 3 + [c_int] * 5 + [c_void_p])
_decl("cunn_b200_adaptive_maxpool_backward", c_int, [c_void_p] * 3 + [c_int] * 5 + [c_void_p])
_decl("cunn_b200_adaptive_avgpool_forward", c_int, [c_void_p] * 2 + [c_int] * 5 + [c_void_p])
_decl("cunn_b200_adaptive_avgpool_backward", c_int, [c_void_p] * 2 + [c_int] * 5 + [c_void_p])
_decl("cunn_b200_maxpool_out_size", c_int, [c_int] * 6)
_decl("cunn_b200_maxpool_forward", c_int, [c_void_p] * 3 + [c_int] * 13 + [c_void_p])
_decl("cunn_b200_maxpool_backward", c_int, [c_void_p] * 3 + [c_int] * 13 + [c_void_p])
_decl("cunn_b200_batchnorm_workspace", c_size_t, [c_int, c_int])
_decl("cunn_b200_batchnorm_counter_bytes", c_size_t, [])
_decl("cunn_b200_convmm_set_tma", None, [c_int])
_decl("cunn_b200_convmm_get_tma", c_int, [])
_decl("cunn_b200_batchnorm_set_grouped", None, [c_int])
_decl("cunn_b200_batchnorm_get_grouped", c_int, [])
_decl("cunn_b200_batchnorm_forward", c_int, [c_void_p] * 8 + [c_int] * 4 + [c_double, c_double, c_void_p, c_size_t, c_void_p])
_decl("cunn_b200_batchnorm_relu_forward", c_int, [c_void_p] * 8 + [c_int] * 4 + [c_double, c_double, c_void_p, c_size_t, c_void_p])
_decl("cunn_b200_batchnorm_relu_backward", c_int, [c_void_p] * 11 + [c_int] * 4 + [c_double, c_double, c_void_p, c_size_t, c_void_p])
_decl("cunn_b200_batchnorm_backward", c_int, [c_void_p] * 10 + [c_int] * 4 + [c_double, c_double, c_void_p, c_size_t, c_void_p])
c_longlong = ctypes.c_longlong
_decl("cunn_b200_threshold_forward", c_int, [c_void_p, c_void_p, c_longlong, c_float, c_float, c_void_p])
_decl("cunn_b200_threshold_backward", c_int, [c_void_p, c_void_p, c_void_p, c_longlong, c_float, c_void_p])
_decl("cunn_b200_avgpool_forward", c_int, [c_void_p, c_void_p] + [c_int] * 13 + [c_void_p])
_decl("cunn_b200_avgpool_backward", c_int, [c_void_p, c_void_p] + [c_int] * 13 + [c_void_p])
_decl("cunn_b200_logsoftmax_forward", c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p])
_decl("cunn_b200_logsoftmax_backward", c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
_decl("cunn_b200_classnll_forward", c_int, [c_void_p] * 4 + [c_int, c_int, c_int, c_longlong, c_void_p])
_decl("cunn_b200_classnll_backward", c_int, [c_void_p] * 4 + [c_int, c_int, c_int, c_longlong, c_void_p])
_decl("cunn_b200_fill", c_int, [c_void_p, c_longlong, c_float, c_void_p])
_decl("cunn_b200_sgd_update", c_int, [c_void_p, c_void_p, c_longlong, c_float, c_void_p])
_decl("cunn_b200_set_deterministic", None, [c_int])
_decl("cunn_b200_get_deterministic", c_int, [])


class CunnError(RuntimeError):
    """Raised when an entry point rejects its arguments or a launch fails."""


def check(rc):
    if rc != 0:
        raise CunnError(lib.cunn_b200_last_error().decode())


def device_status():
    return lib.cunn_b200_device_status()
