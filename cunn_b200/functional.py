"""Flat-ABI calls on torch CUDA tensors.

Each function mirrors one entry point of include/cunn_b200.h.  torch is used
for device memory and the current stream only; all arithmetic happens in
libTHCUNN.so.  Inputs must be contiguous fp32 CUDA tensors.
"""
import torch

from ._lib import lib, check

_workspaces = {}


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _chk(*ts):
    for t in ts:
        if t is None:
            continue
        if not (t.is_cuda and t.is_contiguous()):
            raise ValueError("expected contiguous CUDA tensors")


def _ptr(t):
    return None if t is None else t.data_ptr()


def workspace(nbytes, device):
    """Grow-only, zero-initialised scratch buffer per (device, stream); the kernels that use it keep its
    control words zero between calls."""
    key = (device.index, torch.cuda.current_stream().cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.zeros(max(int(nbytes), 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def conv_out(size, k, d, pad):
    return (size + 2 * pad - k) // d + 1 if d > 0 else 0


def dwconv_forward(x, weight, bias, dH, dW, padH, padW, out=None):
    _chk(x, weight, bias)
    N, C, H, W = x.shape
    M, _, kH, kW = weight.shape
    oH, oW = conv_out(H, kH, dH, padH), conv_out(W, kW, dW, padW)
    if out is None:
        out = torch.empty((N, C * M, max(oH, 0), max(oW, 0)), dtype=torch.float32, device=x.device)
    check(lib.cunn_b200_dwconv_forward(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), N, C, H, W, M, kH, kW,
                                       dH, dW, padH, padW, _stream()))
    return out


def dwconv_grad_input(gy, weight, H, W, dH, dW, padH, padW, out=None):
    _chk(gy, weight)
    M, C, kH, kW = weight.shape
    N = gy.shape[0]
    if out is None:
        out = torch.empty((N, C, H, W), dtype=torch.float32, device=gy.device)
    check(lib.cunn_b200_dwconv_grad_input(_ptr(gy), _ptr(weight), _ptr(out), N, C, H, W, M, kH, kW,
                                          dH, dW, padH, padW, _stream()))
    return out


def dwconv_acc_grad(x, gy, grad_weight, grad_bias, dH, dW, padH, padW, scale=1.0):
    """Accumulates into grad_weight [M,C,kH,kW] and grad_bias [M,C] (may be None) in place."""
    _chk(x, gy, grad_weight, grad_bias)
    N, C, H, W = x.shape
    M, _, kH, kW = grad_weight.shape
    need = lib.cunn_b200_dwconv_acc_grad_workspace(N, C, H, W, M, kH, kW, dH, dW, padH, padW)
    ws = workspace(need, x.device) if need else None
    check(lib.cunn_b200_dwconv_acc_grad(_ptr(x), _ptr(gy), _ptr(grad_weight), _ptr(grad_bias), N, C, H, W, M, kH, kW,
                                        dH, dW, padH, padW, scale, _ptr(ws), ws.numel() if ws is not None else 0,
                                        _stream()))
    return grad_weight, grad_bias
