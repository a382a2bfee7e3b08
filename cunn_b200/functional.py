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


def workspace(nbytes, device, tag="scratch"):
    """Grow-only, zero-initialised scratch buffer per (device, stream, tag).  The depthwise parameter
    gradient (tag "dwconv") and batch normalisation (tag "batchnorm") keep ticket counters in their buffers
    that must stay zero between calls, so no other operator may write there; everything else shares the
    "scratch" buffer."""
    key = (device.index, torch.cuda.current_stream().cuda_stream, tag)
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
    ws = workspace(need, x.device, "dwconv") if need else None
    check(lib.cunn_b200_dwconv_acc_grad(_ptr(x), _ptr(gy), _ptr(grad_weight), _ptr(grad_bias), N, C, H, W, M, kH, kW,
                                        dH, dW, padH, padW, scale, _ptr(ws), ws.numel() if ws is not None else 0,
                                        _stream()))
    return grad_weight, grad_bias


def maxpool_out_size(size, k, d, pad, ceil_mode, dil=1):
    return lib.cunn_b200_maxpool_out_size(size, k, d, pad, dil, int(ceil_mode))


def maxpool_forward(x, kH, kW, dH, dW, padH, padW, ceil_mode=False, out=None, indices=None):
    _chk(x)
    N, C, H, W = x.shape
    oH = max(maxpool_out_size(H, kH, dH, padH, ceil_mode), 0) if dH > 0 and kH > 0 else 0
    oW = max(maxpool_out_size(W, kW, dW, padW, ceil_mode), 0) if dW > 0 and kW > 0 else 0
    if out is None:
        out = torch.empty((N, C, oH, oW), dtype=torch.float32, device=x.device)
    if indices is None:
        indices = torch.empty((N, C, oH, oW), dtype=torch.int64, device=x.device)
    check(lib.cunn_b200_maxpool_forward(_ptr(x), _ptr(out), _ptr(indices), N, C, H, W, kH, kW, dH, dW, padH, padW,
                                        1, 1, int(ceil_mode), _stream()))
    return out, indices


def maxpool_backward(gy, indices, H, W, kH, kW, dH, dW, padH, padW, ceil_mode=False, out=None):
    _chk(gy, indices)
    N, C = gy.shape[:2]
    if out is None:
        out = torch.empty((N, C, H, W), dtype=torch.float32, device=gy.device)
    check(lib.cunn_b200_maxpool_backward(_ptr(gy), _ptr(indices), _ptr(out), N, C, H, W, kH, kW, dH, dW, padH, padW,
                                         1, 1, int(ceil_mode), _stream()))
    return out


def _bn_dims(x):
    N, C = x.shape[0], x.shape[1]
    S = 1
    for d in x.shape[2:]:
        S *= d
    return N, C, S


def batchnorm_forward(x, weight, bias, running_mean, running_var, train, momentum=0.1, eps=1e-5, out=None,
                      save_mean=None, save_std=None):
    """Updates running_mean / running_var in place when train; returns (y, save_mean, save_std)."""
    _chk(x, weight, bias, running_mean, running_var)
    N, C, S = _bn_dims(x)
    if out is None:
        out = torch.empty_like(x)
    if save_mean is None:
        save_mean = torch.empty(C, dtype=torch.float32, device=x.device)
    if save_std is None:
        save_std = torch.empty(C, dtype=torch.float32, device=x.device)
    ws = workspace(lib.cunn_b200_batchnorm_workspace(N, C), x.device, "batchnorm")
    check(lib.cunn_b200_batchnorm_forward(_ptr(x), _ptr(out), _ptr(weight), _ptr(bias), _ptr(running_mean),
                                          _ptr(running_var), _ptr(save_mean), _ptr(save_std), N, C, S, int(train),
                                          momentum, eps, _ptr(ws), ws.numel(), _stream()))
    return out, save_mean, save_std


def batchnorm_backward(x, gy, weight, running_mean, running_var, save_mean, save_std, train, scale=1.0, eps=1e-5,
                       grad_weight=None, grad_bias=None, want_gx=True, out=None):
    """Accumulates into grad_weight / grad_bias in place (each may be None); returns gx or None."""
    _chk(x, gy, weight, grad_weight, grad_bias)
    N, C, S = _bn_dims(x)
    if want_gx and out is None:
        out = torch.empty_like(x)
    ws = workspace(lib.cunn_b200_batchnorm_workspace(N, C), x.device, "batchnorm")
    check(lib.cunn_b200_batchnorm_backward(_ptr(x), _ptr(gy), _ptr(out) if want_gx else None, _ptr(grad_weight),
                                           _ptr(grad_bias), _ptr(weight), _ptr(running_mean), _ptr(running_var),
                                           _ptr(save_mean), _ptr(save_std), N, C, S, int(train), scale, eps,
                                           _ptr(ws), ws.numel(), _stream()))
    return out if want_gx else None


def convmm_forward(x, weight, bias, dH, dW, padH, padW, out=None):
    """weight: [K, C, kH, kW] contiguous (the reference's [K, C*kH*kW] view of the same memory)."""
    _chk(x, weight, bias)
    N, C, H, W = x.shape
    K, _, kH, kW = weight.shape
    oH, oW = conv_out(H, kH, dH, padH), conv_out(W, kW, dW, padW)
    if out is None:
        out = torch.empty((N, K, max(oH, 0), max(oW, 0)), dtype=torch.float32, device=x.device)
    check(lib.cunn_b200_convmm_forward(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), N, C, H, W, K, kH, kW,
                                       dH, dW, padH, padW, _stream()))
    return out


def convmm_grad_input(gy, weight, H, W, dH, dW, padH, padW, out=None):
    _chk(gy, weight)
    K, C, kH, kW = weight.shape
    N = gy.shape[0]
    if out is None:
        out = torch.empty((N, C, H, W), dtype=torch.float32, device=gy.device)
    check(lib.cunn_b200_convmm_grad_input(_ptr(gy), _ptr(weight), _ptr(out), N, C, H, W, K, kH, kW,
                                          dH, dW, padH, padW, _stream()))
    return out


def convmm_acc_grad(x, gy, grad_weight, grad_bias, dH, dW, padH, padW, scale=1.0):
    """Accumulates into grad_weight [K,C,kH,kW] and grad_bias [K] (may be None) in place."""
    _chk(x, gy, grad_weight, grad_bias)
    N, C, H, W = x.shape
    K, _, kH, kW = grad_weight.shape
    need = lib.cunn_b200_convmm_acc_grad_workspace(N, C, H, W, K, kH, kW, dH, dW, padH, padW)
    ws = workspace(need, x.device)
    check(lib.cunn_b200_convmm_acc_grad(_ptr(x), _ptr(gy), _ptr(grad_weight), _ptr(grad_bias), N, C, H, W, K, kH, kW,
                                        dH, dW, padH, padW, scale, _ptr(ws), ws.numel(), _stream()))
    return grad_weight, grad_bias


def dilated_conv_out(size, k, d, pad, dil):
    return (size + 2 * pad - (dil * (k - 1) + 1)) // d + 1 if d > 0 else 0


def dilated_conv_forward(x, weight, bias, dH, dW, padH, padW, dilH, dilW, out=None):
    """SpatialDilatedConvolution forward; weight [K, C, kH, kW]."""
    _chk(x, weight, bias)
    N, C, H, W = x.shape
    K, _, kH, kW = weight.shape
    oH, oW = dilated_conv_out(H, kH, dH, padH, dilH), dilated_conv_out(W, kW, dW, padW, dilW)
    if out is None:
        out = torch.empty((N, K, max(oH, 0), max(oW, 0)), dtype=torch.float32, device=x.device)
    check(lib.cunn_b200_dilated_conv_forward(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), N, C, H, W, K, kH, kW,
                                             dH, dW, padH, padW, dilH, dilW, _stream()))
    return out


def dilated_conv_grad_input(gy, weight, H, W, dH, dW, padH, padW, dilH, dilW, out=None):
    _chk(gy, weight)
    K, C, kH, kW = weight.shape
    N = gy.shape[0]
    if out is None:
        out = torch.empty((N, C, H, W), dtype=torch.float32, device=gy.device)
    check(lib.cunn_b200_dilated_conv_grad_input(_ptr(gy), _ptr(weight), _ptr(out), N, C, H, W, K, kH, kW,
                                                dH, dW, padH, padW, dilH, dilW, _stream()))
    return out


def dilated_conv_acc_grad(x, gy, grad_weight, grad_bias, dH, dW, padH, padW, dilH, dilW, scale=1.0):
    """Accumulates into grad_weight [K,C,kH,kW] and grad_bias [K] (may be None) in place."""
    _chk(x, gy, grad_weight, grad_bias)
    N, C, H, W = x.shape
    K, _, kH, kW = grad_weight.shape
    need = lib.cunn_b200_dilated_conv_acc_grad_workspace(N, C, H, W, K, kH, kW, dH, dW, padH, padW, dilH, dilW)
    ws = workspace(need, x.device)
    check(lib.cunn_b200_dilated_conv_acc_grad(_ptr(x), _ptr(gy), _ptr(grad_weight), _ptr(grad_bias), N, C, H, W, K, kH, kW,
                                              dH, dW, padH, padW, dilH, dilW, scale, _ptr(ws), ws.numel(), _stream()))
    return grad_weight, grad_bias


def full_conv_out(size, k, d, pad, dil, adj):
    return (size - 1) * d - 2 * pad + dil * (k - 1) + 1 + adj


def full_conv_forward(x, weight, bias, dH, dW, padH, padW, dilH=1, dilW=1, adjH=0, adjW=0, out=None):
    """SpatialFullDilatedConvolution (transposed convolution) forward; weight [P, Q, kH, kW], x [N, P, H, W]."""
    _chk(x, weight, bias)
    N, P, H, W = x.shape
    _, Q, kH, kW = weight.shape
    OH, OW = full_conv_out(H, kH, dH, padH, dilH, adjH), full_conv_out(W, kW, dW, padW, dilW, adjW)
    if out is None:
        out = torch.empty((N, Q, max(OH, 0), max(OW, 0)), dtype=torch.float32, device=x.device)
    check(lib.cunn_b200_full_conv_forward(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), N, P, H, W, Q, kH, kW,
                                          dH, dW, padH, padW, dilH, dilW, adjH, adjW, _stream()))
    return out


def full_conv_grad_input(gy, weight, H, W, dH, dW, padH, padW, dilH=1, dilW=1, adjH=0, adjW=0, out=None):
    _chk(gy, weight)
    P, Q, kH, kW = weight.shape
    N = gy.shape[0]
    if out is None:
        out = torch.empty((N, P, H, W), dtype=torch.float32, device=gy.device)
    check(lib.cunn_b200_full_conv_grad_input(_ptr(gy), _ptr(weight), _ptr(out), N, P, H, W, Q, kH, kW,
                                             dH, dW, padH, padW, dilH, dilW, adjH, adjW, _stream()))
    return out


def full_conv_acc_grad(x, gy, grad_weight, grad_bias, dH, dW, padH, padW, dilH=1, dilW=1, adjH=0, adjW=0, scale=1.0):
    """Accumulates into grad_weight [P,Q,kH,kW] and grad_bias [Q] (may be None) in place."""
    _chk(x, gy, grad_weight, grad_bias)
    N, P, H, W = x.shape
    _, Q, kH, kW = grad_weight.shape
    geo = (N, P, H, W, Q, kH, kW, dH, dW, padH, padW, dilH, dilW, adjH, adjW)
    ws = workspace(lib.cunn_b200_full_conv_acc_grad_workspace(*geo), x.device)
    check(lib.cunn_b200_full_conv_acc_grad(_ptr(x), _ptr(gy), _ptr(grad_weight), _ptr(grad_bias), *geo, scale,
                                           _ptr(ws), ws.numel(), _stream()))
    return grad_weight, grad_bias


def threshold_forward(x, threshold=0.0, value=0.0, out=None):
    _chk(x, out)
    if out is None:
        out = torch.empty_like(x)
    check(lib.cunn_b200_threshold_forward(_ptr(x), _ptr(out), x.numel(), threshold, value, _stream()))
    return out


def threshold_backward(x, gy, threshold=0.0, out=None):
    _chk(x, gy, out)
    if out is None:
        out = torch.empty_like(x)
    check(lib.cunn_b200_threshold_backward(_ptr(x), _ptr(gy), _ptr(out), x.numel(), threshold, _stream()))
    return out


def avgpool_forward(x, kH, kW, dH, dW, padH, padW, ceil_mode=False, count_include_pad=True, out=None):
    _chk(x)
    N, C, H, W = x.shape
    oH, oW = maxpool_out_size(H, kH, dH, padH, ceil_mode), maxpool_out_size(W, kW, dW, padW, ceil_mode)
    if out is None:
        out = torch.empty((N, C, oH, oW), dtype=torch.float32, device=x.device)
    check(lib.cunn_b200_avgpool_forward(_ptr(x), _ptr(out), N, C, H, W, oH, oW, kH, kW, dH, dW, padH, padW,
                                        int(count_include_pad), _stream()))
    return out


def avgpool_backward(gy, H, W, kH, kW, dH, dW, padH, padW, count_include_pad=True, out=None):
    _chk(gy)
    N, C, oH, oW = gy.shape
    if out is None:
        out = torch.empty((N, C, H, W), dtype=torch.float32, device=gy.device)
    check(lib.cunn_b200_avgpool_backward(_ptr(gy), _ptr(out), N, C, H, W, oH, oW, kH, kW, dH, dW, padH, padW,
                                         int(count_include_pad), _stream()))
    return out


def logsoftmax_forward(x, out=None):
    _chk(x)
    if out is None:
        out = torch.empty_like(x)
    check(lib.cunn_b200_logsoftmax_forward(_ptr(x), _ptr(out), x.shape[0], x.shape[1], _stream()))
    return out


def logsoftmax_backward(y, gy, out=None):
    _chk(y, gy)
    if out is None:
        out = torch.empty_like(y)
    check(lib.cunn_b200_logsoftmax_backward(_ptr(y), _ptr(gy), _ptr(out), y.shape[0], y.shape[1], _stream()))
    return out


def classnll_forward(logprob, target, weights=None, size_average=True, ignore_index=-100, out=None):
    """Returns a 2-element device tensor [loss, total_weight]."""
    _chk(logprob, target, weights)
    if out is None:
        out = torch.zeros(2, dtype=torch.float32, device=logprob.device)
    check(lib.cunn_b200_classnll_forward(_ptr(logprob), _ptr(target), _ptr(weights), _ptr(out), logprob.shape[0],
                                         logprob.shape[1], int(size_average), ignore_index, _stream()))
    return out


def classnll_backward(target, loss_and_weight, B, D, weights=None, size_average=True, ignore_index=-100, out=None):
    _chk(target, weights)
    if out is None:
        out = torch.zeros((B, D), dtype=torch.float32, device=target.device)
    check(lib.cunn_b200_classnll_backward(_ptr(target), _ptr(weights), loss_and_weight[1:].data_ptr(), _ptr(out), B, D,
                                          int(size_average), ignore_index, _stream()))
    return out


def sgd_update(params, grads, lr):
    _chk(params, grads)
    check(lib.cunn_b200_sgd_update(_ptr(params), _ptr(grads), params.numel(), lr, _stream()))
    return params


def batchnorm_relu_forward(x, weight, bias, running_mean, running_var, train, momentum=0.1, eps=1e-5, out=None):
    """y = max(0, BN(x)) in one pass; returns (y, save_mean, save_std)."""
    _chk(x, weight, bias, running_mean, running_var)
    N, C, S = _bn_dims(x)
    if out is None:
        out = torch.empty_like(x)
    save_mean = torch.empty(C, dtype=torch.float32, device=x.device)
    save_std = torch.empty(C, dtype=torch.float32, device=x.device)
    ws = workspace(lib.cunn_b200_batchnorm_workspace(N, C), x.device, "batchnorm")
    check(lib.cunn_b200_batchnorm_relu_forward(_ptr(x), _ptr(out), _ptr(weight), _ptr(bias), _ptr(running_mean),
                                               _ptr(running_var), _ptr(save_mean), _ptr(save_std), N, C, S, int(train),
                                               momentum, eps, _ptr(ws), ws.numel(), _stream()))
    return out, save_mean, save_std


def batchnorm_relu_backward(x, gy, weight, bias, running_mean, running_var, save_mean, save_std, train, scale=1.0, eps=1e-5,
                            grad_weight=None, grad_bias=None):
    """Backward of batchnorm_relu_forward (same x, weight, bias and statistics); accumulates into grad_weight / grad_bias."""
    _chk(x, gy, weight, bias, grad_weight, grad_bias)
    N, C, S = _bn_dims(x)
    out = torch.empty_like(x)
    ws = workspace(lib.cunn_b200_batchnorm_workspace(N, C), x.device, "batchnorm")
    check(lib.cunn_b200_batchnorm_relu_backward(_ptr(x), _ptr(gy), _ptr(out), _ptr(grad_weight), _ptr(grad_bias),
                                                _ptr(weight), _ptr(bias), _ptr(running_mean), _ptr(running_var), _ptr(save_mean),
                                                _ptr(save_std), N, C, S, int(train), scale, eps, _ptr(ws), ws.numel(),
                                                _stream()))
    return out


def local_conv_forward(x, weight, bias, kH, kW, dH, dW, padH, padW, out=None):
    """SpatialConvolutionLocal forward; weight [oH*oW, K, C*kH*kW], bias [K, oH, oW] or None."""
    _chk(x, weight, bias)
    N, C, H, W = x.shape
    K = weight.shape[1]
    oH, oW = conv_out(H, kH, dH, padH), conv_out(W, kW, dW, padW)
    if out is None:
        out = torch.empty((N, K, oH, oW), dtype=torch.float32, device=x.device)
    check(lib.cunn_b200_local_conv_forward(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), N, C, H, W, K, kH, kW, dH, dW, padH, padW,
                                           oH, oW, _stream()))
    return out


def local_conv_grad_input(gy, weight, C, H, W, kH, kW, dH, dW, padH, padW, out=None):
    _chk(gy, weight)
    N, K, oH, oW = gy.shape
    if out is None:
        out = torch.empty((N, C, H, W), dtype=torch.float32, device=gy.device)
    check(lib.cunn_b200_local_conv_grad_input(_ptr(gy), _ptr(weight), _ptr(out), N, C, H, W, K, kH, kW, dH, dW, padH, padW, oH, oW,
                                              _stream()))
    return out


def local_conv_acc_grad(x, gy, grad_weight, grad_bias, kH, kW, dH, dW, padH, padW, scale=1.0):
    """Accumulates into grad_weight [oH*oW, K, C*kH*kW] and grad_bias [K, oH, oW] (may be None) in place."""
    _chk(x, gy, grad_weight, grad_bias)
    N, C, H, W = x.shape
    _, K, oH, oW = gy.shape
    check(lib.cunn_b200_local_conv_acc_grad(_ptr(x), _ptr(gy), _ptr(grad_weight), _ptr(grad_bias), N, C, H, W, K, kH, kW, dH, dW, padH,
                                            padW, oH, oW, scale, _stream()))
    return grad_weight, grad_bias


def adaptive_maxpool_forward(x, oH, oW):
    """Returns y [N, C, oH, oW] and int64 indices [2, N, C, oH, oW]: row and column of the maximum inside its window."""
    _chk(x)
    N, C, H, W = x.shape
    y = torch.empty((N, C, oH, oW), dtype=torch.float32, device=x.device)
    ind = torch.empty((2, N, C, oH, oW), dtype=torch.int64, device=x.device)
    check(lib.cunn_b200_adaptive_maxpool_forward(_ptr(x), _ptr(y), _ptr(ind), N * C, H, W, oH, oW, _stream()))
    return y, ind


def adaptive_maxpool_backward(gy, indices, H, W):
    _chk(gy, indices)
    N, C, oH, oW = gy.shape
    gx = torch.empty((N, C, H, W), dtype=torch.float32, device=gy.device)
    check(lib.cunn_b200_adaptive_maxpool_backward(_ptr(gy), _ptr(indices), _ptr(gx), N * C, H, W, oH, oW, _stream()))
    return gx


def adaptive_avgpool_forward(x, oH, oW):
    _chk(x)
    N, C, H, W = x.shape
    y = torch.empty((N, C, oH, oW), dtype=torch.float32, device=x.device)
    check(lib.cunn_b200_adaptive_avgpool_forward(_ptr(x), _ptr(y), N * C, H, W, oH, oW, _stream()))
    return y


def adaptive_avgpool_backward(gy, H, W):
    _chk(gy)
    N, C, oH, oW = gy.shape
    gx = torch.empty((N, C, H, W), dtype=torch.float32, device=gy.device)
    check(lib.cunn_b200_adaptive_avgpool_backward(_ptr(gy), _ptr(gx), N * C, H, W, oH, oW, _stream()))
    return gx
