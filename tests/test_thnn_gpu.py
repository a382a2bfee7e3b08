"""THNN_Cuda* entry points (the reference's C ABI, tensor structs, callee-resized outputs, error hook)
against the flat ABI, which the other test files pin to the oracle.  Mirrors what the reference's tests
exercise at this level: strided inputs, 3-D (unbatched) inputs, bias / no bias, accumulate with scale."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nnb():
    from cunn_b200 import thnn
    b = thnn.THNN()
    yield b
    b.close()


@pytest.fixture(scope="module")
def F():
    import cunn_b200.functional as F
    return F


def non_contiguous(t):
    """Same values, strided memory (the reference's makeNonContiguous, test.lua:62-83)."""
    big = torch.empty(t.shape + (2,), device=t.device, dtype=t.dtype)
    big[..., 0] = t
    return big[..., 0]


def close(a, b, tol=1e-6):
    return float((a - b).abs().max()) <= tol * max(1.0, float(b.abs().max()))


def test_depthwise_entry_points(nnb, F):
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.rand((3, 6, 14, 14), device="cuda", generator=g)
    w = torch.rand((2, 6, 3, 3), device="cuda", generator=g) - 0.5
    b = torch.rand((2, 6), device="cuda", generator=g)
    for xin in (x, non_contiguous(x)):
        y = nnb.SpatialDepthWiseConvolution_updateOutput(xin, w, b, 3, 3, 1, 1, 1, 1)
        assert tuple(y.shape) == (3, 12, 14, 14)
        assert close(y, F.dwconv_forward(x, w, b, 1, 1, 1, 1))
    # 2-D weight [M, C*kH*kW] is accepted; no bias
    y = nnb.SpatialDepthWiseConvolution_updateOutput(x, w.view(2, 54), None, 3, 3, 2, 2, 1, 1)
    assert close(y, F.dwconv_forward(x, w, None, 2, 2, 1, 1))
    # unbatched input gives a 3-D output
    y3 = nnb.SpatialDepthWiseConvolution_updateOutput(x[0], w, b, 3, 3, 1, 1, 1, 1)
    assert tuple(y3.shape) == (12, 14, 14) and close(y3, F.dwconv_forward(x[:1], w, b, 1, 1, 1, 1)[0])
    gy = torch.randn((3, 12, 14, 14), device="cuda", generator=g)
    gx = nnb.SpatialDepthWiseConvolution_updateGradInput(x, non_contiguous(gy), w, 3, 3, 1, 1, 1, 1)
    assert close(gx, F.dwconv_grad_input(gy, w, 14, 14, 1, 1, 1, 1))
    gw, gb = torch.ones_like(w), torch.ones_like(b)
    nnb.SpatialDepthWiseConvolution_accGradParameters(x, gy, gw, gb, 3, 3, 1, 1, 1, 1, 0.5)
    rw, rb = torch.ones_like(w), torch.ones_like(b)
    F.dwconv_acc_grad(x, gy, rw, rb, 1, 1, 1, 1, 0.5)
    assert close(gw, rw) and close(gb, rb)


def test_convmm_entry_points(nnb, F):
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn((2, 8, 10, 9), device="cuda", generator=g)
    w = torch.randn((16, 8, 3, 3), device="cuda", generator=g) * 0.1
    b = torch.randn(16, device="cuda", generator=g)
    y = nnb.SpatialConvolutionMM_updateOutput(non_contiguous(x), w.view(16, 72), b, 3, 3, 1, 1, 1, 1)
    assert tuple(y.shape) == (2, 16, 10, 9) and close(y, F.convmm_forward(x, w, b, 1, 1, 1, 1))
    gy = torch.randn_like(y)
    gx = nnb.SpatialConvolutionMM_updateGradInput(x, gy, w, 3, 3, 1, 1, 1, 1)
    assert close(gx, F.convmm_grad_input(gy, w, 10, 9, 1, 1, 1, 1))
    gw, gb = torch.zeros_like(w), torch.zeros_like(b)
    nnb.SpatialConvolutionMM_accGradParameters(x, gy, gw, gb, 3, 3, 1, 1, 1, 1, 2.0)
    rw, rb = torch.zeros_like(w), torch.zeros_like(b)
    F.convmm_acc_grad(x, gy, rw, rb, 1, 1, 1, 1, 2.0)
    assert close(gw, rw, 1e-5) and close(gb, rb, 1e-5)
    # no bias, unbatched
    y3 = nnb.SpatialConvolutionMM_updateOutput(x[1], w, None, 3, 3, 2, 2, 0, 0)
    assert y3.dim() == 3 and close(y3, F.convmm_forward(x[1:2], w, None, 2, 2, 0, 0)[0])


def test_batchnorm_entry_points(nnb, F):
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn((4, 5, 6, 7), device="cuda", generator=g) * 2 + 0.5
    w, b = torch.rand(5, device="cuda", generator=g), torch.rand(5, device="cuda", generator=g)
    rm, rv = torch.zeros(5, device="cuda"), torch.ones(5, device="cuda")
    rm2, rv2 = rm.clone(), rv.clone()
    y, sm, ss = nnb.BatchNormalization_updateOutput(non_contiguous(x), w, b, rm, rv, True, 0.1, 1e-5)
    ry, rsm, rss = F.batchnorm_forward(x, w, b, rm2, rv2, True, 0.1, 1e-5)
    assert tuple(y.shape) == tuple(x.shape) and close(y, ry) and close(sm, rsm) and close(ss, rss) and close(rm, rm2) and close(rv, rv2)
    gy = torch.randn_like(x)
    gw, gb = torch.zeros(5, device="cuda"), torch.zeros(5, device="cuda")
    gx = nnb.BatchNormalization_backward(x, gy, gw, gb, w, rm, rv, sm, ss, True, 1.0, 1e-5)
    rgw, rgb = torch.zeros(5, device="cuda"), torch.zeros(5, device="cuda")
    rgx = F.batchnorm_backward(x, gy, w, rm2, rv2, rsm, rss, True, 1.0, 1e-5, grad_weight=rgw, grad_bias=rgb)
    assert close(gx, rgx) and close(gw, rgw) and close(gb, rgb)
    # inference mode, no affine, parameters only
    y, _, _ = nnb.BatchNormalization_updateOutput(x, None, None, rm, rv, False, 0.1, 1e-5)
    assert close(y, F.batchnorm_forward(x, None, None, rm2, rv2, False, 0.1, 1e-5)[0])
    assert nnb.BatchNormalization_backward(x, gy, gw, None, None, rm, rv, sm, ss, True, 1.0, 1e-5, want_gx=False) is None


def test_maxpool_entry_points(nnb, F):
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn((2, 3, 16, 24), device="cuda", generator=g)
    for ceil_mode in (False, True):
        y, ind = nnb.SpatialMaxPooling_updateOutput(non_contiguous(x), 3, 3, 2, 2, 1, 1, ceil_mode)
        ry, rind = F.maxpool_forward(x, 3, 3, 2, 2, 1, 1, ceil_mode)
        assert torch.equal(y, ry) and torch.equal(ind, rind)
        gy = torch.randn_like(ry)
        gx = nnb.SpatialMaxPooling_updateGradInput(x, gy, ind, 3, 3, 2, 2, 1, 1, ceil_mode)
        assert torch.equal(gx, F.maxpool_backward(gy, rind, 16, 24, 3, 3, 2, 2, 1, 1, ceil_mode))
    y3, ind3 = nnb.SpatialMaxPooling_updateOutput(x[0], 2, 2, 2, 2, 0, 0, False)
    assert y3.dim() == 3 and ind3.dim() == 4          # indices stay 4-D, as in the reference


def test_errors_reach_the_hook_with_the_reference_messages(nnb):
    from cunn_b200.thnn import THNNError
    x = torch.zeros((1, 4, 2, 2), device="cuda")
    with pytest.raises(THNNError, match="Output size is too small"):
        nnb.SpatialConvolutionMM_updateOutput(x, torch.zeros((8, 4, 5, 5), device="cuda"), None, 5, 5, 1, 1, 0, 0)
    with pytest.raises(THNNError, match="Need input of dimension 4 and input.size\\[1\\] == 3"):
        nnb.SpatialDepthWiseConvolution_updateOutput(x, torch.zeros((1, 3, 3, 3), device="cuda"), None, 3, 3, 1, 1, 1, 1)
    with pytest.raises(THNNError, match="pad should be smaller than half of kernel size"):
        nnb.SpatialMaxPooling_updateOutput(torch.zeros((1, 1, 8, 8), device="cuda"), 2, 2, 2, 2, 2, 2, False)
    with pytest.raises(THNNError, match="weight tensor has to be contiguous"):
        w = torch.zeros((8, 4, 3, 6), device="cuda")[..., ::2]
        nnb.SpatialConvolutionMM_updateOutput(x, w, None, 3, 3, 1, 1, 1, 1)
