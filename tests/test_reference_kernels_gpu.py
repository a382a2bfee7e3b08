"""The CUDA path against the reference's OWN device kernels running on the same GPU.

oracle/_ref/librefk_gpu.so holds the reference's MaxPoolForward / MaxPoolBackward, AvePoolForward /
AvePoolBackward, the three BatchNormalization kernels and im2col / col2im, compiled unchanged from the
reference tree; the convolutions run in the reference's schedule (per-image unfold + cuBLAS SGEMM,
per-(image, channel) for the depthwise module).  This is the direct comparison the reference's
test-suite makes between two implementations (test.lua: forward 1e-4, backward 1e-2 absolute); the
bars here are the tighter ones of this build: pooling values and indices identical, forward 1e-5,
gradients and GEMM results 1e-4 (tensor-normalised; the reference's fp32 summation order is itself
that far from exact, so the element-wise figure is recorded only through the fp64-oracle tests).
"""
import numpy as np
import pytest

from conftest import norm_err

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def refk():
    from oracle import ref_kernels
    if not ref_kernels.available_gpu():
        pytest.skip("oracle/_ref/librefk_gpu.so was not built (needs the reference tree at build time)")
    return ref_kernels.RefKernelsGPU()


@pytest.fixture(scope="module")
def F():
    import cunn_b200.functional as F
    from cunn_b200 import device_status
    yield F
    assert device_status() == 0


def gen(seed):
    return torch.Generator(device="cuda").manual_seed(seed)


def nerr(a, b):
    return float((a.double() - b.double()).abs().max() / b.double().abs().max().clamp_min(1e-30))


@pytest.mark.parametrize("shape", [
    (256, 64, 112, 112, 3, 2, 1),     # the benchmarked pooling layer at full size
    (4, 8, 56, 56, 3, 2, 1), (3, 5, 31, 40, 3, 2, 1), (2, 3, 20, 20, 2, 2, 0), (2, 2, 15, 15, 3, 1, 1),
    (2, 2, 14, 14, 5, 3, 2),
])
@pytest.mark.parametrize("ties", [False, True])
def test_maxpool_identical_to_reference_kernels(F, refk, shape, ties):
    N, C, H, W, k, d, pad = shape
    g = gen(N * 7 + k)
    if ties:
        x = torch.randint(-3, 4, (N, C, H, W), device="cuda", generator=g).float() * 0.5
    else:
        x = torch.randn((N, C, H, W), device="cuda", generator=g)
    y, ind = F.maxpool_forward(x, k, k, d, d, pad, pad, False)
    y_r, ind_r = refk.maxpool_forward(x, y.shape[2], y.shape[3], k, k, d, d, pad, pad)
    assert torch.equal(y, y_r)
    assert int((ind != ind_r).sum()) == 0
    gy = torch.randn(y.shape, device="cuda", generator=g)
    gx = F.maxpool_backward(gy, ind, H, W, k, k, d, d, pad, pad, False)
    gx_r = refk.maxpool_backward(gy, ind_r, H, W, k, k, d, d, pad, pad)
    assert nerr(gx, gx_r) < 1e-6


def test_avgpool_against_reference_kernels(F, refk):
    g = gen(3)
    x = torch.randn((16, 1024, 7, 7), device="cuda", generator=g)
    y = F.avgpool_forward(x, 7, 7, 1, 1, 0, 0)
    assert nerr(y, refk.avgpool_forward(x, 1, 1, 7, 7, 1, 1, 0, 0)) < 1e-5
    gy = torch.randn(y.shape, device="cuda", generator=g)
    gx = F.avgpool_backward(gy, 7, 7, 7, 7, 1, 1, 0, 0)
    assert nerr(gx, refk.avgpool_backward(gy, 7, 7, 7, 7, 1, 1, 0, 0)) < 1e-6
    x = torch.randn((3, 5, 19, 23), device="cuda", generator=g)
    for include_pad in (True, False):
        y = F.avgpool_forward(x, 3, 3, 2, 2, 1, 1, False, include_pad)
        assert nerr(y, refk.avgpool_forward(x, y.shape[2], y.shape[3], 3, 3, 2, 2, 1, 1, include_pad)) < 1e-6


@pytest.mark.parametrize("shape", [(256, 64, 112 * 112), (32, 512, 196), (16, 1024, 49), (8, 7, 33)])
def test_batchnorm_against_reference_kernels(F, refk, shape):
    N, C, S = shape
    g = gen(C)
    x = torch.randn((N, C, S), device="cuda", generator=g) * 2 + 0.5
    w = torch.rand(C, device="cuda", generator=g)
    b = torch.randn(C, device="cuda", generator=g)
    rm0, rv0 = torch.randn(C, device="cuda", generator=g), torch.rand(C, device="cuda", generator=g) + 0.5
    y_r, rm_r, rv_r, sm_r, ss_r = refk.bn_forward(x, w, b, rm0, rv0, True, 0.1, 1e-5)
    rm, rv = rm0.clone(), rv0.clone()
    y, sm, ss = F.batchnorm_forward(x, w, b, rm, rv, True, 0.1, 1e-5)
    # the reference sums 3.2 M values per channel sequentially in fp32: its own distance to exact is ~1e-5
    assert nerr(y, y_r) < 5e-5
    assert nerr(sm, sm_r) < 5e-5 and nerr(ss, ss_r) < 5e-5
    assert nerr(rm, rm_r) < 5e-5 and nerr(rv, rv_r) < 5e-5
    ye_r = refk.bn_forward(x, w, b, rm0, rv0, False, 0.1, 1e-5)[0]
    ye = F.batchnorm_forward(x, w, b, rm0.clone(), rv0.clone(), False, 0.1, 1e-5)[0]
    assert nerr(ye, ye_r) < 1e-5
    gy = torch.randn(x.shape, device="cuda", generator=g)
    gw0, gb0 = torch.randn(C, device="cuda", generator=g), torch.randn(C, device="cuda", generator=g)
    for train in (True, False):
        gx_r, gw_r, gb_r = refk.bn_backward(x, gy, w, rm0, rv0, sm_r, ss_r, train, 0.5, 1e-5, gw=gw0, gb=gb0)
        gw, gb = gw0.clone(), gb0.clone()
        gx = F.batchnorm_backward(x, gy, w, rm0, rv0, sm_r, ss_r, train, 0.5, 1e-5, grad_weight=gw, grad_bias=gb)
        assert nerr(gx, gx_r) < 1e-4
        assert nerr(gw, gw_r) < 1e-4 and nerr(gb, gb_r) < 1e-4


@pytest.mark.parametrize("shape", [
    # N, C, H, W, K, k, d, pad
    (128, 256, 14, 14, 256, 3, 1, 1),       # the two benchmarked GEMM convolutions at full size
    (128, 1024, 14, 14, 256, 1, 1, 0),
    (4, 32, 112, 112, 64, 1, 1, 0), (4, 3, 224, 224, 32, 3, 2, 1), (3, 16, 23, 19, 24, 5, 2, 2), (2, 8, 30, 30, 16, 7, 3, 3),
])
def test_gemm_convolution_against_reference_schedule(F, refk, shape):
    N, C, H, W, K, k, d, pad = shape
    g = gen(C + k)
    x = torch.randn((N, C, H, W), device="cuda", generator=g)
    w = torch.randn((K, C, k, k), device="cuda", generator=g) * (2.0 / (C * k * k)) ** 0.5
    b = torch.rand(K, device="cuda", generator=g)
    y = F.convmm_forward(x, w, b, d, d, pad, pad)
    assert nerr(y, refk.convmm_forward(x, w, b, d, d, pad, pad)) < 1e-4
    gy = torch.randn(y.shape, device="cuda", generator=g)
    gx = F.convmm_grad_input(gy, w, H, W, d, d, pad, pad)
    assert nerr(gx, refk.convmm_grad_input(gy, w, H, W, d, d, pad, pad)) < 1e-4
    gw0, gb0 = torch.randn(w.shape, device="cuda", generator=g), torch.randn(K, device="cuda", generator=g)
    gw, gb = gw0.clone(), gb0.clone()
    F.convmm_acc_grad(x, gy, gw, gb, d, d, pad, pad, 0.75)
    gw_r, gb_r = refk.convmm_acc_grad(x, gy, gw0, gb0, d, d, pad, pad, 0.75)
    assert nerr(gw, gw_r) < 1e-4 and nerr(gb, gb_r) < 1e-4


@pytest.mark.parametrize("shape", [
    # N, C, H, W, M, k, d, pad
    (8, 32, 56, 56, 1, 3, 1, 1),      # the single-layer correctness configuration
    (2, 64, 112, 112, 1, 3, 2, 1), (2, 512, 14, 14, 1, 3, 1, 1), (2, 512, 14, 14, 1, 3, 2, 1), (2, 1024, 7, 7, 1, 3, 1, 1),
    (3, 3, 28, 28, 4, 3, 1, 1),       # the reference's own depthwise test shape (multiplier 4)
    (2, 5, 15, 17, 2, 5, 3, 2),
])
def test_depthwise_against_reference_schedule(F, refk, shape):
    N, C, H, W, M, k, d, pad = shape
    g = gen(C + H)
    x = torch.rand((N, C, H, W), device="cuda", generator=g) * 2 - 1
    w = (torch.rand((M, C, k, k), device="cuda", generator=g) * 2 - 1) / k
    b = (torch.rand((M, C), device="cuda", generator=g) * 2 - 1) / k
    y = F.dwconv_forward(x, w, b, d, d, pad, pad)
    assert nerr(y, refk.dwconv_forward(x, w, b, d, d, pad, pad)) < 1e-5
    gy = torch.randn(y.shape, device="cuda", generator=g)
    gx = F.dwconv_grad_input(gy, w, H, W, d, d, pad, pad)
    assert nerr(gx, refk.dwconv_grad_input(gy, w, H, W, d, d, pad, pad)) < 1e-4
    gw0, gb0 = torch.randn(w.shape, device="cuda", generator=g), torch.randn(b.shape, device="cuda", generator=g)
    gw, gb = gw0.clone(), gb0.clone()
    F.dwconv_acc_grad(x, gy, gw, gb, d, d, pad, pad, 0.5)
    gw_r, gb_r = refk.dwconv_acc_grad(x, gy, gw0, gb0, d, d, pad, pad, 0.5)
    assert nerr(gw, gw_r) < 1e-4 and nerr(gb, gb_r) < 1e-4
