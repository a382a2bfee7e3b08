"""THNN_CudaDouble* entry points of the hot path (the reference instantiates and tests every operator for
float and double: THCUNN.lua:131-132, test.lua:12-15) against the CPU oracle built for fp64 tensors.
The kernels accumulate in fp64, so the bar is 1e-11 of the largest element; pooling indices are identical."""
import numpy as np
import pytest

from conftest import norm_err

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

TOL = 1e-11


@pytest.fixture(scope="module")
def nnd():
    from cunn_b200 import thnn, device_status
    b = thnn.THNN(dtype=torch.float64)
    yield b
    b.close()
    assert device_status() == 0


def dev(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()


def H(t):
    return None if t is None else t.detach().cpu().numpy()


def non_contiguous(t):
    big = torch.empty(t.shape + (2,), device=t.device, dtype=t.dtype)
    big[..., 0] = t
    return big[..., 0]


@pytest.mark.parametrize("shape", [
    # N, C, H, W, M, k, d, pad, bias
    (8, 32, 56, 56, 1, 3, 1, 1, True),      # the single-layer configuration
    (3, 3, 28, 28, 4, 3, 1, 1, True),       # the reference's own depthwise test shape
    (2, 16, 14, 14, 1, 3, 2, 1, False), (2, 5, 15, 17, 2, 5, 3, 2, True), (1, 7, 7, 7, 1, 3, 1, 1, True),
])
def test_depthwise_double(nnd, refd, shape):
    N, C, Hh, W, M, k, d, pad, bias = shape
    rng = np.random.default_rng(abs(hash(shape)) % 9973)
    x = rng.uniform(-1, 1, (N, C, Hh, W))
    w = rng.uniform(-1, 1, (M, C, k, k)) / k
    b = rng.uniform(-1, 1, (M, C)) / k if bias else None
    y = nnd.SpatialDepthWiseConvolution_updateOutput(non_contiguous(dev(x)), dev(w), dev(b), k, k, d, d, pad, pad)
    assert y.dtype == torch.float64
    assert norm_err(H(y), refd.dwconv_forward(x, w, b, d, d, pad, pad)) < TOL
    gy = rng.standard_normal(tuple(y.shape))
    gx = nnd.SpatialDepthWiseConvolution_updateGradInput(dev(x), dev(gy), dev(w), k, k, d, d, pad, pad)
    assert norm_err(H(gx), refd.dwconv_grad_input(gy, w, Hh, W, d, d, pad, pad)) < TOL
    gw0, gb0 = rng.standard_normal(w.shape), (rng.standard_normal((M, C)) if bias else None)
    gw, gb = dev(gw0), dev(gb0)
    nnd.SpatialDepthWiseConvolution_accGradParameters(dev(x), dev(gy), gw, gb, k, k, d, d, pad, pad, 0.5)
    rgw, rgb = refd.dwconv_acc_grad(x, gy, gw0, gb0, d, d, pad, pad, 0.5)
    assert norm_err(H(gw), rgw) < TOL
    if bias:
        assert norm_err(H(gb), rgb) < TOL


@pytest.mark.parametrize("shape", [
    # N, C, H, W, K, k, d, pad, bias
    (4, 64, 14, 14, 96, 3, 1, 1, True), (3, 128, 14, 14, 80, 1, 1, 0, True), (2, 3, 33, 31, 32, 3, 2, 1, True),
    (2, 6, 13, 12, 10, 5, 2, 2, False), (3, 20, 7, 7, 70, 7, 1, 3, True), (70, 4, 5, 5, 3, 3, 1, 1, True),
])
def test_gemm_convolution_double(nnd, refd, shape):
    N, C, Hh, W, K, k, d, pad, bias = shape
    rng = np.random.default_rng(abs(hash(shape)) % 9973)
    x = rng.standard_normal((N, C, Hh, W))
    w = rng.standard_normal((K, C, k, k)) * (2.0 / (C * k * k)) ** 0.5
    b = rng.uniform(-1, 1, K) if bias else None
    y = nnd.SpatialConvolutionMM_updateOutput(dev(x), dev(w).view(K, C * k * k), dev(b), k, k, d, d, pad, pad)
    assert y.dtype == torch.float64
    assert norm_err(H(y), refd.convmm_forward(x, w, b, d, d, pad, pad)) < TOL
    gy = rng.standard_normal(tuple(y.shape))
    gx = nnd.SpatialConvolutionMM_updateGradInput(dev(x), non_contiguous(dev(gy)), dev(w), k, k, d, d, pad, pad)
    assert norm_err(H(gx), refd.convmm_grad_input(gy, w, Hh, W, d, d, pad, pad)) < TOL
    gw0, gb0 = rng.standard_normal(w.shape), (rng.standard_normal(K) if bias else None)
    gw, gb = dev(gw0), dev(gb0)
    nnd.SpatialConvolutionMM_accGradParameters(dev(x), dev(gy), gw, gb, k, k, d, d, pad, pad, 0.75)
    rgw, rgb = refd.convmm_acc_grad(x, gy, gw0, gb0, d, d, pad, pad, 0.75)
    assert norm_err(H(gw), rgw) < TOL
    if bias:
        assert norm_err(H(gb), rgb) < TOL


@pytest.mark.parametrize("shape,affine", [((16, 64, 28, 28), True), ((5, 7, 3, 11), False), ((300, 3, 1, 1), True)])
def test_batchnorm_double(nnd, refd, shape, affine):
    rng = np.random.default_rng(shape[1])
    C = shape[1]
    x = rng.standard_normal(shape) * 2 + 100.0                 # |mean| >> std: the shifted sums must cope
    w = rng.uniform(0, 1, C) if affine else None
    b = rng.standard_normal(C) if affine else None
    rm0, rv0 = rng.standard_normal(C), rng.uniform(0.5, 1.5, C)
    rm, rv = dev(rm0), dev(rv0)
    y, sm, ss = nnd.BatchNormalization_updateOutput(dev(x), dev(w), dev(b), rm, rv, True, 0.1, 1e-5)
    ry, rrm, rrv, rsm, rss = refd.bn_forward(x, w, b, rm0, rv0, True, 0.1, 1e-5)
    for got, want in ((y, ry), (sm, rsm), (ss, rss), (rm, rrm), (rv, rrv)):
        assert norm_err(H(got), want) < 1e-10
    gy = rng.standard_normal(shape)
    gw0, gb0 = rng.standard_normal(C), rng.standard_normal(C)
    for train in (True, False):
        gw, gb = dev(gw0), dev(gb0)
        gx = nnd.BatchNormalization_backward(dev(x), dev(gy), gw, gb, dev(w), dev(rm0), dev(rv0), dev(rsm), dev(rss), train, 0.5, 1e-5)
        rgx, rgw, rgb = refd.bn_backward(x, gy, w, rm0, rv0, rsm, rss, train, 0.5, 1e-5, gw=gw0, gb=gb0)
        assert norm_err(H(gx), rgx) < 1e-9 and norm_err(H(gw), rgw) < 1e-9 and norm_err(H(gb), rgb) < 1e-10
    ye, _, _ = nnd.BatchNormalization_updateOutput(dev(x), dev(w), dev(b), dev(rm0), dev(rv0), False, 0.1, 1e-5)
    assert norm_err(H(ye), refd.bn_forward(x, w, b, rm0, rv0, False, 0.1, 1e-5)[0]) < TOL


@pytest.mark.parametrize("shape", [
    # N, C, H, W, k, d, pad, ceil
    (4, 8, 112, 112, 3, 2, 1, False), (2, 5, 31, 40, 3, 2, 1, True), (1, 3, 20, 20, 2, 2, 0, False), (2, 2, 14, 14, 5, 3, 2, True),
])
def test_maxpool_double(nnd, refd, shape):
    N, C, Hh, W, k, d, pad, ceil_mode = shape
    rng = np.random.default_rng(k * 100 + d)
    x = rng.integers(-4, 5, (N, C, Hh, W)).astype(np.float64) * 0.25 + rng.integers(0, 2, (N, C, Hh, W)) * 1e-13   # ties and near-ties
    y, ind = nnd.SpatialMaxPooling_updateOutput(dev(x), k, k, d, d, pad, pad, ceil_mode)
    ry, rind = refd.maxpool_forward(x, k, k, d, d, pad, pad, ceil_mode)
    assert y.dtype == torch.float64 and np.array_equal(H(y), ry) and np.array_equal(H(ind), rind)
    gy = rng.standard_normal(ry.shape)
    gx = nnd.SpatialMaxPooling_updateGradInput(dev(x), dev(gy), ind, k, k, d, d, pad, pad, ceil_mode)
    assert norm_err(H(gx), refd.maxpool_backward(gy, rind, Hh, W, k, k, d, d, pad, pad)) < TOL


def test_double_errors_and_unimplemented_names(nnd):
    from cunn_b200.thnn import THNNError, lib
    import ctypes
    with pytest.raises(THNNError, match="Output size is too small"):
        nnd.SpatialConvolutionMM_updateOutput(torch.zeros((1, 4, 2, 2), device="cuda", dtype=torch.float64),
                                              torch.zeros((8, 4, 5, 5), device="cuda", dtype=torch.float64), None, 5, 5, 1, 1, 0, 0)
    f = lib.THNN_CudaDoubleAbs_updateOutput            # outside the hot path: reports through the hook
    f.restype, f.argtypes = None, [ctypes.c_void_p]
    f(nnd.state)
    assert "THNN_CudaDoubleAbs_updateOutput is not implemented" in nnd.errors[-1]
