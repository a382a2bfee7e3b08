"""The CPU oracle against the reference's OWN pooling kernels, executed on the host.

oracle/_ref/librefk_cpu.so is the reference's MaxPoolForward / MaxPoolBackward
(lib/THCUNN/SpatialDilatedMaxPooling.cu:8-80) and AvePoolForward / AvePoolBackward
(lib/THCUNN/SpatialAveragePooling.cu:7-82), compiled unchanged from the reference tree with each CUDA
thread run as one loop iteration.  These tests are the pin of the oracle's pooling routines on the
reference itself: values, int64 indices and input gradients must be bit-identical.  Shapes follow the
ranges of the reference's own pooling tests (test.lua:2052-2250): kernel 2..4, stride 1..3,
padding <= kernel/2, ceil and floor mode, plus dilation.  No GPU needed.
"""
import numpy as np
import pytest

from oracle import ref_kernels


@pytest.fixture(scope="module")
def refk():
    ref_kernels.build()
    if not ref_kernels.available_cpu():
        pytest.skip("oracle/_ref/librefk_cpu.so not built (the reference tree is absent on this machine)")
    return ref_kernels.RefKernelsCPU()


def _cases():
    rng = np.random.default_rng(20240611)
    out = []
    for _ in range(40):
        kH, kW = int(rng.integers(2, 5)), int(rng.integers(2, 5))
        dH, dW = int(rng.integers(1, 4)), int(rng.integers(1, 4))
        padH, padW = int(rng.integers(0, kH // 2 + 1)), int(rng.integers(0, kW // 2 + 1))
        dil = int(rng.integers(1, 3))
        H = int(rng.integers((kH - 1) * dil + 1, 24))
        W = int(rng.integers((kW - 1) * dil + 1, 24))
        out.append((int(rng.integers(1, 4)), int(rng.integers(1, 5)), H, W, kH, kW, dH, dW, padH, padW, dil,
                    bool(rng.integers(0, 2))))
    out.append((2, 3, 112, 112, 3, 3, 2, 2, 1, 1, 1, False))      # the geometry of the benchmarked pooling layer
    out.append((1, 2, 7, 7, 7, 7, 1, 1, 0, 0, 1, False))          # global window
    return out


@pytest.mark.parametrize("case", _cases())
def test_maxpool_oracle_equals_reference_kernels(ref64, refk, case):
    N, C, H, W, kH, kW, dH, dW, padH, padW, dil, ceil_mode = case
    assert ref64.index_base == refk.index_base
    rng = np.random.default_rng(abs(hash(case)) % (2 ** 32))
    # values drawn from a small set so that ties inside a window are frequent
    x = rng.integers(-4, 5, (N, C, H, W)).astype(np.float32) * 0.25
    y, ind = ref64.maxpool_forward(x, kH, kW, dH, dW, padH, padW, ceil_mode, dil, dil)
    oH, oW = y.shape[2:]
    y_r, ind_r = refk.maxpool_forward(x, oH, oW, kH, kW, dH, dW, padH, padW, dil, dil)
    assert np.array_equal(y, y_r)
    assert np.array_equal(ind, ind_r)
    gy = rng.standard_normal(y.shape).astype(np.float32)
    gx = ref64.maxpool_backward(gy, ind, H, W, kH, kW, dH, dW, padH, padW, dil, dil)
    gx_r = refk.maxpool_backward(gy, ind_r, H, W, kH, kW, dH, dW, padH, padW, dil, dil)
    # overlapping windows add up to ceil(k/s)^2 terms in fp32 in the reference and in fp64 here
    assert np.max(np.abs(gx - gx_r)) <= 4e-7 * max(1.0, float(np.max(np.abs(gx_r))))


def test_maxpool_nan_and_inf_windows_equal_reference_kernels(ref64, refk):
    x = np.random.default_rng(5).standard_normal((1, 2, 8, 8)).astype(np.float32)
    x[0, 0, :4, :4] = np.nan
    x[0, 1, 4:, :] = -np.inf
    x[0, 1, 0, 0] = np.inf
    y, ind = ref64.maxpool_forward(x, 2, 2, 2, 2, 0, 0, False)
    y_r, ind_r = refk.maxpool_forward(x, 4, 4, 2, 2, 2, 2, 0, 0)
    assert np.array_equal(ind, ind_r)
    assert np.array_equal(y, y_r)
    assert ind_r[0, 0, 0, 0] == -1 + refk.index_base


def _close(a, b, tol=1e-6):
    """Equal up to fp32-vs-fp64 summation rounding; non-finite entries (a ceil-mode window that lies
    wholly in the padding divides 0 by 0 in the reference) must sit in the same places."""
    fa, fb = np.isfinite(a), np.isfinite(b)
    assert np.array_equal(fa, fb)
    assert np.array_equal(np.isnan(a), np.isnan(b))
    if fb.any():
        assert np.max(np.abs(a[fb] - b[fb])) <= tol * max(1.0, float(np.max(np.abs(b[fb]))))


@pytest.mark.parametrize("case", _cases()[:20] + [(2, 4, 7, 7, 7, 7, 1, 1, 0, 0, 1, False)])
@pytest.mark.parametrize("include_pad", [True, False])
def test_avgpool_oracle_equals_reference_kernels(ref64, refk, case, include_pad):
    N, C, H, W, kH, kW, dH, dW, padH, padW, _, ceil_mode = case
    rng = np.random.default_rng(abs(hash(case)) % (2 ** 32))
    x = rng.standard_normal((N, C, H, W)).astype(np.float32)
    y = ref64.avgpool_forward(x, kH, kW, dH, dW, padH, padW, ceil_mode, include_pad)
    oH, oW = y.shape[2:]
    y_r = refk.avgpool_forward(x, oH, oW, kH, kW, dH, dW, padH, padW, include_pad)
    _close(y, y_r)
    gy = rng.standard_normal(y.shape).astype(np.float32)
    gx = ref64.avgpool_backward(gy, H, W, kH, kW, dH, dW, padH, padW, include_pad)
    gx_r = refk.avgpool_backward(gy, H, W, kH, kW, dH, dW, padH, padW, include_pad)
    _close(gx, gx_r)


@pytest.mark.parametrize("shape", [(2, 3, 7, 7, 3, 3), (1, 4, 10, 13, 4, 5), (2, 2, 8, 8, 8, 8), (1, 3, 5, 9, 7, 2), (3, 2, 14, 14, 1, 1),
                                   (1, 2, 6, 6, 4, 4)])
def test_adaptive_pooling_oracle_equals_reference_kernels(ref64, refk, shape):
    # SpatialAdaptiveMaxPooling / SpatialAdaptiveAveragePooling: the reference's kernels (window bounds in float
    # arithmetic, two index planes relative to the window start) run on the host, one emulated thread per block.
    N, C, H, W, oH, oW = shape
    rng = np.random.default_rng(abs(hash(shape)) % (2 ** 32))
    x = rng.integers(-4, 5, (N, C, H, W)).astype(np.float32) * 0.25           # ties inside windows
    y, ind = ref64.adaptive_maxpool_forward(x, oH, oW)
    y_r, ind_r = refk.adaptive_maxpool_forward(x, oH, oW)
    assert np.array_equal(y, y_r) and np.array_equal(ind, ind_r)
    gy = rng.standard_normal(y.shape).astype(np.float32)
    _close(ref64.adaptive_maxpool_backward(gy, ind, H, W), refk.adaptive_maxpool_backward(gy, ind_r, H, W))
    x = rng.standard_normal((N, C, H, W)).astype(np.float32)
    _close(ref64.adaptive_avgpool_forward(x, oH, oW), refk.adaptive_avgpool_forward(x, oH, oW))
    _close(ref64.adaptive_avgpool_backward(gy, H, W), refk.adaptive_avgpool_backward(gy, H, W))
