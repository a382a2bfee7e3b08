"""SpatialDilatedConvolution on the tensor-core convolution kernel (gathering loader with dilated taps) against the
CPU oracle and the committed PyTorch-CPU fixtures; flat C ABI and the THNN entry points.  GEMM-path tolerance
1e-4 (element-wise relative error with a 1 % floor)."""
import numpy as np
import pytest

from conftest import golden, rel_err

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

TOL = 1e-4


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.detach().cpu().numpy()


@pytest.fixture(scope="module")
def F():
    import cunn_b200.functional as F
    from cunn_b200 import device_status
    yield F
    assert device_status() == 0


def run_all(F, x, w, b, gy, gw0, gb0, d, pad, dil, scale):
    H, W = x.shape[2:]
    y = F.dilated_conv_forward(dev(x), dev(w), None if b is None else dev(b), d, d, pad, pad, dil, dil)
    gx = F.dilated_conv_grad_input(dev(gy), dev(w), H, W, d, d, pad, pad, dil, dil)
    gw = dev(gw0)
    gb = None if gb0 is None else dev(gb0)
    F.dilated_conv_acc_grad(dev(x), dev(gy), gw, gb, d, d, pad, pad, dil, dil, scale)
    torch.cuda.synchronize()
    return host(y), host(gx), host(gw), None if gb is None else host(gb)


@pytest.mark.parametrize("name", ["dilconv_3x3_d2", "dilconv_3x3_d3_s2"])
def test_dilated_conv_golden(F, name):
    g = golden(name)
    K, k, d, pad, dil, has_b = [int(v) for v in g["params"]]
    y, gx, gw, gb = run_all(F, g["x"], g["w"], g["b"] if has_b else None, g["gy"], g["gw0"],
                            g["gb0"] if has_b else None, d, pad, dil, float(g["scale"]))
    assert rel_err(y, g["y"]) < TOL
    assert rel_err(gx, g["gx"]) < TOL
    assert rel_err(gw, g["gw"]) < TOL
    if has_b:
        assert rel_err(gb, g["gb"]) < TOL


@pytest.mark.parametrize("shape", [
    # N, C, H, W, K, k, stride, pad, dilation, bias
    (2, 16, 14, 14, 32, 3, 1, 2, 2, True),     # "same" 3x3, dilation 2
    (3, 8, 20, 17, 24, 3, 1, 0, 3, True),      # no padding, dilation 3, odd width
    (2, 6, 25, 25, 10, 5, 2, 4, 2, False),     # 5x5 (25 taps), stride 2: gather-form input gradient
    (2, 40, 9, 9, 130, 3, 1, 4, 4, True),      # dilation larger than half the plane, two column tiles
    (4, 64, 28, 28, 64, 3, 1, 2, 2, True),     # a DeepLab-style block
    (2, 12, 10, 10, 20, 1, 1, 0, 3, True),     # 1x1: dilation has no effect
])
def test_dilated_conv_shapes(F, ref64, shape):
    N, C, H, W, K, k, d, pad, dil, bias = shape
    rng = np.random.default_rng(abs(hash(shape)) % 99991)
    x = rng.standard_normal((N, C, H, W)).astype(np.float32)
    w = (rng.standard_normal((K, C, k, k)) * np.sqrt(2.0 / (C * k * k))).astype(np.float32)
    b = rng.uniform(-0.5, 0.5, K).astype(np.float32) if bias else None
    oH = (H + 2 * pad - (dil * (k - 1) + 1)) // d + 1
    oW = (W + 2 * pad - (dil * (k - 1) + 1)) // d + 1
    gy = rng.standard_normal((N, K, oH, oW)).astype(np.float32)
    gw0 = rng.standard_normal((K, C, k, k)).astype(np.float32)
    gb0 = rng.standard_normal(K).astype(np.float32) if bias else None
    y, gx, gw, gb = run_all(F, x, w, b, gy, gw0, gb0, d, pad, dil, 0.75)
    assert rel_err(y, ref64.dilconv_forward(x, w, b, d, d, pad, pad, dil, dil)) < TOL
    assert rel_err(gx, ref64.dilconv_grad_input(gy, w, H, W, d, d, pad, pad, dil, dil)) < TOL
    rgw, rgb = ref64.dilconv_acc_grad(x, gy, gw0, gb0, d, d, pad, pad, dil, dil, 0.75)
    assert rel_err(gw, rgw) < TOL
    if bias:
        assert rel_err(gb, rgb) < TOL


def test_dilation_one_equals_convolution_mm(F):
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn((3, 10, 12, 12), device="cuda", generator=g)
    w = torch.randn((7, 10, 3, 3), device="cuda", generator=g)
    b = torch.randn((7,), device="cuda", generator=g)
    assert torch.equal(F.dilated_conv_forward(x, w, b, 1, 1, 1, 1, 1, 1), F.convmm_forward(x, w, b, 1, 1, 1, 1))


def test_dilated_conv_errors(F):
    from cunn_b200 import CunnError
    x = torch.zeros((1, 2, 8, 8), device="cuda")
    with pytest.raises(CunnError, match="dilation should be greater than zero"):
        F.dilated_conv_forward(x, torch.zeros((2, 2, 3, 3), device="cuda"), None, 1, 1, 0, 0, 0, 1)
    with pytest.raises(CunnError, match="Output size is too small"):
        F.dilated_conv_forward(x, torch.zeros((2, 2, 3, 3), device="cuda"), None, 1, 1, 0, 0, 4, 4)
    with pytest.raises(CunnError, match="more than 32 taps"):
        F.dilated_conv_forward(torch.zeros((1, 2, 40, 40), device="cuda"), torch.zeros((2, 2, 7, 7), device="cuda"), None,
                               1, 1, 0, 0, 2, 2)


def test_thnn_dilated_convolution_entry_points(ref64):
    from cunn_b200.thnn import THNN
    rng = np.random.default_rng(12)
    N, C, H, W, K, k, pad, dil = 2, 6, 13, 11, 9, 3, 2, 2
    x = rng.standard_normal((N, C, H, W)).astype(np.float32)
    w = rng.standard_normal((K, C, k, k)).astype(np.float32) * 0.2
    b = rng.standard_normal(K).astype(np.float32)
    gy = rng.standard_normal((N, K, H, W)).astype(np.float32)
    th = THNN()
    try:
        y = th.SpatialDilatedConvolution_updateOutput(dev(x), dev(w), dev(b), k, k, 1, 1, pad, pad, dil, dil)
        assert tuple(y.shape) == (N, K, H, W)
        assert rel_err(host(y), ref64.dilconv_forward(x, w, b, 1, 1, pad, pad, dil, dil)) < TOL
        gx = th.SpatialDilatedConvolution_updateGradInput(dev(x), dev(gy), dev(w), k, k, 1, 1, pad, pad, dil, dil)
        assert rel_err(host(gx), ref64.dilconv_grad_input(gy, w, H, W, 1, 1, pad, pad, dil, dil)) < TOL
        gw, gb = dev(np.zeros_like(w)), dev(np.zeros_like(b))
        th.SpatialDilatedConvolution_accGradParameters(dev(x), dev(gy), gw, gb, k, k, 1, 1, pad, pad, dil, dil, 0.5)
        rgw, rgb = ref64.dilconv_acc_grad(x, gy, np.zeros_like(w), np.zeros_like(b), 1, 1, pad, pad, dil, dil, 0.5)
        assert rel_err(host(gw), rgw) < TOL and rel_err(host(gb), rgb) < TOL
        # 3-D (unbatched) input gives a 3-D output, as in the reference
        y3 = th.SpatialDilatedConvolution_updateOutput(dev(x[0]), dev(w), dev(b), k, k, 1, 1, pad, pad, dil, dil)
        assert tuple(y3.shape) == (K, H, W) and rel_err(host(y3), host(y)[0]) < 1e-6
    finally:
        th.close()
