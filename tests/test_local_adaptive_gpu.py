"""SpatialConvolutionLocal and the adaptive poolings on the GPU (flat ABI and THNN_Cuda* entry points) against the CPU
oracle.  Bars: forward 1e-5 (the local convolution is a long fp32 dot product: 1e-4), gradients 1e-4, indices identical."""
import numpy as np
import pytest

from conftest import rel_err

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def dev(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()


def H_(t):
    return t.detach().cpu().numpy()


@pytest.fixture(scope="module")
def nnb():
    from cunn_b200 import thnn, device_status
    b = thnn.THNN()
    yield b
    b.close()
    assert device_status() == 0


@pytest.mark.parametrize("shape", [(4, 16, 12, 12, 24, 3, 3, 1, 1, 1, 1), (10, 3, 17, 9, 5, 5, 3, 2, 1, 2, 1), (2, 8, 7, 7, 8, 1, 1, 1, 1, 0, 0)])
def test_local_convolution(nnb, ref64, shape):
    import cunn_b200.functional as F
    N, C, H, W, K, kH, kW, dH, dW, padH, padW = shape
    rng = np.random.default_rng(abs(hash(shape)) % 9973)
    oH, oW = (H + 2 * padH - kH) // dH + 1, (W + 2 * padW - kW) // dW + 1
    P, R = oH * oW, C * kH * kW
    x = rng.standard_normal((N, C, H, W)).astype(np.float32)
    w = (rng.standard_normal((P, K, R)) / np.sqrt(R)).astype(np.float32)
    b = rng.standard_normal((K, oH, oW)).astype(np.float32)
    gy = rng.standard_normal((N, K, oH, oW)).astype(np.float32)
    ry = ref64.localconv_forward(x, w, b, kH, kW, dH, dW, padH, padW)
    assert rel_err(H_(F.local_conv_forward(dev(x), dev(w), dev(b), kH, kW, dH, dW, padH, padW)), ry) < 1e-4
    # THNN entry point with the 6-D weight a Lua module holds, strided input
    big = torch.empty((N, C, H, W, 2), device="cuda")
    big[..., 0] = dev(x)
    y = nnb.SpatialConvolutionLocal_updateOutput(big[..., 0], dev(w).view(oH, oW, K, C, kH, kW), dev(b), kW, kH, dW, dH, padW, padH, W, H, oW, oH)
    assert tuple(y.shape) == (N, K, oH, oW) and rel_err(H_(y), ry) < 1e-4
    gx = nnb.SpatialConvolutionLocal_updateGradInput(dev(x), dev(gy), dev(w), kW, kH, dW, dH, padW, padH, W, H, oW, oH)
    assert rel_err(H_(gx), ref64.localconv_grad_input(gy, w, C, H, W, kH, kW, dH, dW, padH, padW)) < 1e-4
    gw0, gb0 = rng.standard_normal(w.shape).astype(np.float32), rng.standard_normal(b.shape).astype(np.float32)
    gw, gb = dev(gw0), dev(gb0)
    nnb.SpatialConvolutionLocal_accGradParameters(dev(x), dev(gy), gw, gb, kW, kH, dW, dH, padW, padH, W, H, oW, oH, 0.5)
    rgw, rgb = ref64.localconv_acc_grad(x, gy, gw0, gb0, kH, kW, dH, dW, padH, padW, 0.5)
    assert rel_err(H_(gw), rgw) < 1e-4 and rel_err(H_(gb), rgb) < 1e-4


@pytest.mark.parametrize("shape", [(2, 3, 7, 7, 3, 3), (3, 16, 56, 56, 7, 7), (1, 4, 10, 13, 4, 5), (2, 2, 8, 8, 8, 8), (1, 3, 5, 9, 7, 2),
                                   (8, 1024, 7, 7, 1, 1)])
def test_adaptive_pooling(nnb, ref64, shape):
    N, C, H, W, oH, oW = shape
    rng = np.random.default_rng(abs(hash(shape)) % 9973)
    x = rng.integers(-4, 5, (N, C, H, W)).astype(np.float32) * 0.25
    y, ind = nnb.SpatialAdaptiveMaxPooling_updateOutput(dev(x), oW, oH)
    ry, rind = ref64.adaptive_maxpool_forward(x, oH, oW)
    assert tuple(ind.shape) == (2, N, C, oH, oW)
    assert np.array_equal(H_(y), ry) and np.array_equal(H_(ind), rind)
    gy = rng.standard_normal(ry.shape).astype(np.float32)
    gx = nnb.SpatialAdaptiveMaxPooling_updateGradInput(dev(x), dev(gy), ind)
    assert rel_err(H_(gx), ref64.adaptive_maxpool_backward(gy, rind, H, W)) < 1e-5
    x = rng.standard_normal((N, C, H, W)).astype(np.float32)
    ya = nnb.SpatialAdaptiveAveragePooling_updateOutput(dev(x), oW, oH)
    assert rel_err(H_(ya), ref64.adaptive_avgpool_forward(x, oH, oW)) < 1e-5
    ga = nnb.SpatialAdaptiveAveragePooling_updateGradInput(dev(x), dev(gy))
    assert rel_err(H_(ga), ref64.adaptive_avgpool_backward(gy, H, W)) < 1e-4
    # unbatched input: 3-D output, indices [2, C, oH, oW]
    y3, ind3 = nnb.SpatialAdaptiveMaxPooling_updateOutput(dev(x[0]), oW, oH)
    assert y3.dim() == 3 and tuple(ind3.shape) == (2, C, oH, oW)
