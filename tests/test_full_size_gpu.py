"""The CUDA path against the fp64 CPU oracle at the sizes the benchmark figures are quoted on:
the 13 depthwise layers of MobileNetV1 at batch 64, the two ResNet-shaped GEMM convolutions at
batch 128 (3x3 256->256 and 1x1 1024->256 on 14x14), and batch normalisation + 3x3/2 max pooling on
256 x 64 x 112 x 112.  Whole tensors are compared (the oracle takes seconds per case on the host
cores).  Bars: forward 1e-5, gradients and every GEMM-path result 1e-4, pooling indices identical;
conftest.assert_parity states how the two error figures are judged and records them.
"""
import numpy as np
import pytest

from conftest import assert_parity

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

FWD_TOL = 1e-5
GRAD_TOL = 1e-4

# (C, H=W, stride) of the 13 depthwise layers
DW_STACK = [(32, 112, 1), (64, 112, 2), (128, 56, 1), (128, 56, 2), (256, 28, 1), (256, 28, 2),
            (512, 14, 1), (512, 14, 1), (512, 14, 1), (512, 14, 1), (512, 14, 1), (512, 14, 2), (1024, 7, 1)]


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.detach().cpu().numpy()


def normal(rng, shape, mean=0.0, std=1.0):
    a = rng.standard_normal(shape, dtype=np.float32)
    if std != 1.0:
        a *= np.float32(std)
    if mean != 0.0:
        a += np.float32(mean)
    return a


def uniform(rng, shape, lo, hi):
    a = rng.random(shape, dtype=np.float32)
    a *= np.float32(hi - lo)
    a += np.float32(lo)
    return a


@pytest.fixture(scope="module")
def F():
    import cunn_b200.functional as F
    from cunn_b200 import device_status
    yield F
    assert device_status() == 0


@pytest.mark.parametrize("layer", range(13))
def test_depthwise_stack_batch64(F, ref64, ref32, layer):
    C, HW, s = DW_STACK[layer]
    N = 64
    rng = np.random.default_rng(1234 + layer)
    oHW = (HW + 2 - 3) // s + 1
    x = uniform(rng, (N, C, HW, HW), -1, 1)
    w = uniform(rng, (1, C, 3, 3), -1 / 3, 1 / 3)
    b = uniform(rng, (1, C), -1 / 3, 1 / 3)
    gy = normal(rng, (N, C, oHW, oHW))
    gw0, gb0 = normal(rng, w.shape), normal(rng, b.shape)
    tag = "dw%02d %dx%dx%d s%d " % (layer + 1, C, HW, HW, s)
    y = host(F.dwconv_forward(dev(x), dev(w), dev(b), s, s, 1, 1))
    assert_parity(tag + "y", y, ref64.dwconv_forward(x, w, b, s, s, 1, 1), FWD_TOL,
                  lambda: ref32.dwconv_forward(x, w, b, s, s, 1, 1))
    del y
    gx = host(F.dwconv_grad_input(dev(gy), dev(w), HW, HW, s, s, 1, 1))
    assert_parity(tag + "gx", gx, ref64.dwconv_grad_input(gy, w, HW, HW, s, s, 1, 1), GRAD_TOL,
                  lambda: ref32.dwconv_grad_input(gy, w, HW, HW, s, s, 1, 1))
    del gx
    gw, gb = dev(gw0), dev(gb0)
    F.dwconv_acc_grad(dev(x), dev(gy), gw, gb, s, s, 1, 1, 0.5)
    rgw, rgb = ref64.dwconv_acc_grad(x, gy, gw0, gb0, s, s, 1, 1, 0.5)
    port = lambda: ref32.dwconv_acc_grad(x, gy, gw0, gb0, s, s, 1, 1, 0.5)
    assert_parity(tag + "gw", host(gw), rgw, GRAD_TOL, lambda: port()[0])
    assert_parity(tag + "gb", host(gb), rgb, GRAD_TOL, lambda: port()[1])


@pytest.mark.parametrize("cfg", [(128, 256, 256, 14, 3, 1), (128, 1024, 256, 14, 1, 0)])
def test_gemm_convolution_batch128(F, ref64, ref32, cfg):
    N, C, K, HW, k, pad = cfg
    rng = np.random.default_rng(77 + k)
    x = normal(rng, (N, C, HW, HW))
    w = normal(rng, (K, C, k, k), std=(2.0 / (C * k * k)) ** 0.5)
    b = uniform(rng, (K,), -1, 1)
    gy = normal(rng, (N, K, HW, HW))
    gw0, gb0 = normal(rng, w.shape), normal(rng, b.shape)
    tag = "mm %dx%d %d->%d " % (k, k, C, K)
    y = host(F.convmm_forward(dev(x), dev(w), dev(b), 1, 1, pad, pad))
    assert_parity(tag + "y", y, ref64.convmm_forward(x, w, b, 1, 1, pad, pad), GRAD_TOL,
                  lambda: ref32.convmm_forward(x, w, b, 1, 1, pad, pad))
    gx = host(F.convmm_grad_input(dev(gy), dev(w), HW, HW, 1, 1, pad, pad))
    assert_parity(tag + "gx", gx, ref64.convmm_grad_input(gy, w, HW, HW, 1, 1, pad, pad), GRAD_TOL,
                  lambda: ref32.convmm_grad_input(gy, w, HW, HW, 1, 1, pad, pad))
    gw, gb = dev(gw0), dev(gb0)
    F.convmm_acc_grad(dev(x), dev(gy), gw, gb, 1, 1, pad, pad, 0.75)
    rgw, rgb = ref64.convmm_acc_grad(x, gy, gw0, gb0, 1, 1, pad, pad, 0.75)
    port = lambda: ref32.convmm_acc_grad(x, gy, gw0, gb0, 1, 1, pad, pad, 0.75)
    assert_parity(tag + "gw", host(gw), rgw, GRAD_TOL, lambda: port()[0])
    assert_parity(tag + "gb", host(gb), rgb, GRAD_TOL, lambda: port()[1])


def test_batchnorm_and_maxpool_256x64x112x112(F, ref64, ref32):
    N, C, HW = 256, 64, 112
    rng = np.random.default_rng(4)
    x = normal(rng, (N, C, HW, HW), 0.5, 2.0)
    g = uniform(rng, (C,), 0, 1)
    beta = np.zeros(C, np.float32)
    rm0, rv0 = np.zeros(C, np.float32), np.ones(C, np.float32)
    mom, eps = 0.1, 1e-5

    # training forward
    rm, rv = dev(rm0), dev(rv0)
    xd = dev(x)
    y, sm, ss = F.batchnorm_forward(xd, dev(g), dev(beta), rm, rv, True, mom, eps)
    ry, rrm, rrv, rsm, rss = ref64.bn_forward(x, g, beta, rm0, rv0, True, mom, eps)
    yh = host(y)
    assert_parity("bn train y", yh, ry, FWD_TOL, lambda: ref32.bn_forward(x, g, beta, rm0, rv0, True, mom, eps)[0])
    assert_parity("bn save_mean", host(sm), rsm, FWD_TOL)
    assert_parity("bn save_invstd", host(ss), rss, FWD_TOL)
    assert_parity("bn running_mean", host(rm), rrm, FWD_TOL)
    assert_parity("bn running_var", host(rv), rrv, FWD_TOL)

    # max pooling 3x3 stride 2 pad 1 on the normalised tensor: values and int64 indices identical
    py, pind = F.maxpool_forward(y, 3, 3, 2, 2, 1, 1, False)
    rpy, rpind = ref64.maxpool_forward(yh, 3, 3, 2, 2, 1, 1, False)
    assert np.array_equal(host(py), rpy)
    assert int(np.count_nonzero(host(pind) != rpind)) == 0
    pgy = normal(rng, rpy.shape)
    pgx = host(F.maxpool_backward(dev(pgy), pind, HW, HW, 3, 3, 2, 2, 1, 1, False))
    assert_parity("maxpool gx", pgx, ref64.maxpool_backward(pgy, rpind, HW, HW, 3, 3, 2, 2, 1, 1), GRAD_TOL)
    del py, pind, rpy, rpind, pgy, pgx, y, yh, ry

    # evaluation forward with the updated running statistics
    ye, _, _ = F.batchnorm_forward(xd, dev(g), dev(beta), rm, rv, False, mom, eps)
    rye = ref64.bn_forward(x, g, beta, rrm, rrv, False, mom, eps)[0]
    assert_parity("bn eval y", host(ye), rye, FWD_TOL, lambda: ref32.bn_forward(x, g, beta, rrm, rrv, False, mom, eps)[0])
    del ye, rye

    # training backward
    gy = normal(rng, x.shape)
    gw0, gb0 = normal(rng, (C,)), normal(rng, (C,))
    gw, gb = dev(gw0), dev(gb0)
    gx = F.batchnorm_backward(xd, dev(gy), dev(g), rm, rv, sm, ss, True, 1.0, eps, grad_weight=gw, grad_bias=gb)
    rgx, rgw, rgb = ref64.bn_backward(x, gy, g, rrm, rrv, rsm, rss, True, 1.0, eps, gw=gw0, gb=gb0)
    port = lambda: ref32.bn_backward(x, gy, g, rrm, rrv, rsm, rss, True, 1.0, eps, gw=gw0, gb=gb0)
    assert_parity("bn train gx", host(gx), rgx, GRAD_TOL, lambda: port()[0])
    assert_parity("bn gw", host(gw), rgw, GRAD_TOL, lambda: port()[1])
    assert_parity("bn gb", host(gb), rgb, GRAD_TOL, lambda: port()[2])
