"""SpatialFullDilatedConvolution / SpatialFullConvolution (transposed convolution) on the kernels of the convolution it is
the adjoint of, against the CPU oracle and the committed PyTorch-CPU fixtures; flat C ABI and the THNN entry points.
GEMM-path tolerance 1e-4 (element-wise relative error with a 1 % floor)."""
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


def run_all(F, x, w, b, gy, gw0, gb0, geo, scale):
    H, W = x.shape[2:]
    y = F.full_conv_forward(dev(x), dev(w), None if b is None else dev(b), *geo)
    gx = F.full_conv_grad_input(dev(gy), dev(w), H, W, *geo)
    gw = dev(gw0)
    gb = None if gb0 is None else dev(gb0)
    F.full_conv_acc_grad(dev(x), dev(gy), gw, gb, *geo, scale=scale)
    torch.cuda.synchronize()
    return host(y), host(gx), host(gw), None if gb is None else host(gb)


@pytest.mark.parametrize("name", ["fullconv_3x3_s2", "fullconv_4x4_s2", "fullconv_3x3_d2"])
def test_full_conv_golden(F, name):
    g = golden(name)
    Q, k, d, pad, dil, adj, has_b = [int(v) for v in g["params"]]
    y, gx, gw, gb = run_all(F, g["x"], g["w"], g["b"] if has_b else None, g["gy"], g["gw0"],
                            g["gb0"] if has_b else None, (d, d, pad, pad, dil, dil, adj, adj), float(g["scale"]))
    assert y.shape == g["y"].shape
    assert rel_err(y, g["y"]) < TOL
    assert rel_err(gx, g["gx"]) < TOL
    assert rel_err(gw, g["gw"]) < TOL
    if has_b:
        assert rel_err(gb, g["gb"]) < TOL


@pytest.mark.parametrize("shape", [
    # N, P (in), H, W, Q (out), k, stride, pad, dilation, adj, bias
    (2, 16, 14, 14, 32, 3, 1, 1, 1, 0, True),     # stride 1: forward runs on the tensor cores
    (3, 24, 9, 11, 12, 4, 2, 1, 1, 0, True),      # 4x4 stride 2 (decoder / generator layer): doubles the plane
    (2, 8, 7, 7, 20, 3, 2, 1, 1, 1, True),        # 3x3 stride 2 with output padding 1
    (2, 130, 6, 6, 40, 1, 1, 0, 1, 0, False),     # 1x1: a plain matrix product, no bias
    (2, 10, 8, 8, 6, 3, 1, 2, 2, 0, True),        # dilation 2
    (1, 5, 5, 6, 7, 5, 3, 0, 1, 2, True),         # 5x5 stride 3, no padding, output padding 2
    (4, 64, 16, 16, 32, 2, 2, 0, 1, 0, True),     # 2x2 stride 2 (U-Net up-convolution)
])
def test_full_conv_shapes(F, ref64, shape):
    N, P, H, W, Q, k, d, pad, dil, adj, bias = shape
    rng = np.random.default_rng(abs(hash(shape)) % 99991)
    x = rng.standard_normal((N, P, H, W)).astype(np.float32)
    w = (rng.standard_normal((P, Q, k, k)) * np.sqrt(2.0 / (P * k * k))).astype(np.float32)
    b = rng.uniform(-0.5, 0.5, Q).astype(np.float32) if bias else None
    geo = (d, d, pad, pad, dil, dil, adj, adj)
    OH, OW = ref64.fullconv_out_size(H, W, k, k, *geo)
    gy = rng.standard_normal((N, Q, OH, OW)).astype(np.float32)
    gw0 = rng.standard_normal((P, Q, k, k)).astype(np.float32)
    gb0 = rng.standard_normal(Q).astype(np.float32) if bias else None
    y, gx, gw, gb = run_all(F, x, w, b, gy, gw0, gb0, geo, 0.75)
    assert y.shape == (N, Q, OH, OW)
    assert rel_err(y, ref64.fullconv_forward(x, w, b, *geo)) < TOL
    assert rel_err(gx, ref64.fullconv_grad_input(gy, w, H, W, *geo)) < TOL
    rgw, rgb = ref64.fullconv_acc_grad(x, gy, gw0, gb0, *geo, scale=0.75)
    assert rel_err(gw, rgw) < TOL
    if bias:
        assert rel_err(gb, rgb) < TOL


def test_full_conv_is_the_adjoint_of_convolution(F):
    # <fullconv(x, W), z> == <x, conv(z, W)> with the same weight array read as [K = P][C = Q]; decoder-sized planes
    g = torch.Generator(device="cuda").manual_seed(4)
    N, P, Q, H, k, d, pad = 8, 128, 64, 28, 4, 2, 1
    x = torch.randn((N, P, H, H), device="cuda", generator=g)
    w = torch.randn((P, Q, k, k), device="cuda", generator=g) * 0.05
    y = F.full_conv_forward(x, w, None, d, d, pad, pad)
    assert tuple(y.shape) == (N, Q, 2 * H, 2 * H)
    z = torch.randn(y.shape, device="cuda", generator=g)
    cz = F.convmm_forward(z, w, None, d, d, pad, pad)
    a = float((y.double() * z.double()).sum())
    b = float((x.double() * cz.double()).sum())
    assert abs(a - b) < 1e-6 * float((y.double().abs() * z.double().abs()).sum())
    assert torch.equal(F.full_conv_grad_input(z, w, H, H, d, d, pad, pad), cz)


def test_full_conv_errors(F):
    from cunn_b200 import CunnError
    x = torch.zeros((1, 2, 8, 8), device="cuda")
    w = torch.zeros((2, 3, 3, 3), device="cuda")
    with pytest.raises(CunnError, match="output padding must be smaller than either stride or dilation"):
        F.full_conv_forward(x, w, None, 2, 2, 1, 1, 1, 1, 2, 2)
    with pytest.raises(CunnError, match="Output size is too small"):
        F.full_conv_forward(torch.zeros((1, 2, 1, 1), device="cuda"), w, None, 1, 1, 2, 2)
    assert tuple(F.full_conv_forward(torch.zeros((0, 2, 8, 8), device="cuda"), w, None, 2, 2, 1, 1).shape) == (0, 3, 15, 15)


def test_thnn_full_convolution_entry_points(ref64):
    from cunn_b200.thnn import THNN
    rng = np.random.default_rng(13)
    N, P, H, W, Q, k, d, pad, adj = 2, 6, 7, 5, 9, 3, 2, 1, 1
    x = rng.standard_normal((N, P, H, W)).astype(np.float32)
    w = rng.standard_normal((P, Q, k, k)).astype(np.float32) * 0.2
    b = rng.standard_normal(Q).astype(np.float32)
    geo = (d, d, pad, pad, 1, 1, adj, adj)
    OH, OW = ref64.fullconv_out_size(H, W, k, k, *geo)
    gy = rng.standard_normal((N, Q, OH, OW)).astype(np.float32)
    th = THNN()
    try:
        y = th.SpatialFullDilatedConvolution_updateOutput(dev(x), dev(w), dev(b), k, k, d, d, pad, pad, 1, 1, adj, adj)
        assert tuple(y.shape) == (N, Q, OH, OW)
        assert rel_err(host(y), ref64.fullconv_forward(x, w, b, *geo)) < TOL
        y2 = th.SpatialFullConvolution_updateOutput(dev(x), dev(w), dev(b), k, k, d, d, pad, pad, adj, adj)
        assert torch.equal(y2, y)
        gx = th.SpatialFullDilatedConvolution_updateGradInput(dev(x), dev(gy), dev(w), k, k, d, d, pad, pad, 1, 1, adj, adj)
        assert rel_err(host(gx), ref64.fullconv_grad_input(gy, w, H, W, *geo)) < TOL
        gw, gb = dev(np.zeros_like(w)), dev(np.zeros_like(b))
        th.SpatialFullDilatedConvolution_accGradParameters(dev(x), dev(gy), gw, gb, k, k, d, d, pad, pad, 1, 1, adj, adj, 0.5)
        rgw, rgb = ref64.fullconv_acc_grad(x, gy, np.zeros_like(w), np.zeros_like(b), *geo, scale=0.5)
        assert rel_err(host(gw), rgw) < TOL and rel_err(host(gb), rgb) < TOL
        # 3-D (unbatched) input gives a 3-D output, as in the reference
        y3 = th.SpatialFullDilatedConvolution_updateOutput(dev(x[0]), dev(w), dev(b), k, k, d, d, pad, pad, 1, 1, adj, adj)
        assert tuple(y3.shape) == (Q, OH, OW) and rel_err(host(y3), host(y)[0]) < 1e-6
        with pytest.raises(Exception, match="output padding must be smaller"):
            th.SpatialFullConvolution_updateOutput(dev(x), dev(w), dev(b), k, k, d, d, pad, pad, 2, 2)
    finally:
        th.close()
