"""SpatialConvolutionMM: tcgen05 implicit-GEMM kernels (flat C ABI) against the CPU oracle and the committed
PyTorch-CPU fixtures.  GEMM-path tolerance 1e-4 (element-wise relative error with a 1 % floor)."""
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


def make_case(seed, N, C, H, W, K, k, d, pad, bias=True):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((N, C, H, W)).astype(np.float32)
    w = (rng.standard_normal((K, C, k, k)) * np.sqrt(2.0 / (C * k * k))).astype(np.float32)
    b = rng.uniform(-0.5, 0.5, K).astype(np.float32) if bias else None
    oH, oW = (H + 2 * pad - k) // d + 1, (W + 2 * pad - k) // d + 1
    gy = rng.standard_normal((N, K, oH, oW)).astype(np.float32)
    gw0 = rng.standard_normal((K, C, k, k)).astype(np.float32)
    gb0 = rng.standard_normal(K).astype(np.float32) if bias else None
    return x, w, b, gy, gw0, gb0


def run_all(F, x, w, b, gy, gw0, gb0, d, pad, scale):
    H, W = x.shape[2:]
    y = F.convmm_forward(dev(x), dev(w), None if b is None else dev(b), d, d, pad, pad)
    gx = F.convmm_grad_input(dev(gy), dev(w), H, W, d, d, pad, pad)
    gw = dev(gw0)
    gb = None if gb0 is None else dev(gb0)
    F.convmm_acc_grad(dev(x), dev(gy), gw, gb, d, d, pad, pad, scale)
    torch.cuda.synchronize()
    return host(y), host(gx), host(gw), None if gb is None else host(gb)


def check_against_oracle(ref64, F, x, w, b, gy, gw0, gb0, d, pad, scale):
    H, W = x.shape[2:]
    y, gx, gw, gb = run_all(F, x, w, b, gy, gw0, gb0, d, pad, scale)
    assert rel_err(y, ref64.convmm_forward(x, w, b, d, d, pad, pad)) < TOL
    assert rel_err(gx, ref64.convmm_grad_input(gy, w, H, W, d, d, pad, pad)) < TOL
    rgw, rgb = ref64.convmm_acc_grad(x, gy, gw0, gb0, d, d, pad, pad, scale)
    assert rel_err(gw, rgw) < TOL
    if gb0 is not None:
        assert rel_err(gb, rgb) < TOL


@pytest.mark.parametrize("name", ["convmm_3x3", "convmm_1x1", "convmm_s2"])
def test_convmm_golden(F, name):
    g = golden(name)
    K, k, d, pad, has_b = [int(v) for v in g["params"]]
    y, gx, gw, gb = run_all(F, g["x"], g["w"], g["b"] if has_b else None, g["gy"], g["gw0"],
                            g["gb0"] if has_b else None, d, pad, float(g["scale"]))
    assert rel_err(y, g["y"]) < TOL
    assert rel_err(gx, g["gx"]) < TOL
    assert rel_err(gw, g["gw"]) < TOL
    if has_b:
        assert rel_err(gb, g["gb"]) < TOL


@pytest.mark.parametrize("shape", [
    # N, C, H, W, K, k, d, pad, bias
    (2, 16, 14, 14, 32, 3, 1, 1, True),      # small 3x3
    (3, 64, 14, 14, 256, 1, 1, 0, True),     # 1x1, several N tiles
    (2, 3, 32, 32, 32, 3, 2, 1, True),       # MobileNet stem geometry (reduced): Kd = 27
    (2, 32, 28, 28, 64, 1, 1, 0, True),      # MobileNet pointwise geometry
    (4, 256, 7, 7, 256, 1, 1, 0, False),     # 7x7 planes (49 pixels: no 16-byte alignment)
    (2, 24, 9, 11, 40, 3, 1, 1, True),       # odd sizes, K not a multiple of 8
    (1, 8, 12, 12, 300, 3, 1, 0, True),      # pad 0, K > 256
    (2, 5, 10, 10, 7, 5, 2, 2, True),        # 5x5 stride 2 (generic k decomposition, gather dgrad)
    (2, 130, 6, 6, 20, 3, 1, 1, True),       # Kd = 1170: many k-blocks, ragged tail
    (9, 4, 5, 5, 4, 1, 2, 0, True),          # 1x1 stride 2
    (2, 3, 20, 20, 8, 7, 2, 3, True),        # 7x7 (49 taps): the kernel for more than 32 taps
    (2, 6, 12, 12, 10, 7, 1, 3, False),      # 7x7 stride 1: tensor-core input gradient of that kernel
    (3, 3, 17, 19, 32, 3, 1, 1, True),       # first-layer kernels: stride 1, odd sizes
    (2, 3, 16, 16, 32, 3, 2, 0, False),      # first-layer kernels: no padding, no bias
    (80, 3, 64, 64, 32, 3, 2, 1, True),      # first-layer kernels: more pixel tiles than CTAs
    (8, 32, 56, 56, 64, 1, 1, 0, True),      # pointwise, one k-block, more tiles than SMs (persistent loop)
    (16, 128, 28, 28, 128, 1, 1, 0, True),   # pointwise, four k-blocks, two accumulator sets
    (2, 1024, 14, 14, 192, 1, 1, 0, False),  # pointwise, long reduction, ragged second column tile
    (2, 30, 6, 6, 50, 1, 1, 0, True),        # pointwise, channel counts not multiples of 4
    (3, 20, 5, 5, 36, 1, 1, 0, True),        # pointwise, 25-pixel planes (scalar loads)
    (40, 512, 7, 7, 96, 1, 1, 0, True),      # pointwise, 49-pixel planes, several row tiles
    (64, 1024, 1, 1, 1000, 1, 1, 0, True),   # classifier geometry: one pixel per image
])
def test_convmm_shapes(F, ref64, shape):
    N, C, H, W, K, k, d, pad, bias = shape
    case = make_case(abs(hash(shape)) % 99991, N, C, H, W, K, k, d, pad, bias)
    check_against_oracle(ref64, F, *case, d, pad, 0.75)


@pytest.fixture(params=[1, 0], ids=["tma", "element-copy"])
def pointwise_loader(request):
    """1x1 convolutions have two operand loaders: tensor-map copies (aligned tensors) and element copies."""
    from cunn_b200._lib import lib
    lib.cunn_b200_convmm_set_tma(request.param)
    yield request.param
    lib.cunn_b200_convmm_set_tma(1)


@pytest.mark.parametrize("shape", [
    # N, C, H, W, K, bias
    (3, 64, 14, 14, 256, True),      # 196-pixel planes: 7 groups of 32, the last one 4 pixels wide; two column tiles
    (5, 96, 14, 14, 40, False),      # row tiles that end inside an image and past the last image; K < 64
    (2, 32, 28, 28, 64, True),       # 784 pixels: 24.5 groups
    (3, 32, 56, 56, 64, True),       # 3136 = 98 x 32 pixels: bulk-store epilogue, one k-block
    (2, 256, 32, 32, 200, True),     # 1024-pixel planes, 8 k-blocks, ragged column tile
    (16, 128, 28, 28, 128, True),    # four k-blocks, two accumulator sets, several tiles per CTA
    (4, 1024, 14, 14, 256, False),   # long reduction: four accumulators, one set
    (3, 40, 64, 64, 24, True),       # 4096-pixel planes, narrow column tile (32): per-column bulk stores
    (2, 64, 40, 40, 128, False),     # 1600-pixel planes: tiles that cross an image boundary in the bulk-store epilogue
    (6, 100, 6, 6, 20, True),        # 36-pixel planes (2 groups per image), C not a multiple of 32
    (2, 36, 2, 2, 24, True),         # 4-pixel planes
    (130, 64, 2, 4, 32, True),       # many tiny images: more groups than one wave of row tiles
])
def test_convmm_pointwise_both_loaders(F, ref64, shape, pointwise_loader):
    N, C, H, W, K, bias = shape
    case = make_case(abs(hash(shape)) % 99991, N, C, H, W, K, 1, 1, 0, bias)
    check_against_oracle(ref64, F, *case, 1, 0, 0.75)


def test_convmm_depthwise_equivalence(F):
    # The reference's own depthwise test (test.lua:6602-6661): depthwise forward == per-channel
    # SpatialConvolution(1, m, 3,3,1,1,1,1) on weight[:, c] / bias[:, c]; n=3, m=4, 28x28, batch 3, within 1e-5.
    rng = np.random.default_rng(7)
    n, m = 3, 4
    x = rng.random((3, n, 28, 28)).astype(np.float32)
    w = rng.random((m, n, 3, 3)).astype(np.float32)
    b = rng.random((m, n)).astype(np.float32)
    y = host(F.dwconv_forward(dev(x), dev(w), dev(b), 1, 1, 1, 1))
    for c in range(n):
        yc = host(F.convmm_forward(dev(x[:, c:c + 1]), dev(w[:, c:c + 1]), dev(b[:, c]), 1, 1, 1, 1))
        assert np.max(np.abs(y[:, c * m:(c + 1) * m] - yc)) < 1e-5


def test_convmm_empty_batch_and_errors(F):
    from cunn_b200 import CunnError
    x = torch.empty((0, 4, 8, 8), device="cuda")
    w = torch.ones((8, 4, 3, 3), device="cuda")
    assert tuple(F.convmm_forward(x, w, None, 1, 1, 1, 1).shape) == (0, 8, 8, 8)
    with pytest.raises(CunnError, match="Output size is too small"):
        F.convmm_forward(torch.zeros((1, 4, 2, 2), device="cuda"), torch.zeros((8, 4, 5, 5), device="cuda"), None,
                         1, 1, 0, 0, out=torch.zeros(1, device="cuda"))


@pytest.mark.parametrize("cfg", [(128, 256, 256, 14, 3, 1), (128, 1024, 256, 14, 1, 0)])
def test_convmm_full_size_adjoint_identities(F, cfg):
    # The two benchmarked GEMM convolutions at full size (a size-independent property beside the whole-tensor
    # oracle comparison of test_full_size_gpu.py): the three passes are the three partial
    # derivatives of one trilinear form, so <conv(x, W), gy> == <x, dgrad(gy, W)> == <wgrad(x, gy), W>, and the
    # bias gradient is the plain sum of gy.  Inner products are taken in fp64; 1e-4 is the GEMM-path bar.
    N, C, K, HW, k, pad = cfg
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn((N, C, HW, HW), device="cuda", generator=g)
    w = torch.randn((K, C, k, k), device="cuda", generator=g) * (2.0 / (C * k * k)) ** 0.5
    gy = torch.randn((N, K, HW, HW), device="cuda", generator=g)
    y = F.convmm_forward(x, w, None, 1, 1, pad, pad)
    gx = F.convmm_grad_input(gy, w, HW, HW, 1, 1, pad, pad)
    gw, gb = torch.zeros_like(w), torch.zeros(K, device="cuda")
    F.convmm_acc_grad(x, gy, gw, gb, 1, 1, pad, pad, 1.0)
    a = float((y.double() * gy.double()).sum())
    b = float((x.double() * gx.double()).sum())
    c = float((gw.double() * w.double()).sum())
    scale = float((y.double().abs() * gy.double().abs()).sum())
    assert abs(a - b) < 1e-6 * scale and abs(a - c) < 1e-6 * scale
    ref_gb = gy.double().sum((0, 2, 3))
    assert float((gb.double() - ref_gb).abs().max()) < 1e-4 * float(ref_gb.abs().max())
    # linearity in x at full size: conv(2 x1 - 3 x2) == 2 conv(x1) - 3 conv(x2)
    x2 = torch.randn((N, C, HW, HW), device="cuda", generator=g)
    lhs = F.convmm_forward(2 * x - 3 * x2, w, None, 1, 1, pad, pad)
    rhs = 2 * y - 3 * F.convmm_forward(x2, w, None, 1, 1, pad, pad)
    assert float((lhs - rhs).abs().max()) < 1e-4 * float(rhs.abs().max())
