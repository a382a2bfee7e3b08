"""Depthwise convolution: CUDA kernels (through the flat C ABI) against the CPU oracle and the
committed PyTorch-CPU fixtures.  Tolerances: forward 1e-5, gradients 1e-4 (element-wise relative
error with a 1 % floor, see conftest.rel_err)."""
import numpy as np
import pytest

from conftest import golden, rel_err, norm_err

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

FWD_TOL = 1e-5
GRAD_TOL = 1e-4

# (C, H=W, stride) of the 13 depthwise layers of MobileNetV1
MOBILENET_DW = [(32, 112, 1), (64, 112, 2), (128, 56, 1), (128, 56, 2), (256, 28, 1), (256, 28, 2),
                (512, 14, 1), (512, 14, 2), (1024, 7, 1)]


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.detach().cpu().numpy()


def make_case(seed, N, C, H, W, M, k, d, pad, bias=True):
    rng = np.random.default_rng(seed)
    x = rng.uniform(-1, 1, (N, C, H, W)).astype(np.float32)
    bound = 1.0 / np.sqrt(k * k)
    w = rng.uniform(-bound, bound, (M, C, k, k)).astype(np.float32)
    b = rng.uniform(-bound, bound, (M, C)).astype(np.float32) if bias else None
    oH, oW = (H + 2 * pad - k) // d + 1, (W + 2 * pad - k) // d + 1
    gy = rng.standard_normal((N, C * M, oH, oW)).astype(np.float32)
    gw0 = rng.standard_normal((M, C, k, k)).astype(np.float32)
    gb0 = rng.standard_normal((M, C)).astype(np.float32) if bias else None
    return x, w, b, gy, gw0, gb0


def run_all(F, x, w, b, gy, gw0, gb0, d, pad, scale):
    H, W = x.shape[2:]
    y = F.dwconv_forward(dev(x), dev(w), None if b is None else dev(b), d, d, pad, pad)
    gx = F.dwconv_grad_input(dev(gy), dev(w), H, W, d, d, pad, pad)
    gw = dev(gw0)
    gb = None if gb0 is None else dev(gb0)
    F.dwconv_acc_grad(dev(x), dev(gy), gw, gb, d, d, pad, pad, scale)
    torch.cuda.synchronize()
    return host(y), host(gx), host(gw), None if gb is None else host(gb)


def check_against_oracle(ref64, F, x, w, b, gy, gw0, gb0, d, pad, scale):
    H, W = x.shape[2:]
    y, gx, gw, gb = run_all(F, x, w, b, gy, gw0, gb0, d, pad, scale)
    assert rel_err(y, ref64.dwconv_forward(x, w, b, d, d, pad, pad)) < FWD_TOL
    assert rel_err(gx, ref64.dwconv_grad_input(gy, w, H, W, d, d, pad, pad)) < GRAD_TOL
    rgw, rgb = ref64.dwconv_acc_grad(x, gy, gw0, gb0, d, d, pad, pad, scale)
    assert rel_err(gw, rgw) < GRAD_TOL
    if gb0 is not None:
        assert rel_err(gb, rgb) < GRAD_TOL


@pytest.fixture(scope="module")
def F():
    import cunn_b200.functional as F
    from cunn_b200 import _lib
    yield F
    assert _lib.device_status() == 0


@pytest.mark.parametrize("name", ["dwconv_m4", "dwconv_s1", "dwconv_s2", "dwconv_s2_odd", "dwconv_k5", "dwconv_w28"])
def test_dwconv_golden(F, name):
    g = golden(name)
    M, k, d, pad, has_b = [int(v) for v in g["params"]]
    y, gx, gw, gb = run_all(F, g["x"], g["w"], g["b"] if has_b else None, g["gy"], g["gw0"],
                            g["gb0"] if has_b else None, d, pad, float(g["scale"]))
    assert rel_err(y, g["y"]) < FWD_TOL
    assert rel_err(gx, g["gx"]) < GRAD_TOL
    assert rel_err(gw, g["gw"]) < GRAD_TOL
    if has_b:
        assert rel_err(gb, g["gb"]) < GRAD_TOL


def test_dwconv_config1(F, ref64):
    # the single-layer configuration: N=8, C=32, 56x56, 3x3 s1 p1 m1; scale 1 and 0.5 on non-zero gradWeight
    case = make_case(1234, 8, 32, 56, 56, 1, 3, 1, 1)
    check_against_oracle(ref64, F, *case, 1, 1, 1.0)
    check_against_oracle(ref64, F, *case, 1, 1, 0.5)


@pytest.mark.parametrize("C,HW,stride", MOBILENET_DW)
@pytest.mark.parametrize("N", [1, 5])
def test_dwconv_mobilenet_layers(F, ref64, C, HW, stride, N):
    case = make_case(C * 1000 + HW + N, N, C, HW, HW, 1, 3, stride, 1)
    check_against_oracle(ref64, F, *case, stride, 1, 1.0)


@pytest.mark.parametrize("shape", [
    # N, C, H, W, M, k, d, pad, bias
    (2, 3, 28, 28, 4, 3, 1, 1, True),     # the reference's own test shape (m = 4)
    (3, 5, 9, 11, 1, 3, 1, 1, True),      # odd sizes -> scalar fast path / generic
    (2, 6, 10, 13, 1, 3, 2, 1, False),    # odd width, stride 2
    (2, 4, 13, 12, 1, 3, 2, 1, True),     # odd height, stride 2
    (1, 7, 7, 7, 1, 3, 1, 1, True),       # channel count not divisible by 4 with 7x7 planes
    (2, 4, 16, 16, 1, 3, 1, 0, True),     # pad 0 -> generic
    (2, 4, 15, 17, 2, 5, 3, 2, True),     # 5x5 stride 3
    (1, 2, 6, 6, 1, 1, 1, 0, True),       # 1x1
    (2, 8, 120, 120, 1, 3, 1, 1, True),   # row-banded tiles, several bands
    (2, 8, 120, 120, 1, 3, 2, 1, True),
    (3, 4, 1, 1, 1, 3, 1, 1, True),       # 1x1 image
    (2, 16, 2, 2, 1, 3, 2, 1, True),
    (65, 8, 14, 14, 1, 3, 1, 1, True),    # more images than splits
])
def test_dwconv_shapes(F, ref64, shape):
    N, C, H, W, M, k, d, pad, bias = shape
    case = make_case(hash(shape) % 100000, N, C, H, W, M, k, d, pad, bias)
    check_against_oracle(ref64, F, *case, d, pad, 0.75)


def test_dwconv_generic_matches_fast(F, ref64):
    # Pointers that are not 16-byte aligned cannot be fetched by bulk copies, so the same layer runs on the
    # shape-generic kernels when its tensors start 4 bytes into their buffers.
    case = make_case(99, 3, 16, 28, 28, 1, 3, 2, 1)
    x, w, b, gy, gw0, gb0 = case
    fast = run_all(F, *case, 2, 1, 1.0)

    def shifted(a):
        buf = torch.empty(a.size + 1, device="cuda")
        v = buf[1:].view(a.shape)
        v.copy_(torch.from_numpy(a))
        assert v.data_ptr() % 16 == 4
        return v

    xs, gys = shifted(x), shifted(gy)
    y = F.dwconv_forward(xs, dev(w), dev(b), 2, 2, 1, 1)
    gx = F.dwconv_grad_input(gys, dev(w), 28, 28, 2, 2, 1, 1)
    gw, gb = dev(gw0), dev(gb0)
    F.dwconv_acc_grad(xs, gys, gw, gb, 2, 2, 1, 1, 1.0)
    for a, b_ in zip(fast, (host(y), host(gx), host(gw), host(gb))):
        assert rel_err(a, b_) < 1e-5


def test_dwconv_empty_batch(F):
    x = torch.empty((0, 4, 8, 8), device="cuda")
    w = torch.ones((1, 4, 3, 3), device="cuda")
    y = F.dwconv_forward(x, w, None, 1, 1, 1, 1)
    assert tuple(y.shape) == (0, 4, 8, 8)
    gw = torch.full((1, 4, 3, 3), 2.0, device="cuda")
    F.dwconv_acc_grad(x, y, gw, None, 1, 1, 1, 1, 1.0)
    assert torch.all(gw == 2.0)


def test_dwconv_rejects_bad_arguments(F):
    from cunn_b200 import CunnError
    x = torch.zeros((1, 2, 2, 2), device="cuda")
    w = torch.zeros((1, 2, 5, 5), device="cuda")
    with pytest.raises(CunnError, match="Output size is too small"):
        F.dwconv_forward(x, w, None, 1, 1, 0, 0, out=torch.zeros(1, device="cuda"))
    w3 = torch.zeros((1, 2, 3, 3), device="cuda")
    with pytest.raises(CunnError, match="stride should be greater than zero"):
        F.dwconv_forward(x, w3, None, 0, 0, 1, 1, out=torch.zeros(1, device="cuda"))


def test_dwconv_unaligned_pointers_take_generic_path(F, ref64):
    x, w, b, gy, gw0, gb0 = make_case(5, 2, 4, 12, 12, 1, 3, 1, 1)
    buf = torch.zeros(x.size + 1, device="cuda")
    xd = buf[1:].view(x.shape)            # 4-byte aligned only
    xd.copy_(dev(x))
    y = F.dwconv_forward(xd, dev(w), dev(b), 1, 1, 1, 1)
    assert rel_err(host(y), ref64.dwconv_forward(x, w, b, 1, 1, 1, 1)) < FWD_TOL


def test_dwconv_linearity_full_size(F):
    # Size-independent property at a MobileNetV1 depthwise layer at batch 64 (C=128, 56x56): conv is linear in x
    # and in gy, and <gy, conv(x)> == <dgrad(gy), x> (adjointness ties forward and input gradient).
    torch.manual_seed(0)
    N, C, HW = 64, 128, 56
    for stride in (1, 2):
        x1 = torch.rand((N, C, HW, HW), device="cuda") * 2 - 1
        x2 = torch.rand((N, C, HW, HW), device="cuda") * 2 - 1
        w = (torch.rand((1, C, 3, 3), device="cuda") * 2 - 1) / 3
        y1 = F.dwconv_forward(x1, w, None, stride, stride, 1, 1)
        y2 = F.dwconv_forward(x2, w, None, stride, stride, 1, 1)
        y12 = F.dwconv_forward(x1 + 2 * x2, w, None, stride, stride, 1, 1)
        assert float((y12 - (y1 + 2 * y2)).abs().max()) < 1e-5
        gy = torch.randn_like(y1)
        gx = F.dwconv_grad_input(gy, w, HW, HW, stride, stride, 1, 1)
        lhs = float((gy.double() * y1.double()).sum())
        rhs = float((gx.double() * x1.double()).sum())
        assert abs(lhs - rhs) < 1e-6 * (abs(lhs) + 1e3)
        # <gw, w'> == <gy, conv_{w'}(x)>: parameter gradient is the adjoint in w
        gw = torch.zeros_like(w)
        gb = torch.zeros((1, C), device="cuda")
        F.dwconv_acc_grad(x1, gy, gw, gb, stride, stride, 1, 1, 1.0)
        lhs = float((gw.double() * w.double()).sum())
        rhs = float((gy.double() * y1.double()).sum())
        assert abs(lhs - rhs) < 1e-6 * (abs(rhs) + 1e3)
        assert rel_err(host(gb).ravel(), host(gy.double().sum(dim=(0, 2, 3)).float())) < GRAD_TOL


def test_dwconv_acc_grad_deterministic_mode(F, ref64):
    # cunn_b200_set_deterministic(1): the ticketed fixed-order reduction; results are bit-identical from run
    # to run and equal the default (atomic) mode within the gradient tolerance
    from cunn_b200._lib import lib
    x, w, b, gy, gw0, gb0 = make_case(31, 9, 64, 28, 28, 1, 3, 1, 1)
    xd, gyd = dev(x), dev(gy)
    rgw, rgb = ref64.dwconv_acc_grad(x, gy, gw0, gb0, 1, 1, 1, 1, 0.5)
    assert lib.cunn_b200_get_deterministic() == 0
    gw, gb = dev(gw0), dev(gb0)
    F.dwconv_acc_grad(xd, gyd, gw, gb, 1, 1, 1, 1, 0.5)
    assert rel_err(host(gw), rgw) < GRAD_TOL and rel_err(host(gb), rgb) < GRAD_TOL
    lib.cunn_b200_set_deterministic(1)
    try:
        first = None
        for _ in range(5):
            gw, gb = dev(gw0), dev(gb0)
            F.dwconv_acc_grad(xd, gyd, gw, gb, 1, 1, 1, 1, 0.5)
            cur = (host(gw), host(gb))
            assert rel_err(cur[0], rgw) < GRAD_TOL and rel_err(cur[1], rgb) < GRAD_TOL
            if first is None:
                first = cur
            assert np.array_equal(first[0], cur[0]) and np.array_equal(first[1], cur[1])
    finally:
        lib.cunn_b200_set_deterministic(0)
