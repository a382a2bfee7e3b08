"""Max pooling and batch normalisation: CUDA kernels (flat C ABI) against the CPU oracle and the committed
PyTorch-CPU fixtures.  Pooling indices must match exactly; values/forward 1e-5, gradients 1e-4."""
import numpy as np
import pytest

from conftest import golden, rel_err

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

FWD_TOL = 1e-5
GRAD_TOL = 1e-4


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


@pytest.fixture(params=[1, 2], ids=["default-kernels", "grouped-kernels"])
def grouped_mode(request):
    """Batch norm has two kernel families: two launches (statistics, then normalise) and one launch that walks
    groups of channels so that the second read comes from L2.  Mode 2 routes every shape the latter applies to
    through it, forward and backward; mode 1 is the library's default choice."""
    from cunn_b200._lib import lib
    lib.cunn_b200_batchnorm_set_grouped(request.param)
    yield request.param
    lib.cunn_b200_batchnorm_set_grouped(1)


# ---------------------------------------------------------------- max pooling
@pytest.mark.parametrize("name", ["maxpool_3s2p1", "maxpool_ceil", "maxpool_ties", "maxpool_2s2"])
def test_maxpool_golden(F, ref64, name):
    g = golden(name)
    k, d, pad, ceil_mode = [int(v) for v in g["params"]]
    y, ind = F.maxpool_forward(dev(g["x"]), k, k, d, d, pad, pad, bool(ceil_mode))
    assert np.array_equal(host(y), g["y"])
    assert np.array_equal(host(ind), g["ind0"] + ref64.index_base)
    H, W = g["x"].shape[2:]
    gx = F.maxpool_backward(dev(g["gy"]), ind, H, W, k, k, d, d, pad, pad, bool(ceil_mode))
    assert rel_err(host(gx), g["gx"]) < 1e-5


@pytest.mark.parametrize("shape", [
    # N, C, H, W, k, d, pad, ceil, ties
    (2, 3, 112, 112, 3, 2, 1, False, False),   # fast path (geometry of the benchmarked pooling layer)
    (2, 5, 32, 48, 3, 2, 1, False, True),      # fast path with many ties
    (3, 2, 31, 40, 3, 2, 1, False, True),      # fast path, odd height
    (2, 3, 112, 112, 3, 2, 1, True, False),    # ceil mode changes the output size -> generic
    (2, 4, 17, 19, 3, 2, 1, True, True),
    (1, 3, 20, 20, 2, 2, 0, False, True),
    (2, 2, 15, 15, 3, 1, 1, False, True),
    (2, 2, 14, 14, 5, 3, 2, True, False),
    (1, 1, 3, 3, 3, 2, 1, False, False),
    (4, 8, 56, 56, 3, 2, 1, False, False),
])
def test_maxpool_shapes(F, ref64, shape):
    N, C, H, W, k, d, pad, ceil_mode, ties = shape
    rng = np.random.default_rng(abs(hash(shape)) % 99991)
    x = rng.standard_normal((N, C, H, W)).astype(np.float32)
    if ties:
        x = np.round(x * 2) / 2
    ry, rind = ref64.maxpool_forward(x, k, k, d, d, pad, pad, ceil_mode)
    y, ind = F.maxpool_forward(dev(x), k, k, d, d, pad, pad, ceil_mode)
    assert tuple(y.shape) == ry.shape
    assert np.array_equal(host(y), ry)
    assert int((host(ind) != rind).sum()) == 0          # indices bit-exact
    gy = rng.standard_normal(ry.shape).astype(np.float32)
    gx = F.maxpool_backward(dev(gy), ind, H, W, k, k, d, d, pad, pad, ceil_mode)
    assert rel_err(host(gx), ref64.maxpool_backward(gy, rind, H, W, k, k, d, d, pad, pad)) < 1e-5  # fp32 sums of up to k*k gradients


def test_maxpool_nan_and_inf_windows(F, ref64):
    # NaN / -inf never win the strict compare; an all-NaN window stores index -1 + base and -FLT_MAX
    x = np.random.default_rng(3).standard_normal((1, 2, 16, 16)).astype(np.float32)
    x[0, 0, :5, :5] = np.nan
    x[0, 1, 4:9, 8:] = -np.inf
    x[0, 1, 0, 0] = np.inf
    for k, d, pad in ((3, 2, 1), (2, 2, 0)):
        ry, rind = ref64.maxpool_forward(x, k, k, d, d, pad, pad, False)
        y, ind = F.maxpool_forward(dev(x), k, k, d, d, pad, pad, False)
        assert np.array_equal(host(ind), rind)
        assert np.array_equal(host(y), ry)
    assert rind.min() >= -1 + ref64.index_base


def test_maxpool_rejects_bad_arguments(F):
    from cunn_b200 import CunnError
    x = torch.zeros((1, 1, 8, 8), device="cuda")
    with pytest.raises(CunnError, match="pad should be smaller than half of kernel size"):
        F.maxpool_forward(x, 2, 2, 2, 2, 2, 2, out=torch.zeros(1, device="cuda"),
                          indices=torch.zeros(1, dtype=torch.int64, device="cuda"))


def test_maxpool_full_size_properties(F):
    # the benchmarked geometry at reduced batch (N=32): the stored index must point at the stored value,
    # and backward must conserve the gradient mass: sum(gx) == sum(gy).
    torch.manual_seed(0)
    x = torch.randn((32, 64, 112, 112), device="cuda") * 2 + 0.5
    y, ind = F.maxpool_forward(x, 3, 3, 2, 2, 1, 1)
    from cunn_b200._lib import lib
    flat = x.view(32 * 64, -1)
    picked = torch.gather(flat, 1, (ind.view(32 * 64, -1) - 1))
    assert torch.equal(picked.view_as(y), y)
    gy = torch.randn_like(y)
    gx = F.maxpool_backward(gy, ind, 112, 112, 3, 3, 2, 2, 1, 1)
    assert abs(float(gx.double().sum()) - float(gy.double().sum())) < 1e-6 * float(gy.double().abs().sum())


# ---------------------------------------------------------------- batch normalisation
def bn_check(F, ref64, x, w, b, rm0, rv0, gy, momentum, eps, scale, gw0=None, gb0=None):
    C = x.shape[1]
    # training forward
    ry, rrm, rrv, rsm, rss = ref64.bn_forward(x, w, b, rm0, rv0, True, momentum, eps)
    rm, rv = dev(rm0), dev(rv0)
    y, sm, ss = F.batchnorm_forward(dev(x), None if w is None else dev(w), None if b is None else dev(b), rm, rv,
                                    True, momentum, eps)
    assert rel_err(host(y), ry) < FWD_TOL
    assert rel_err(host(sm), rsm) < FWD_TOL and rel_err(host(ss), rss) < FWD_TOL
    assert rel_err(host(rm), rrm) < FWD_TOL and rel_err(host(rv), rrv) < FWD_TOL
    # training backward (accumulating into non-zero gradWeight / gradBias with scale)
    gw0 = np.zeros(C, np.float32) if gw0 is None else gw0
    gb0 = np.zeros(C, np.float32) if gb0 is None else gb0
    rgx, rgw, rgb = ref64.bn_backward(x, gy, w, rrm, rrv, rsm, rss, True, scale, eps, gw=gw0, gb=gb0)
    gw, gb = dev(gw0), dev(gb0)
    gx = F.batchnorm_backward(dev(x), dev(gy), None if w is None else dev(w), rm, rv, sm, ss, True, scale, eps,
                              grad_weight=gw, grad_bias=gb)
    assert rel_err(host(gx), rgx) < GRAD_TOL
    assert rel_err(host(gw), rgw) < GRAD_TOL and rel_err(host(gb), rgb) < GRAD_TOL
    # inference forward / backward on the given running statistics
    ry, rm2, rv2, _, _ = ref64.bn_forward(x, w, b, rm0, rv0, False, momentum, eps)
    rm, rv = dev(rm0), dev(rv0)
    y, _, _ = F.batchnorm_forward(dev(x), None if w is None else dev(w), None if b is None else dev(b), rm, rv,
                                  False, momentum, eps)
    assert rel_err(host(y), ry) < FWD_TOL
    assert np.array_equal(host(rm), rm0) and np.array_equal(host(rv), rv0)   # untouched in inference
    rgx, rgw, rgb = ref64.bn_backward(x, gy, w, rm0, rv0, rsm, rss, False, scale, eps, gw=gw0, gb=gb0)
    gw, gb = dev(gw0), dev(gb0)
    gx = F.batchnorm_backward(dev(x), dev(gy), None if w is None else dev(w), rm, rv, sm, ss, False, scale, eps,
                              grad_weight=gw, grad_bias=gb)
    assert rel_err(host(gx), rgx) < GRAD_TOL
    assert rel_err(host(gw), rgw) < GRAD_TOL and rel_err(host(gb), rgb) < GRAD_TOL
    # gradInput only / parameters only (the reference lets any of the three be NULL)
    gx_only = F.batchnorm_backward(dev(x), dev(gy), None if w is None else dev(w), rm, rv, sm, ss, True, scale, eps)
    rgx_t, _, _ = ref64.bn_backward(x, gy, w, rrm, rrv, rsm, rss, True, scale, eps)
    assert rel_err(host(gx_only), rgx_t) < GRAD_TOL
    gw = dev(gw0)
    assert F.batchnorm_backward(dev(x), dev(gy), None if w is None else dev(w), rm, rv, sm, ss, True, scale, eps,
                                grad_weight=gw, want_gx=False) is None
    _, rgw_t, _ = ref64.bn_backward(x, gy, w, rrm, rrv, rsm, rss, True, scale, eps, gw=gw0, want_gx=False)
    assert rel_err(host(gw), rgw_t) < GRAD_TOL


@pytest.mark.parametrize("name", ["bn_affine", "bn_plain"])
def test_bn_golden(F, name):
    g = golden(name)
    affine = int(g["params"][0])
    w = dev(g["g"]) if affine else None
    b = dev(g["b"]) if affine else None
    mom, eps, scale = float(g["momentum"]), float(g["eps"]), float(g["scale"])
    rm, rv = dev(g["rm0"]), dev(g["rv0"])
    y, sm, ss = F.batchnorm_forward(dev(g["x"]), w, b, rm, rv, True, mom, eps)
    assert rel_err(host(y), g["y_train"]) < FWD_TOL
    assert rel_err(host(rm), g["rm_train"]) < FWD_TOL and rel_err(host(rv), g["rv_train"]) < FWD_TOL
    assert rel_err(host(sm), g["save_mean"]) < FWD_TOL and rel_err(host(ss), g["save_std"]) < FWD_TOL
    C = g["x"].shape[1]
    gw, gb = torch.zeros(C, device="cuda"), torch.zeros(C, device="cuda")
    gx = F.batchnorm_backward(dev(g["x"]), dev(g["gy"]), w, rm, rv, sm, ss, True, scale, eps, grad_weight=gw, grad_bias=gb)
    assert rel_err(host(gx), g["gx_train"]) < GRAD_TOL
    if affine:
        assert rel_err(host(gw), g["gw_train"]) < GRAD_TOL and rel_err(host(gb), g["gb_train"]) < GRAD_TOL
    rm, rv = dev(g["rm0"]), dev(g["rv0"])
    y, _, _ = F.batchnorm_forward(dev(g["x"]), w, b, rm, rv, False, mom, eps)
    assert rel_err(host(y), g["y_eval"]) < FWD_TOL


@pytest.mark.parametrize("shape,affine", [
    ((4, 64, 112, 112), True),     # the benchmarked geometry, reduced batch
    ((7, 5, 9, 11), True),         # S not a multiple of 4 -> scalar path
    ((3, 16, 32, 32), False),      # H*W = 1024, the reference's extra case; no affine
    ((300, 3, 2, 2), True),        # more images than chunks
    ((2, 1024, 7, 7), True),
    ((6, 24, 14, 14), True),       # 196-element planes: a multiple of 16 bytes, yet on the flat elementwise kernels
    ((4, 8, 2, 3), True),          # 24 elements per channel
    ((16, 4100, 2, 2), True),      # more channels than ticket counters: the merge runs as a separate launch
    ((40, 2, 16, 16), True),       # 40 chunks per channel: more than one warp-lane round in the merge
    ((64, 6, 28, 28), True),       # grouped kernels: several channels per CTA share
    ((12, 37, 20, 20), False),     # grouped kernels: a channel count that does not divide into equal groups
    ((48, 3, 112, 112), True),     # grouped kernels: planes longer than a stage
])
def test_bn_shapes(F, ref64, shape, affine, grouped_mode):
    rng = np.random.default_rng(abs(hash(shape)) % 99991)
    C = shape[1]
    x = (0.5 + 2.0 * rng.standard_normal(shape)).astype(np.float32)
    w = rng.uniform(0, 1, C).astype(np.float32) if affine else None
    b = rng.uniform(-1, 1, C).astype(np.float32) if affine else None
    rm0 = rng.standard_normal(C).astype(np.float32)
    rv0 = rng.uniform(0.5, 2, C).astype(np.float32)
    gy = rng.standard_normal(shape).astype(np.float32)
    bn_check(F, ref64, x, w, b, rm0, rv0, gy, 0.1, 1e-5, 0.5,
             gw0=rng.standard_normal(C).astype(np.float32), gb0=rng.standard_normal(C).astype(np.float32))


def test_bn_large_mean_small_std(F, ref64, grouped_mode):
    # |mean| >> std: a plain sum-of-squares in fp32 would lose the variance; the shifted sums must not.
    rng = np.random.default_rng(11)
    x = (100.0 + 0.01 * rng.standard_normal((8, 4, 28, 28))).astype(np.float32)
    rm0, rv0 = np.zeros(4, np.float32), np.ones(4, np.float32)
    _, _, _, rsm, rss = ref64.bn_forward(x, None, None, rm0, rv0, True, 0.1, 1e-5)
    rm, rv = dev(rm0), dev(rv0)
    _, sm, ss = F.batchnorm_forward(dev(x), None, None, rm, rv, True, 0.1, 1e-5)
    assert rel_err(host(sm), rsm) < 1e-6
    assert rel_err(host(ss), rss) < 1e-4


def test_bn_single_element_and_zero_variance(F):
    # n = 1 gives NaN running_var (division by n - 1 = 0) and, with eps = 0, invstd = 0 — both are the
    # reference's behaviour (BatchNormalization.cu:188-200) and are kept.
    x = torch.full((1, 2, 1, 1), 3.0, device="cuda")
    rm, rv = torch.zeros(2, device="cuda"), torch.ones(2, device="cuda")
    y, sm, ss = F.batchnorm_forward(x, None, None, rm, rv, True, 0.1, 0.0)
    assert torch.all(ss == 0) and torch.all(y == 0) and torch.all(sm == 3.0)
    assert torch.all(torch.isnan(rv))


@pytest.mark.parametrize("shape", [(4, 8, 14, 14), (3, 5, 7, 9), (64, 6, 28, 28)])
def test_bn_relu_fused_equals_separate_calls(F, shape, grouped_mode):
    # the fused BN+ReLU pair must equal BatchNormalization followed by Threshold(0, 0), forward and backward
    g = torch.Generator(device="cuda").manual_seed(9)
    C = shape[1]
    x = torch.randn(shape, device="cuda", generator=g) * 2 + 0.3
    w, b = torch.rand(C, device="cuda", generator=g), torch.rand(C, device="cuda", generator=g) - 0.5
    gy = torch.randn(shape, device="cuda", generator=g)
    rm1, rv1, rm2, rv2 = (torch.zeros(C, device="cuda"), torch.ones(C, device="cuda"), torch.zeros(C, device="cuda"),
                          torch.ones(C, device="cuda"))
    z, sm, ss = F.batchnorm_forward(x, w, b, rm1, rv1, True)
    y_ref = F.threshold_forward(z)
    y, sm2, ss2 = F.batchnorm_relu_forward(x, w, b, rm2, rv2, True)
    assert torch.equal(y, y_ref) and torch.equal(sm, sm2) and torch.equal(ss, ss2) and torch.equal(rm1, rm2)
    gw1, gb1, gw2, gb2 = (torch.zeros(C, device="cuda") for _ in range(4))
    gx_ref = F.batchnorm_backward(x, F.threshold_backward(z, gy), w, rm1, rv1, sm, ss, True, grad_weight=gw1, grad_bias=gb1)
    gx = F.batchnorm_relu_backward(x, gy, w, b, rm2, rv2, sm2, ss2, True, grad_weight=gw2, grad_bias=gb2)
    assert torch.equal(gx, gx_ref) and torch.equal(gw1, gw2) and torch.equal(gb1, gb2)


def test_bn_full_size_properties(F):
    # the benchmarked geometry at reduced batch (N = 64; test_full_size_gpu.py runs the full 256):
    # with gamma = 1, beta = 0 the training output has zero mean and unit biased variance per channel, the
    # saved statistics are those of x, and the input gradient is orthogonal to 1 and to (x - mean).
    g = torch.Generator(device="cuda").manual_seed(8)
    N, C, HW = 64, 64, 112
    x = torch.randn((N, C, HW, HW), device="cuda", generator=g) * 2 + 0.5
    rm, rv = torch.zeros(C, device="cuda"), torch.ones(C, device="cuda")
    y, sm, ss = F.batchnorm_forward(x, None, None, rm, rv, True, 0.1, 1e-5)
    xd = x.double()
    mean = xd.mean((0, 2, 3))
    var = xd.var((0, 2, 3), unbiased=False)
    assert float((sm.double() - mean).abs().max()) < 1e-5 * float(mean.abs().max())
    assert float((ss.double() - 1 / torch.sqrt(var + 1e-5)).abs().max()) < 1e-5
    yd = y.double()
    assert float(yd.mean((0, 2, 3)).abs().max()) < 1e-5
    assert float((yd.var((0, 2, 3), unbiased=False) - 1).abs().max()) < 1e-4
    n = N * HW * HW
    assert float((rv.double() - (0.9 + 0.1 * var * n / (n - 1))).abs().max()) < 1e-5 * float(var.max())
    gy = torch.randn((N, C, HW, HW), device="cuda", generator=g)
    gx = F.batchnorm_backward(x, gy, None, rm, rv, sm, ss, True)
    gxd = gx.double()
    scale = float(gxd.abs().sum((0, 2, 3)).max())
    assert float(gxd.sum((0, 2, 3)).abs().max()) < 1e-5 * scale
    assert float((gxd * (xd - mean.view(1, C, 1, 1))).sum((0, 2, 3)).abs().max()) < 1e-5 * scale * 2
