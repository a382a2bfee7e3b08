"""The CPU oracle against the committed fixtures — outputs of the reference's own device kernels run on a
B200 (tests/golden/refk_*.npz, made by tests/golden/make_golden_refkernels.py) and outputs of PyTorch's CPU
operators (the other files, tests/golden/make_golden.py) — and against the reference's own self-consistency
tests.  No GPU needed."""
import numpy as np
import pytest

from conftest import golden, rel_err

DW = ["dwconv_m4", "dwconv_s1", "dwconv_s2", "dwconv_s2_odd", "dwconv_k5", "dwconv_w28"]
MM = ["convmm_3x3", "convmm_1x1", "convmm_s2"]
MP = ["maxpool_3s2p1", "maxpool_ceil", "maxpool_ties", "maxpool_2s2"]


@pytest.mark.parametrize("name", DW)
def test_dwconv_oracle_vs_golden(ref64, name):
    g = golden(name)
    M, k, d, pad, has_b = [int(v) for v in g["params"]]
    b = g["b"] if has_b else None
    H, W = g["x"].shape[2:]
    assert rel_err(ref64.dwconv_forward(g["x"], g["w"], b, d, d, pad, pad), g["y"]) < 1e-6
    assert rel_err(ref64.dwconv_grad_input(g["gy"], g["w"], H, W, d, d, pad, pad), g["gx"]) < 1e-6
    gw, gb = ref64.dwconv_acc_grad(g["x"], g["gy"], g["gw0"], g["gb0"] if has_b else None, d, d, pad, pad,
                                   float(g["scale"]))
    assert rel_err(gw, g["gw"]) < 1e-6
    if has_b:
        assert rel_err(gb, g["gb"]) < 1e-6


@pytest.mark.parametrize("name", MM)
def test_convmm_oracle_vs_golden(ref64, name):
    g = golden(name)
    K, k, d, pad, has_b = [int(v) for v in g["params"]]
    b = g["b"] if has_b else None
    H, W = g["x"].shape[2:]
    assert rel_err(ref64.convmm_forward(g["x"], g["w"], b, d, d, pad, pad), g["y"]) < 1e-6
    assert rel_err(ref64.convmm_grad_input(g["gy"], g["w"], H, W, d, d, pad, pad), g["gx"]) < 1e-6
    gw, gb = ref64.convmm_acc_grad(g["x"], g["gy"], g["gw0"], g["gb0"] if has_b else None, d, d, pad, pad,
                                   float(g["scale"]))
    assert rel_err(gw, g["gw"]) < 1e-6
    if has_b:
        assert rel_err(gb, g["gb"]) < 1e-6


@pytest.mark.parametrize("name", ["bn_affine", "bn_plain"])
def test_bn_oracle_vs_golden(ref64, name):
    g = golden(name)
    affine = int(g["params"][0])
    w = g["g"] if affine else None
    b = g["b"] if affine else None
    mom, eps, scale = float(g["momentum"]), float(g["eps"]), float(g["scale"])
    y, rm, rv, sm, ss = ref64.bn_forward(g["x"], w, b, g["rm0"], g["rv0"], True, mom, eps)
    assert rel_err(y, g["y_train"]) < 1e-6
    assert rel_err(rm, g["rm_train"]) < 1e-6
    assert rel_err(rv, g["rv_train"]) < 1e-6
    assert rel_err(sm, g["save_mean"]) < 1e-6
    assert rel_err(ss, g["save_std"]) < 1e-6
    C = g["x"].shape[1]
    z = np.zeros(C, np.float32)
    gx, gw, gb = ref64.bn_backward(g["x"], g["gy"], w, rm, rv, sm, ss, True, scale, eps, gw=z, gb=z)
    assert rel_err(gx, g["gx_train"]) < 2e-6
    if affine:
        assert rel_err(gw, g["gw_train"]) < 2e-6
        assert rel_err(gb, g["gb_train"]) < 2e-6
    y, rm2, rv2, _, _ = ref64.bn_forward(g["x"], w, b, g["rm0"], g["rv0"], False, mom, eps)
    assert rel_err(y, g["y_eval"]) < 1e-6
    assert np.array_equal(rm2, g["rm0"]) and np.array_equal(rv2, g["rv0"])
    gx, gw, gb = ref64.bn_backward(g["x"], g["gy"], w, g["rm0"], g["rv0"], sm, ss, False, scale, eps, gw=z, gb=z)
    assert rel_err(gx, g["gx_eval"]) < 2e-6
    if affine:
        assert rel_err(gw, g["gw_eval"]) < 2e-6
        assert rel_err(gb, g["gb_eval"]) < 2e-6


@pytest.mark.parametrize("name", MP)
def test_maxpool_oracle_vs_golden(ref64, name):
    g = golden(name)
    k, d, pad, ceil_mode = [int(v) for v in g["params"]]
    y, ind = ref64.maxpool_forward(g["x"], k, k, d, d, pad, pad, bool(ceil_mode))
    assert y.shape == g["y"].shape
    assert np.array_equal(y, g["y"])
    assert np.array_equal(ind, g["ind0"] + ref64.index_base)          # bit-exact indices
    H, W = g["x"].shape[2:]
    gx = ref64.maxpool_backward(g["gy"], ind, H, W, k, k, d, d, pad, pad)
    assert rel_err(gx, g["gx"]) < 1e-6


def test_maxpool_all_nan_window(ref64):
    # A window of NaN / -inf never beats the -FLT_MAX start value: stored index is -1 + base
    # (lib/THCUNN/SpatialDilatedMaxPooling.cu:28-40).
    x = np.full((1, 1, 4, 4), np.nan, np.float32)
    x[0, 0, 2:, 2:] = 1.0
    y, ind = ref64.maxpool_forward(x, 2, 2, 2, 2, 0, 0, False)
    assert ind[0, 0, 0, 0] == -1 + ref64.index_base
    assert y[0, 0, 0, 0] == -np.finfo(np.float32).max
    assert ind[0, 0, 1, 1] == 2 * 4 + 2 + ref64.index_base


def test_support_oracle_vs_golden(ref64):
    g = golden("support")
    lp = ref64.logsoftmax_forward(g["x"])
    assert rel_err(lp, g["lp"]) < 1e-6
    tgt = g["target0"] + ref64.index_base
    loss, tw = ref64.classnll_forward(lp, tgt)
    assert abs(loss - float(g["loss"])) < 1e-6 * abs(float(g["loss"])) and tw == 5.0
    gl = ref64.classnll_backward(tgt, tw, 5, 1000)
    assert rel_err(ref64.logsoftmax_backward(lp, gl), g["gx"]) < 1e-5
    assert rel_err(ref64.avgpool_forward(g["a"], 7, 7, 1, 1, 0, 0), g["ap"]) < 1e-6
    assert rel_err(ref64.avgpool_backward(g["gap"], 7, 7, 7, 7, 1, 1, 0, 0), g["ga"]) < 1e-6
    assert rel_err(ref64.avgpool_forward(g["a2"], 3, 3, 2, 2, 1, 1), g["ap2"]) < 1e-6
    assert rel_err(ref64.avgpool_backward(g["gap2"], 9, 10, 3, 3, 2, 2, 1, 1), g["ga2"]) < 1e-6
    x = g["a"]
    assert np.array_equal(ref64.threshold_forward(x), np.maximum(x, 0))
    assert np.array_equal(ref64.threshold_backward(x, x * 2), np.where(x > 0, x * 2, 0))


def test_avgpool_includepad_known_answer(ref64):
    # Known answers of the reference's SpatialAveragePooling_includepad test (test.lua:2597-2616):
    # 2x2 input of 3s, kernel 2, stride 1, pad 1 -> centre 3; corner 3 with exclude-pad, 3/4 with include-pad.
    x = np.full((1, 1, 2, 2), 3.0, np.float32)
    inc = ref64.avgpool_forward(x, 2, 2, 1, 1, 1, 1, count_include_pad=True)
    exc = ref64.avgpool_forward(x, 2, 2, 1, 1, 1, 1, count_include_pad=False)
    assert inc[0, 0, 0, 0] == pytest.approx(3.0 / 4) and exc[0, 0, 0, 0] == pytest.approx(3.0)
    assert inc[0, 0, 1, 1] == pytest.approx(3.0)


def test_dwconv_equals_per_channel_convolution(ref64):
    # The reference's only depthwise test (test.lua:6602-6661): depthwise forward equals, channel by
    # channel, SpatialConvolution(1, m, 3,3,1,1,1,1) fed weight[:, c] and bias[:, c]; n=3, m=4, 28x28, batch 3.
    rng = np.random.default_rng(7)
    n, m = 3, 4
    x = rng.random((3, n, 28, 28)).astype(np.float32)
    w = rng.random((m, n, 3, 3)).astype(np.float32)
    b = rng.random((m, n)).astype(np.float32)
    y = ref64.dwconv_forward(x, w, b, 1, 1, 1, 1)
    for c in range(n):
        yc = ref64.convmm_forward(x[:, c:c + 1], w[:, c:c + 1], b[:, c], 1, 1, 1, 1)
        assert np.max(np.abs(y[:, c * m:(c + 1) * m] - yc)) < 1e-5


def test_pool_out_size_matches_float_formula(ref64):
    import math
    for size in range(1, 40):
        for k in (1, 2, 3, 5):
            for d in (1, 2, 3):
                for pad in range(0, k // 2 + 1):
                    for ceil_mode in (False, True):
                        if size + 2 * pad < k:
                            continue
                        f = np.float32(size - k + 2 * pad) / np.float32(d)
                        o = int((math.ceil if ceil_mode else math.floor)(f)) + 1
                        if pad and (o - 1) * d >= size + pad:
                            o -= 1
                        assert ref64.pool_out_size(size, k, d, pad, 1, ceil_mode) == o


def test_slice_range_matches_reference_rule(ref64):
    # DataParallelTable.lua:469-479 (1-based there, 0-based here)
    for n in (0, 1, 2, 7, 9, 15, 16, 1024):
        for g in (1, 2, 3, 4, 8):
            pos = 0
            for i in range(g):
                s, c = ref64.slice_range(n, g, i)
                per, extra = n // g, n - (n // g) * g
                want = per + 1 if i + 1 <= extra else per
                assert (s, c) == (pos, want)
                pos += c
            assert pos == n


def test_ref32_close_to_ref64(ref32, ref64):
    g = golden("dwconv_s1")
    a = ref32.dwconv_forward(g["x"], g["w"], g["b"], 1, 1, 1, 1)
    b = ref64.dwconv_forward(g["x"], g["w"], g["b"], 1, 1, 1, 1)
    assert rel_err(a, b) < 1e-5


@pytest.mark.parametrize("name", ["dilconv_3x3_d2", "dilconv_3x3_d3_s2"])
def test_dilated_conv_oracle_vs_golden(ref64, name):
    g = golden(name)
    K, k, d, pad, dil, has_b = [int(v) for v in g["params"]]
    H, W = g["x"].shape[2:]
    b = g["b"] if has_b else None
    assert rel_err(ref64.dilconv_forward(g["x"], g["w"], b, d, d, pad, pad, dil, dil), g["y"]) < 1e-6
    assert rel_err(ref64.dilconv_grad_input(g["gy"], g["w"], H, W, d, d, pad, pad, dil, dil), g["gx"]) < 1e-6
    gw, gb = ref64.dilconv_acc_grad(g["x"], g["gy"], g["gw0"], g["gb0"] if has_b else None, d, d, pad, pad, dil, dil,
                                    float(g["scale"]))
    assert rel_err(gw, g["gw"]) < 1e-6
    if has_b:
        assert rel_err(gb, g["gb"]) < 1e-6


@pytest.mark.parametrize("name", ["fullconv_3x3_s2", "fullconv_4x4_s2", "fullconv_3x3_d2"])
def test_full_conv_oracle_vs_golden(ref64, name):
    # SpatialFullDilatedConvolution restatement against PyTorch-CPU conv_transpose2d fixtures
    g = golden(name)
    Q, k, d, pad, dil, adj, has_b = [int(v) for v in g["params"]]
    H, W = g["x"].shape[2:]
    b = g["b"] if has_b else None
    geo = (d, d, pad, pad, dil, dil, adj, adj)
    assert rel_err(ref64.fullconv_forward(g["x"], g["w"], b, *geo), g["y"]) < 1e-6
    assert rel_err(ref64.fullconv_grad_input(g["gy"], g["w"], H, W, *geo), g["gx"]) < 1e-6
    gw, gb = ref64.fullconv_acc_grad(g["x"], g["gy"], g["gw0"], g["gb0"] if has_b else None, *geo, float(g["scale"]))
    assert rel_err(gw, g["gw"]) < 1e-6
    if has_b:
        assert rel_err(gb, g["gb"]) < 1e-6


# ---------------------------------------------------------------------------------------------------
# Fixtures computed by the reference's own kernels (fp32 arithmetic in the reference's summation order,
# so agreement with the fp64 oracle is to fp32 rounding of these small cases, not to 1e-6).
REFK_TOL = 2e-5


@pytest.mark.parametrize("name", ["refk_convmm_3x3", "refk_convmm_5x5_s2", "refk_convmm_1x1"])
def test_convmm_oracle_vs_refkernel_golden(ref64, name):
    g = golden(name)
    K, k, d, pad, has_b = [int(v) for v in g["params"]]
    b = g["b"] if has_b else None
    H, W = g["x"].shape[2:]
    assert rel_err(ref64.convmm_forward(g["x"], g["w"], b, d, d, pad, pad), g["y"]) < REFK_TOL
    assert rel_err(ref64.convmm_grad_input(g["gy"], g["w"], H, W, d, d, pad, pad), g["gx"]) < REFK_TOL
    gw, gb = ref64.convmm_acc_grad(g["x"], g["gy"], g["gw0"], g["gb0"] if has_b else None, d, d, pad, pad, float(g["scale"]))
    assert rel_err(gw, g["gw"]) < REFK_TOL
    if has_b:
        assert rel_err(gb, g["gb"]) < REFK_TOL


@pytest.mark.parametrize("name", ["refk_dwconv_s1", "refk_dwconv_s2_m3", "refk_dwconv_k5_nobias"])
def test_dwconv_oracle_vs_refkernel_golden(ref64, name):
    g = golden(name)
    M, k, d, pad, has_b = [int(v) for v in g["params"]]
    b = g["b"] if has_b else None
    H, W = g["x"].shape[2:]
    assert rel_err(ref64.dwconv_forward(g["x"], g["w"], b, d, d, pad, pad), g["y"]) < REFK_TOL
    assert rel_err(ref64.dwconv_grad_input(g["gy"], g["w"], H, W, d, d, pad, pad), g["gx"]) < REFK_TOL
    gw, gb = ref64.dwconv_acc_grad(g["x"], g["gy"], g["gw0"], g["gb0"] if has_b else None, d, d, pad, pad, float(g["scale"]))
    assert rel_err(gw, g["gw"]) < REFK_TOL
    if has_b:
        assert rel_err(gb, g["gb"]) < REFK_TOL


@pytest.mark.parametrize("name", ["refk_bn_affine", "refk_bn_plain"])
def test_bn_oracle_vs_refkernel_golden(ref64, name):
    g = golden(name)
    affine = int(g["params"][0])
    w = g["g"] if affine else None
    b = g["b"] if affine else None
    mom, eps, scale = float(g["momentum"]), float(g["eps"]), float(g["scale"])
    y, rm, rv, sm, ss = ref64.bn_forward(g["x"], w, b, g["rm0"], g["rv0"], True, mom, eps)
    for got, key in ((y, "y_train"), (rm, "rm_train"), (rv, "rv_train"), (sm, "save_mean"), (ss, "save_std")):
        assert rel_err(got, g[key]) < REFK_TOL, key
    for train, sfx in ((True, "_train"), (False, "_eval")):
        gx, gw, gb = ref64.bn_backward(g["x"], g["gy"], w, g["rm0"], g["rv0"], g["save_mean"], g["save_std"], train, scale, eps,
                                       gw=g["gw0"], gb=g["gb0"])
        assert rel_err(gx, g["gx" + sfx]) < REFK_TOL
        assert rel_err(gw, g["gw" + sfx]) < REFK_TOL and rel_err(gb, g["gb" + sfx]) < REFK_TOL
    assert rel_err(ref64.bn_forward(g["x"], w, b, g["rm0"], g["rv0"], False, mom, eps)[0], g["y_eval"]) < REFK_TOL


@pytest.mark.parametrize("name", ["refk_unfold_3x3_s2", "refk_unfold_3x2_dil2"])
def test_unfold_index_math_vs_refkernel_golden(name):
    """im2col / col2im of the reference (lib/THCUNN/im2col.h:10-121) against a direct restatement of their index
    arithmetic: col[(c*kH+i)*kW+j, oh*oW+ow] = x[c, oh*dH-padH+i*dilH, ow*dW-padW+j*dilW] (0 outside), and the
    fold is its transpose.  Values are copied, so equality is exact for the unfold."""
    g = golden(name)
    kH, kW, padH, padW, dH, dW, dilH, dilW = [int(v) for v in g["params"]]
    x = g["x"]
    C, H, W = x.shape
    oH = (H + 2 * padH - (dilH * (kH - 1) + 1)) // dH + 1
    oW = (W + 2 * padW - (dilW * (kW - 1) + 1)) // dW + 1
    col = np.zeros((C * kH * kW, oH * oW), np.float32)
    folded = np.zeros((C, H, W), np.float64)
    for c in range(C):
        for i in range(kH):
            for j in range(kW):
                r = (c * kH + i) * kW + j
                for oh in range(oH):
                    for ow in range(oW):
                        h, w_ = oh * dH - padH + i * dilH, ow * dW - padW + j * dilW
                        if 0 <= h < H and 0 <= w_ < W:
                            col[r, oh * oW + ow] = x[c, h, w_]
                            folded[c, h, w_] += g["col_in"][r, oh * oW + ow]
    assert np.array_equal(col, g["col"])
    assert rel_err(folded, g["folded"]) < 5e-6      # the reference folds in fp32
