"""Generates tests/golden/*.npz: small seeded inputs with the outputs PyTorch's
CPU operators give for them.

PyTorch's CPU convolution, batch-norm and pooling kernels descend from the
torch/nn THNN code that the reference's own tests compare against, so these
files pin the CPU oracle (oracle/thnn_ref.c) from a second, independent
implementation.  The reference tree itself holds no golden vectors.

Run from the repository root:  python tests/golden/make_golden.py
Pooling indices are stored 0-based as PyTorch returns them; the tests add the
index base of the build under test.
"""
import os

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
torch.set_num_threads(1)
torch.backends.mkldnn.enabled = False  # plain native CPU kernels, deterministic order


def t(a, grad=False):
    x = torch.from_numpy(np.ascontiguousarray(a)).double()
    x.requires_grad_(grad)
    return x


def save(name, **arrs):
    out = {}
    for k, v in arrs.items():
        if isinstance(v, torch.Tensor):
            v = v.detach().numpy()
        v = np.asarray(v)
        if v.dtype == np.float64:
            v = v.astype(np.float32)
        out[k] = v
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)


def dwconv_case(name, rng, N, C, H, W, M, k, d, pad, bias=True, scale=1.0):
    x = rng.uniform(-1, 1, (N, C, H, W)).astype(np.float32)
    bound = 1.0 / np.sqrt(k * k)
    w = rng.uniform(-bound, bound, (M, C, k, k)).astype(np.float32)
    b = rng.uniform(-bound, bound, (M, C)).astype(np.float32) if bias else None
    oH = (H + 2 * pad - k) // d + 1
    oW = (W + 2 * pad - k) // d + 1
    gy = rng.standard_normal((N, C * M, oH, oW)).astype(np.float32)
    gw0 = rng.standard_normal((M, C, k, k)).astype(np.float32)
    gb0 = rng.standard_normal((M, C)).astype(np.float32)
    # torch groups=C weight layout: [C*M, 1, k, k] with output channel c*M+j
    xt = t(x, True)
    wt = t(w, True)
    wg = wt.permute(1, 0, 2, 3).reshape(C * M, 1, k, k)
    bt = t(b, True) if bias else None
    bg = bt.permute(1, 0).reshape(C * M) if bias else None
    y = F.conv2d(xt, wg, bg, stride=d, padding=pad, groups=C)
    y.backward(t(gy))
    arrs = dict(x=x, w=w, gy=gy, y=y, gx=xt.grad, gw0=gw0, gb0=gb0,
                gw=t(gw0) + scale * wt.grad, params=np.array([M, k, d, pad, int(bias)]),
                scale=np.float32(scale))
    if bias:
        arrs.update(b=b, gb=t(gb0) + scale * bt.grad)
    save(name, **arrs)


def convmm_case(name, rng, N, C, H, W, K, k, d, pad, bias=True, scale=1.0):
    x = rng.standard_normal((N, C, H, W)).astype(np.float32)
    w = (rng.standard_normal((K, C, k, k)) * np.sqrt(2.0 / (C * k * k))).astype(np.float32)
    b = rng.uniform(-0.5, 0.5, K).astype(np.float32) if bias else None
    oH = (H + 2 * pad - k) // d + 1
    oW = (W + 2 * pad - k) // d + 1
    gy = rng.standard_normal((N, K, oH, oW)).astype(np.float32)
    gw0 = rng.standard_normal((K, C, k, k)).astype(np.float32)
    gb0 = rng.standard_normal(K).astype(np.float32)
    xt, wt = t(x, True), t(w, True)
    bt = t(b, True) if bias else None
    y = F.conv2d(xt, wt, bt, stride=d, padding=pad)
    y.backward(t(gy))
    arrs = dict(x=x, w=w, gy=gy, y=y, gx=xt.grad, gw0=gw0, gb0=gb0, gw=t(gw0) + scale * wt.grad,
                params=np.array([K, k, d, pad, int(bias)]), scale=np.float32(scale))
    if bias:
        arrs.update(b=b, gb=t(gb0) + scale * bt.grad)
    save(name, **arrs)


def dilconv_case(name, rng, N, C, H, W, K, k, d, pad, dil, bias=True, scale=1.0):
    """SpatialDilatedConvolution: torch.nn.functional.conv2d with dilation, forward and gradients."""
    x = rng.standard_normal((N, C, H, W)).astype(np.float32)
    w = (rng.standard_normal((K, C, k, k)) * np.sqrt(2.0 / (C * k * k))).astype(np.float32)
    b = rng.uniform(-0.5, 0.5, K).astype(np.float32) if bias else None
    oH = (H + 2 * pad - (dil * (k - 1) + 1)) // d + 1
    oW = (W + 2 * pad - (dil * (k - 1) + 1)) // d + 1
    gy = rng.standard_normal((N, K, oH, oW)).astype(np.float32)
    gw0 = rng.standard_normal((K, C, k, k)).astype(np.float32)
    gb0 = rng.standard_normal(K).astype(np.float32)
    xt, wt = t(x, True), t(w, True)
    bt = t(b, True) if bias else None
    y = F.conv2d(xt, wt, bt, stride=d, padding=pad, dilation=dil)
    y.backward(t(gy))
    arrs = dict(x=x, w=w, gy=gy, y=y, gx=xt.grad, gw0=gw0, gb0=gb0, gw=t(gw0) + scale * wt.grad,
                params=np.array([K, k, d, pad, dil, int(bias)]), scale=np.float32(scale))
    if bias:
        arrs.update(b=b, gb=t(gb0) + scale * bt.grad)
    save(name, **arrs)


def fullconv_case(name, rng, N, P, H, W, Q, k, d, pad, dil, adj, bias=True, scale=1.0):
    """SpatialFullDilatedConvolution: torch.nn.functional.conv_transpose2d, forward and gradients."""
    x = rng.standard_normal((N, P, H, W)).astype(np.float32)
    w = (rng.standard_normal((P, Q, k, k)) * np.sqrt(2.0 / (P * k * k))).astype(np.float32)
    b = rng.uniform(-0.5, 0.5, Q).astype(np.float32) if bias else None
    xt, wt = t(x, True), t(w, True)
    bt = t(b, True) if bias else None
    y = F.conv_transpose2d(xt, wt, bt, stride=d, padding=pad, output_padding=adj, dilation=dil)
    gy = rng.standard_normal(tuple(y.shape)).astype(np.float32)
    gw0 = rng.standard_normal((P, Q, k, k)).astype(np.float32)
    gb0 = rng.standard_normal(Q).astype(np.float32)
    y.backward(t(gy))
    arrs = dict(x=x, w=w, gy=gy, y=y, gx=xt.grad, gw0=gw0, gb0=gb0, gw=t(gw0) + scale * wt.grad,
                params=np.array([Q, k, d, pad, dil, adj, int(bias)]), scale=np.float32(scale))
    if bias:
        arrs.update(b=b, gb=t(gb0) + scale * bt.grad)
    save(name, **arrs)


def bn_case(name, rng, N, C, H, W, affine=True, momentum=0.1, eps=1e-5, scale=1.0):
    x = (0.5 + 2.0 * rng.standard_normal((N, C, H, W))).astype(np.float32)
    g = rng.uniform(0, 1, C).astype(np.float32) if affine else None
    b = rng.uniform(-1, 1, C).astype(np.float32) if affine else None
    rm0 = rng.standard_normal(C).astype(np.float32)
    rv0 = rng.uniform(0.5, 2, C).astype(np.float32)
    gy = rng.standard_normal((N, C, H, W)).astype(np.float32)
    arrs = dict(x=x, gy=gy, rm0=rm0, rv0=rv0, params=np.array([int(affine)]),
                momentum=np.float64(momentum), eps=np.float64(eps), scale=np.float32(scale))
    if affine:
        arrs.update(g=g, b=b)
    for train in (True, False):
        xt = t(x, True)
        gt = t(g, True) if affine else None
        bt = t(b, True) if affine else None
        rm, rv = t(rm0).clone(), t(rv0).clone()
        y = F.batch_norm(xt, rm, rv, gt, bt, training=train, momentum=momentum, eps=eps)
        y.backward(t(gy))
        tag = "train" if train else "eval"
        arrs["y_" + tag] = y
        arrs["gx_" + tag] = xt.grad
        if affine:
            arrs["gw_" + tag] = scale * gt.grad
            arrs["gb_" + tag] = scale * bt.grad
        if train:
            xd = t(x)
            mean = xd.mean(dim=(0, 2, 3))
            var = xd.var(dim=(0, 2, 3), unbiased=False)
            arrs.update(rm_train=rm, rv_train=rv, save_mean=mean, save_std=1.0 / torch.sqrt(var + eps))
    save(name, **arrs)


def maxpool_case(name, rng, N, C, H, W, k, d, pad, ceil_mode, ties=False):
    x = rng.standard_normal((N, C, H, W)).astype(np.float32)
    if ties:
        x = np.round(x * 2) / 2  # many equal values: exercises "first maximum wins"
    xt = torch.from_numpy(x).clone().requires_grad_(True)
    y, ind = F.max_pool2d(xt, k, d, pad, ceil_mode=ceil_mode, return_indices=True)
    gy = rng.standard_normal(tuple(y.shape)).astype(np.float32)
    y.backward(torch.from_numpy(gy))
    save(name, x=x, y=y, ind0=ind.numpy().astype(np.int64), gy=gy, gx=xt.grad,
         params=np.array([k, d, pad, int(ceil_mode)]))


def support_case(name, rng):
    x = rng.standard_normal((5, 1000)).astype(np.float32) * 3
    target0 = rng.integers(0, 1000, 5).astype(np.int64)
    xt = t(x, True)
    lp = F.log_softmax(xt, dim=1)
    loss = F.nll_loss(lp, torch.from_numpy(target0))
    loss.backward()
    a = rng.standard_normal((3, 8, 7, 7)).astype(np.float32)
    at = t(a, True)
    ap = F.avg_pool2d(at, 7, 1, 0)
    gap = rng.standard_normal(tuple(ap.shape)).astype(np.float32)
    ap.backward(t(gap))
    a2 = rng.standard_normal((2, 3, 9, 10)).astype(np.float32)
    a2t = t(a2, True)
    ap2 = F.avg_pool2d(a2t, 3, 2, 1, count_include_pad=True)
    gap2 = rng.standard_normal(tuple(ap2.shape)).astype(np.float32)
    ap2.backward(t(gap2))
    save(name, x=x, target0=target0, lp=lp, loss=loss, gx=xt.grad,
         a=a, ap=ap, gap=gap, ga=at.grad, a2=a2, ap2=ap2, gap2=gap2, ga2=a2t.grad)


def main():
    rng = np.random.default_rng(1234)
    # depthwise: the reference's only test shape (m=4, 28x28 would be large; use 12x12), MobileNet-like
    dwconv_case("dwconv_m4", rng, 3, 3, 12, 12, 4, 3, 1, 1)
    dwconv_case("dwconv_s1", rng, 2, 8, 14, 14, 1, 3, 1, 1, scale=0.5)
    dwconv_case("dwconv_s2", rng, 2, 8, 14, 14, 1, 3, 2, 1)
    dwconv_case("dwconv_s2_odd", rng, 2, 4, 7, 9, 1, 3, 2, 1, bias=False)
    dwconv_case("dwconv_k5", rng, 1, 2, 11, 10, 2, 5, 2, 2)
    dwconv_case("dwconv_w28", rng, 2, 4, 28, 28, 1, 3, 1, 1)
    convmm_case("convmm_3x3", rng, 2, 5, 9, 8, 8, 3, 1, 1, scale=0.5)
    convmm_case("convmm_1x1", rng, 3, 16, 7, 7, 24, 1, 1, 0)
    convmm_case("convmm_s2", rng, 2, 3, 12, 12, 8, 3, 2, 1, bias=False)
    bn_case("bn_affine", rng, 4, 6, 5, 7, scale=0.5)
    bn_case("bn_plain", rng, 3, 4, 8, 8, affine=False)
    maxpool_case("maxpool_3s2p1", rng, 2, 3, 12, 12, 3, 2, 1, False)
    maxpool_case("maxpool_ceil", rng, 2, 3, 11, 13, 3, 2, 1, True)
    maxpool_case("maxpool_ties", rng, 2, 3, 10, 10, 3, 2, 1, False, ties=True)
    maxpool_case("maxpool_2s2", rng, 1, 4, 9, 9, 2, 2, 0, True)
    support_case("support", rng)
    dilated_cases()
    fullconv_cases()


def dilated_cases():
    # own generator: added after the fixtures above were committed, and must not shift their random streams
    rng = np.random.default_rng(20240)
    dilconv_case("dilconv_3x3_d2", rng, 2, 5, 11, 10, 8, 3, 1, 2, 2, scale=0.5)
    dilconv_case("dilconv_3x3_d3_s2", rng, 2, 4, 15, 13, 6, 3, 2, 3, 3, bias=False)


def fullconv_cases():
    # own generator, for the same reason
    rng = np.random.default_rng(20241)
    fullconv_case("fullconv_3x3_s2", rng, 2, 6, 7, 6, 5, 3, 2, 1, 1, 1, scale=0.5)
    fullconv_case("fullconv_4x4_s2", rng, 2, 4, 5, 6, 8, 4, 2, 1, 1, 0, bias=False)
    fullconv_case("fullconv_3x3_d2", rng, 1, 3, 8, 9, 4, 3, 1, 2, 2, 0)


if __name__ == "__main__":
    import sys
    if len(sys.argv) > 1 and sys.argv[1] == "dilated":
        dilated_cases()                      # only the dilated-convolution fixtures
    elif len(sys.argv) > 1 and sys.argv[1] == "full":
        fullconv_cases()                     # only the transposed-convolution fixtures
    else:
        main()
