"""Generates tests/golden/refk_*.npz: small seeded inputs with the outputs of the reference's OWN
device kernels (oracle/_ref/librefk_gpu.so: the reference's BatchNormalization kernels and its
im2col / col2im around cuBLAS SGEMM, compiled unchanged from the reference tree).  Needs a GPU:

    python tests/golden/make_golden_refkernels.py [output folder, default tests/golden]

The files pin the CPU oracle on results the reference's code itself produced, for the operators whose
kernels cannot run on the host (tests/test_oracle_golden.py::test_*_refkernel_golden).
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle.ref_kernels import RefKernelsGPU  # noqa: E402

OUT = sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__))
os.makedirs(OUT, exist_ok=True)
rk = RefKernelsGPU()
d = lambda a: None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()
h = lambda t: None if t is None else t.cpu().numpy()


def conv_case(name, kind, rng, N, C, H, W, KM, k, s, pad, bias=True, scale=0.75):
    x = rng.uniform(-1, 1, (N, C, H, W)).astype(np.float32)
    fan = (C if kind == "convmm" else 1) * k * k
    wshape = (KM, C, k, k)
    w = (rng.standard_normal(wshape) * np.sqrt(2.0 / fan)).astype(np.float32)
    b = rng.uniform(-1, 1, (KM,) if kind == "convmm" else (KM, C)).astype(np.float32) if bias else None
    fwd, dgrad, wgrad = [getattr(rk, kind + "_" + n) for n in ("forward", "grad_input", "acc_grad")]
    y = fwd(d(x), d(w), d(b), s, s, pad, pad)
    gy = rng.standard_normal(tuple(y.shape)).astype(np.float32)
    gx = dgrad(d(gy), d(w), H, W, s, s, pad, pad)
    gw0 = rng.standard_normal(wshape).astype(np.float32)
    gb0 = rng.standard_normal(b.shape).astype(np.float32) if bias else None
    gw, gb = wgrad(d(x), d(gy), d(gw0), d(gb0), s, s, pad, pad, scale)
    arrs = dict(x=x, w=w, gy=gy, y=h(y), gx=h(gx), gw0=gw0, gw=h(gw), params=np.array([KM, k, s, pad, int(bias)]),
                scale=np.float32(scale))
    if bias:
        arrs.update(b=b, gb0=gb0, gb=h(gb))
    np.savez_compressed(os.path.join(OUT, name + ".npz"), **arrs)


def bn_case(name, rng, N, C, S, affine):
    x = (rng.standard_normal((N, C, S)) * 2 + 0.5).astype(np.float32)
    g = rng.uniform(0, 1, C).astype(np.float32) if affine else None
    b = rng.standard_normal(C).astype(np.float32) if affine else None
    rm0, rv0 = rng.standard_normal(C).astype(np.float32), rng.uniform(0.5, 1.5, C).astype(np.float32)
    gy = rng.standard_normal(x.shape).astype(np.float32)
    gw0, gb0 = rng.standard_normal(C).astype(np.float32), rng.standard_normal(C).astype(np.float32)
    mom, eps, scale = 0.1, 1e-5, 0.5
    y, rm, rv, sm, ss = rk.bn_forward(d(x), d(g), d(b), d(rm0), d(rv0), True, mom, eps)
    gx, gw, gb = rk.bn_backward(d(x), d(gy), d(g), d(rm0), d(rv0), sm, ss, True, scale, eps, gw=d(gw0), gb=d(gb0))
    ye = rk.bn_forward(d(x), d(g), d(b), d(rm0), d(rv0), False, mom, eps)[0]
    gxe, gwe, gbe = rk.bn_backward(d(x), d(gy), d(g), d(rm0), d(rv0), sm, ss, False, scale, eps, gw=d(gw0), gb=d(gb0))
    arrs = dict(x=x, rm0=rm0, rv0=rv0, gy=gy, gw0=gw0, gb0=gb0, y_train=h(y), rm_train=h(rm), rv_train=h(rv),
                save_mean=h(sm), save_std=h(ss), gx_train=h(gx), gw_train=h(gw), gb_train=h(gb), y_eval=h(ye),
                gx_eval=h(gxe), gw_eval=h(gwe), gb_eval=h(gbe), params=np.array([int(affine)]),
                momentum=np.float64(mom), eps=np.float64(eps), scale=np.float64(scale))
    if affine:
        arrs.update(g=g, b=b)
    np.savez_compressed(os.path.join(OUT, name + ".npz"), **arrs)


def unfold_case(name, rng, C, H, W, kH, kW, padH, padW, dH, dW, dilH, dilW):
    x = rng.standard_normal((C, H, W)).astype(np.float32)
    col = rk.im2col(d(x), kH, kW, padH, padW, dH, dW, dilH, dilW)
    c2 = rng.standard_normal(tuple(col.shape)).astype(np.float32)
    back = rk.col2im(d(c2), C, H, W, kH, kW, padH, padW, dH, dW, dilH, dilW)
    np.savez_compressed(os.path.join(OUT, name + ".npz"), x=x, col=h(col), col_in=c2, folded=h(back),
                        params=np.array([kH, kW, padH, padW, dH, dW, dilH, dilW]))


rng = np.random.default_rng(20240612)
conv_case("refk_convmm_3x3", "convmm", rng, 3, 5, 9, 11, 7, 3, 1, 1)
conv_case("refk_convmm_5x5_s2", "convmm", rng, 2, 4, 13, 12, 6, 5, 2, 2, bias=False)
conv_case("refk_convmm_1x1", "convmm", rng, 2, 16, 7, 7, 12, 1, 1, 0)
conv_case("refk_dwconv_s1", "dwconv", rng, 2, 6, 14, 14, 1, 3, 1, 1)
conv_case("refk_dwconv_s2_m3", "dwconv", rng, 2, 4, 11, 12, 3, 3, 2, 1)
conv_case("refk_dwconv_k5_nobias", "dwconv", rng, 1, 3, 9, 9, 2, 5, 1, 2, bias=False)
bn_case("refk_bn_affine", rng, 4, 6, 50, True)
bn_case("refk_bn_plain", rng, 3, 5, 33, False)
unfold_case("refk_unfold_3x3_s2", rng, 3, 9, 10, 3, 3, 1, 1, 2, 2, 1, 1)
unfold_case("refk_unfold_3x2_dil2", rng, 2, 11, 9, 3, 2, 2, 1, 1, 2, 2, 2)
print("wrote", sorted(f for f in os.listdir(OUT) if f.startswith("refk_")))
