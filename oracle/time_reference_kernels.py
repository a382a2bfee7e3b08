"""Times the reference's own GPU schedule (oracle/_ref/librefk_gpu.so) on the current CUDA device.

Test infrastructure, like everything under oracle/: it answers "what does the reference's algorithm cost on this GPU"
for the workloads the benchmark times, so that the library's figures can be read against the reference's schedule on the
same hardware and not only against a CPU port.  What runs is the reference's code compiled where it lies: its
`im2col` / `col2im` kernels and per-image (depthwise: per image AND per channel) cuBLAS SGEMM loop
(generic/SpatialConvolutionMM.cu:58-486, generic/SpatialDepthWiseConvolution.cu:58-650), its batch-norm kernels
(BatchNormalization.cu:141-283) and its max-pooling kernels (SpatialDilatedMaxPooling.cu:8-80).

    python oracle/time_reference_kernels.py [--batch 64] [--out FILE]

Prints one JSON object.  Times are CUDA events on the legacy default stream, which is the stream the reference's launches
use; every figure is the second of two runs (the first warms cuBLAS and the allocator).
"""
import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

# (channels, height = width, stride) of MobileNetV1's 13 depthwise 3x3 layers
DW_LAYERS = [(32, 112, 1), (64, 112, 2), (128, 56, 1), (128, 56, 2), (256, 28, 1), (256, 28, 2)] + \
    [(512, 14, 1)] * 5 + [(512, 14, 2), (1024, 7, 1)]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64, help="images per depthwise layer")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()

    import torch
    from oracle import ref_kernels
    if not ref_kernels.available_gpu():
        print(json.dumps({"unavailable": "oracle/_ref/librefk_gpu.so is not built"}))
        return
    rk = ref_kernels.RefKernelsGPU()
    dev = torch.device("cuda")
    g = torch.Generator(device=dev)
    g.manual_seed(1234)

    def timed(fn):
        fn()                                   # warm-up
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b)

    out = {"device": torch.cuda.get_device_name(0)}

    # depthwise stack: forward + input gradient + parameter gradient of every layer -------------------------------
    N = args.batch
    total_ms, total_bytes, per_layer = 0.0, 0, []
    for (C, H, s) in DW_LAYERS:
        oH = (H + 2 - 3) // s + 1
        x = torch.rand((N, C, H, H), device=dev, generator=g) * 2 - 1
        w = (torch.rand((1, C, 3, 3), device=dev, generator=g) * 2 - 1) / 3
        b = (torch.rand((1, C), device=dev, generator=g) * 2 - 1) / 3
        gy = torch.randn((N, C, oH, oH), device=dev, generator=g)
        gw, gb = torch.zeros_like(w), torch.zeros_like(b)
        ms = [timed(lambda: rk.dwconv_forward(x, w, b, s, s, 1, 1)),
              timed(lambda: rk.dwconv_grad_input(gy, w, H, H, s, s, 1, 1)),
              timed(lambda: rk.dwconv_acc_grad(x, gy, gw, gb, s, s, 1, 1, 1.0))]
        nbytes = 3 * 4 * (x.numel() + gy.numel())
        per_layer.append({"C": C, "HW": H, "stride": s, "fwd_ms": round(ms[0], 2), "dgrad_ms": round(ms[1], 2),
                          "wgrad_ms": round(ms[2], 2), "gbs": round(nbytes / sum(ms) / 1e6, 2)})
        total_ms += sum(ms)
        total_bytes += nbytes
        del x, gy
    out["depthwise_stack"] = {"batch": N, "ms_per_step": round(total_ms, 1), "algorithmic_bytes": total_bytes,
                              "gbs": round(total_bytes / total_ms / 1e6, 2), "layers": per_layer,
                              "schedule": "per image and channel: im2col + cublasSgemm (M = 1 filter per channel)"}

    # SpatialConvolutionMM, per-image im2col + SGEMM ----------------------------------------------------------------
    def convmm(name, Nb, C, K, H, k, pad):
        x = torch.randn((Nb, C, H, H), device=dev, generator=g)
        w = torch.randn((K, C, k, k), device=dev, generator=g) * (2.0 / (C * k * k)) ** 0.5
        b = torch.zeros(K, device=dev)
        gy = torch.randn((Nb, K, H, H), device=dev, generator=g)
        gw, gb = torch.zeros_like(w), torch.zeros_like(b)
        flops = 2.0 * Nb * K * C * k * k * H * H
        f = timed(lambda: rk.convmm_forward(x, w, b, 1, 1, pad, pad))
        d = timed(lambda: rk.convmm_grad_input(gy, w, H, H, 1, 1, pad, pad))
        a = timed(lambda: rk.convmm_acc_grad(x, gy, gw, gb, 1, 1, pad, pad, 1.0))
        out[name] = {"fwd_us": round(f * 1e3, 1), "dgrad_us": round(d * 1e3, 1), "wgrad_us": round(a * 1e3, 1),
                     "fwd_tflops": round(flops / f / 1e9, 2), "dgrad_tflops": round(flops / d / 1e9, 2),
                     "wgrad_tflops": round(flops / a / 1e9, 2), "schedule": "per image: im2col + cublasSgemm (fp32)"}

    convmm("convmm_3x3_256to256_14x14_n128", 128, 256, 256, 14, 3, 1)
    convmm("convmm_1x1_1024to256_14x14_n128", 128, 1024, 256, 14, 1, 0)

    # batch norm and max pooling at 256 x 64 x 112 x 112 ----------------------------------------------------------------
    Nb, C, H = 256, 64, 112
    x = torch.randn((Nb, C, H, H), device=dev, generator=g) * 2 + 0.5
    gy = torch.randn((Nb, C, H, H), device=dev, generator=g)
    gam, bet = torch.rand(C, device=dev, generator=g), torch.zeros(C, device=dev)
    rm, rv = torch.zeros(C, device=dev), torch.ones(C, device=dev)
    S = 4.0 * x.numel()
    res = {}
    f = timed(lambda: res.__setitem__("f", rk.bn_forward(x, gam, bet, rm, rv, True, 0.1, 1e-5)))
    _, _, _, sm, ss = res["f"]
    e = timed(lambda: rk.bn_forward(x, gam, bet, rm, rv, False, 0.1, 1e-5))
    gw, gb = torch.zeros(C, device=dev), torch.zeros(C, device=dev)
    bwd = timed(lambda: rk.bn_backward(x, gy, gam, rm, rv, sm, ss, True, 1.0, 1e-5, gw, gb))
    out["batchnorm_256x64x112x112"] = {
        "train_fwd_us": round(f * 1e3, 1), "eval_fwd_us": round(e * 1e3, 1), "train_bwd_us": round(bwd * 1e3, 1),
        "train_fwd_gbs": round(2 * S / f / 1e6, 1), "eval_fwd_gbs": round(2 * S / e / 1e6, 1),
        "train_bwd_gbs": round(3 * S / bwd / 1e6, 1),
        "note": "includes the wrapper's allocation of the output and copies of the running statistics"}
    del res, gy
    oH = (H + 2 - 3) // 2 + 1
    res = {}
    f = timed(lambda: res.__setitem__("p", rk.maxpool_forward(x, oH, oH, 3, 3, 2, 2, 1, 1)))
    y, ind = res["p"]
    gyp = torch.randn_like(y)
    bwd = timed(lambda: rk.maxpool_backward(gyp, ind, H, H, 3, 3, 2, 2, 1, 1))
    nbytes = 4.0 * x.numel() + 4.0 * y.numel() + 8.0 * y.numel()
    out["maxpool_3x3s2_256x64x112x112"] = {"fwd_us": round(f * 1e3, 1), "bwd_us": round(bwd * 1e3, 1),
                                           "fwd_gbs": round(nbytes / f / 1e6, 1), "bwd_gbs": round(nbytes / bwd / 1e6, 1)}

    line = json.dumps(out)
    print(line)
    if args.out:
        with open(args.out, "w") as fh:
            fh.write(line + "\n")


if __name__ == "__main__":
    main()
