#!/usr/bin/env python
"""Benchmark of the depthwise-convolution hot path: the 13 depthwise 3x3 layers of MobileNetV1, fp32 NCHW,
batch 64 per GPU, forward + input gradient + parameter gradient per layer.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = 39 kernel launches: all 13 forwards, then all 13 input gradients, then all 13 parameter
gradients.  The tensors of one step total 2.5 GB, so every kernel finds its inputs in HBM, not in L2.
With N > 1 (launched by torch.distributed.run, one rank per GPU) every rank runs the same stack on its
own batch of 64 images (weak scaling) and the ranks all-reduce the flat depthwise weight-gradient buffer
over NCCL at the end of each step, as the batch-sharded DataParallelTable does.

Prints ONE JSON line (rank 0).  `value` is whole-job algorithmic GB/s with inputs resident in HBM
(`single_stream` beside it: the same launches in one stream, as a network with dependent layers sees
them); `e2e` is the same metric through the THNN_Cuda* entry points with pinned host buffers,
host<->device copies timed; `roofline` describes the kernel launch that takes the most time;
`cpu_baseline` is the fp32 CPU port of the oracle timed on this box's host cores on the same 64 images;
`parity` holds the error figures of the benchmarked kernels against the fp64 oracle.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# (C, H=W, stride) of MobileNetV1's depthwise layers; the 512x14x14 stride-1 layer occurs five times.
LAYERS = [(32, 112, 1), (64, 112, 2), (128, 56, 1), (128, 56, 2), (256, 28, 1), (256, 28, 2),
          (512, 14, 1), (512, 14, 1), (512, 14, 1), (512, 14, 1), (512, 14, 1), (512, 14, 2), (1024, 7, 1)]
BATCH = 64
SEED = 1234
METRIC = "dwconv_fwd_bwd_hbm_gbs"

# DRAM traffic (read + write, MB) of one launch of the kernels that can top the per-launch time, from an
# ncu capture of this command's depthwise launches (key: "<op>_<layer>").
NCU_TRAFFIC_MB = {"wgrad_2": 261.3, "wgrad_1": 209.7, "fwd_2": 239.1, "dgrad_2": 199.1, "fwd_1": 155.1, "dgrad_1": 154.6,
                  "wgrad_3": 209.9, "fwd_3": 153.7, "dgrad_3": 153.2}


def out_size(hw, stride):
    return (hw + 2 - 3) // stride + 1


def layer_bytes(C, HW, stride, n):
    """Algorithmic bytes of one pass (forward, input gradient or parameter gradient) of one layer:
    4 bytes per element of the layer's input-side and output-side tensors."""
    o = out_size(HW, stride)
    return 4 * n * C * (HW * HW + o * o)


def step_bytes(n):
    return 3 * sum(layer_bytes(C, HW, s, n) for C, HW, s in LAYERS)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, uuid=None):
        self.proc = None
        self.file = None
        self.uuid = uuid

    def start(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            cmd = ["nvidia-smi", "--query-gpu=" + self.Q, "--format=csv,noheader,nounits", "-lms", "100"]
            if self.uuid:
                cmd += ["-i", self.uuid]
            self.proc = subprocess.Popen(cmd, stdout=self.file, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if not self.proc:
            return out
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        clocks, maxes, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                clocks.append(float(parts[0]))
                maxes.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.unlink(self.file.name)
        except OSError:
            pass
        if clocks:
            clocks.sort()
            out.update(sm_mhz=clocks[len(clocks) // 2], sm_max_mhz=max(maxes), reasons=sorted(reasons),
                       samples=len(clocks))
        return out


def make_host_inputs(n):
    """Seeded synthetic inputs of the workload: x ~ U(-1,1), weights and bias ~ U(-1/3, 1/3)
    (kaiming-uniform bound 1/sqrt(fan_in), fan_in = 9), gy ~ N(0,1)."""
    import numpy as np
    rng = np.random.default_rng(SEED)
    data = []
    for C, HW, s in LAYERS:
        o = out_size(HW, s)
        data.append(dict(
            x=rng.uniform(-1, 1, (n, C, HW, HW)).astype(np.float32),
            gy=rng.standard_normal((n, C, o, o), dtype=np.float32),
            w=rng.uniform(-1 / 3, 1 / 3, (1, C, 3, 3)).astype(np.float32),
            b=rng.uniform(-1 / 3, 1 / 3, (1, C)).astype(np.float32)))
    return data


def run_reference(args, emit):
    """--impl reference: the CPU arm.  torch/nn's CPU THNN (what the reference's tests compare with) is not
    part of the reference tree and the reference's own depthwise path is GPU code, so this times the fp32
    OpenMP port of the oracle on all host cores, on the full workload (64 images per layer), every step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    res = cpu_baseline(steps=args.steps, warmup=min(args.warmup, 1), budget_seconds=150.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": res["value"], "unit": "GB/s", "n_gpus": args.gpus,
        "steps": res["steps"], "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(res["sample_images"], 1),
        "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample", "pytorch_cpu") if k in res},
        "e2e": {"value": res["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def cpu_baseline(steps=1, warmup=0, budget_seconds=30.0):
    """Times the fp32 CPU port (oracle/thnn_ref.c, ref32_*) of the same 13-layer fwd+dgrad+wgrad stack on the
    full batch of 64 images per layer, on every host core (the OpenMP thread count is set explicitly:
    launchers export OMP_NUM_THREADS=1).  Runs `steps` steps, fewer only if they would exceed budget_seconds."""
    import numpy as np
    from oracle.thnn_ref import Ref
    ref = Ref("ref32_")
    cores = os.cpu_count() or 1
    threads = ref.set_threads(cores)

    def one_step(data):
        for (C, HW, s), d in zip(LAYERS, data):
            ref.dwconv_forward(d["x"], d["w"], d["b"], s, s, 1, 1)
        for (C, HW, s), d in zip(LAYERS, data):
            ref.dwconv_grad_input(d["gy"], d["w"], HW, HW, s, s, 1, 1)
        for (C, HW, s), d in zip(LAYERS, data):
            ref.dwconv_acc_grad(d["x"], d["gy"], np.zeros_like(d["w"]), np.zeros_like(d["b"]), s, s, 1, 1, 1.0)

    n = BATCH
    data = make_host_inputs(n)
    t0 = time.perf_counter()
    one_step(data)                                   # first touch of the pages, thread pool start
    first = time.perf_counter() - t0
    steps = int(max(1, min(steps, budget_seconds / max(first, 1e-3) - warmup - 1)))
    for _ in range(max(warmup - 1, 0)):
        one_step(data)
    t0 = time.perf_counter()
    for _ in range(steps):
        one_step(data)
    dt = (time.perf_counter() - t0) / steps
    out = {"value": step_bytes(n) / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
           "sample": "13-layer depthwise stack fwd+dgrad+wgrad on all %d images per layer, fp32 OpenMP port of the "
                     "oracle on %d threads, %d step(s)" % (n, threads, steps),
           "ms_per_step": dt * 1e3, "sample_images": n, "steps": steps}
    try:
        out["pytorch_cpu"] = pytorch_cpu_baseline(data, cores)
    except Exception as exc:                         # a secondary figure: never fails the run
        out["pytorch_cpu"] = {"unavailable": str(exc)[:200]}
    return out


def pytorch_cpu_baseline(data, threads):
    """A second CPU figure for the same stack: PyTorch's CPU operators (grouped conv2d and its two gradient functions, the
    living descendants of torch/nn's THNN CPU code), same tensors, same thread count, one warm-up and one timed step."""
    import torch
    import torch.nn.functional as Fn
    from torch.nn import grad as G
    old = torch.get_num_threads()
    torch.set_num_threads(threads)
    try:
        T = [dict(x=torch.from_numpy(d["x"]), gy=torch.from_numpy(d["gy"]), w=torch.from_numpy(d["w"]).permute(1, 0, 2, 3).contiguous(),
                  b=torch.from_numpy(d["b"]).reshape(-1)) for d in data]

        def one_step():
            with torch.no_grad():
                for (C, HW, s), t in zip(LAYERS, T):
                    Fn.conv2d(t["x"], t["w"], t["b"], stride=s, padding=1, groups=C)
                for (C, HW, s), t in zip(LAYERS, T):
                    G.conv2d_input(t["x"].shape, t["w"], t["gy"], stride=s, padding=1, groups=C)
                for (C, HW, s), t in zip(LAYERS, T):
                    G.conv2d_weight(t["x"], t["w"].shape, t["gy"], stride=s, padding=1, groups=C)
                    t["gy"].sum(dim=(0, 2, 3))
        one_step()
        t0 = time.perf_counter()
        one_step()
        dt = time.perf_counter() - t0
        n = data[0]["x"].shape[0]
        return {"value": step_bytes(n) / dt / 1e9, "unit": "GB/s", "threads": threads, "ms_per_step": dt * 1e3,
                "what": "torch %s CPU: F.conv2d(groups=C), torch.nn.grad.conv2d_input / conv2d_weight, bias gradient by sum" % torch.__version__}
    finally:
        torch.set_num_threads(old)


def parity_check(T, fwd, dgrad, wgrad, layers=(7, 12, 13)):
    """Runs three of the benchmarked layers (the 14x14 stride-1 and stride-2 and the 7x7 one, all 64 images) once
    more and compares y, gx and the parameter gradients with the fp64 oracle: worst tensor-normalised error
    max|got-want|/max|want| and worst element-wise relative error with a floor of 1e-3 max|want|."""
    import numpy as np
    import torch
    from oracle.thnn_ref import Ref
    ref = Ref("ref64_")
    ref.set_threads(os.cpu_count() or 1)

    def errs(got, want):
        got, want = got.astype(np.float64), want.astype(np.float64)
        m = float(np.max(np.abs(want)))
        d = np.abs(got - want)
        return float(d.max() / m), float(np.max(d / np.maximum(np.abs(want), 1e-3 * m)))

    worst = {"fwd": [0.0, 0.0], "grad": [0.0, 0.0]}
    for li in layers:
        t = T[li - 1]
        s, HW = t["s"], t["HW"]
        t["gw"].zero_()
        t["gb"].zero_()
        fwd(t)
        dgrad(t)
        wgrad(t)
        torch.cuda.synchronize()
        x, w, b, gy = (t[k].cpu().numpy() for k in ("x", "w", "b", "gy"))
        rgw, rgb = ref.dwconv_acc_grad(x, gy, np.zeros_like(w), np.zeros_like(b), s, s, 1, 1, 1.0)
        pairs = [("fwd", t["y"].cpu().numpy(), ref.dwconv_forward(x, w, b, s, s, 1, 1)),
                 ("grad", t["gx"].cpu().numpy(), ref.dwconv_grad_input(gy, w, HW, HW, s, s, 1, 1)),
                 ("grad", t["gw"].cpu().numpy(), rgw), ("grad", t["gb"].cpu().numpy(), rgb)]
        for kind, got, want in pairs:
            n, r = errs(got, want)
            worst[kind][0] = max(worst[kind][0], n)
            worst[kind][1] = max(worst[kind][1], r)
    return {"against": "fp64 CPU oracle, whole tensors, layers %s at batch %d" % (list(layers), BATCH),
            "forward": {"norm_err": worst["fwd"][0], "rel_err_floor_1e-3": worst["fwd"][1], "bar": 1e-5},
            "gradients": {"norm_err": worst["grad"][0], "rel_err_floor_1e-3": worst["grad"][1], "bar": 1e-4},
            "ok": worst["fwd"][0] <= 1e-5 and worst["grad"][0] <= 1e-4}


def workload_config(n, world):
    return {"workload": "MobileNetV1 depthwise stack: 13 SpatialDepthWiseConvolution 3x3 pad 1 layers, "
                        "fwd + updateGradInput + accGradParameters each",
            "batch_per_gpu": n, "global_batch": n * world, "layers": len(LAYERS),
            "layout": "NCHW fp32", "l2": "inputs larger than L2: one step touches 2.5 GB of tensors per GPU and a "
                                         "tensor is re-read only after >= 1.2 GB of other traffic",
            "parallelism": "dp%d (batch-sharded; ncclAllReduce of the depthwise weight gradients issued by the library's "
                           "DataParallelTable on a communication stream)" % world
                           if world > 1 else "single GPU",
            "launch": "39 kernels per step replayed from CUDA graphs, consecutive (independent) layers on alternating "
                      "streams; with N > 1 the weight-gradient all-reduce overlaps the input-gradient kernels",
            "timing": "rounds of exactly --steps steps, back to back for >= 1 s; ms_per_step is the mean over all rounds"}


def other_configs_bench(dev):
    """The other single-GPU configurations of the path, one kernel at a time (device-resident inputs, CUDA events on
    the launching stream, median of the repeats): im2col-GEMM convolution (ResNet-shaped 3x3 and 1x1 layers at
    batch 128, 3xTF32 on the tensor cores; TFLOP/s are fp32-equivalent: 2*N*K*C*kH*kW*oH*oW per pass) and batch
    normalisation + 3x3/2 max pooling at 256x64x112x112 (GB/s are algorithmic bytes: BN 2 tensors forward and 3
    backward, pooling input + output + int64 indices).  Buffers rotate so that successive launches never
    find their operands in L2."""
    import torch
    import cunn_b200.functional as F
    peak, _ = measured_peaks()
    gen = torch.Generator(device=dev)
    gen.manual_seed(SEED + 99)

    def timed(fn, nbuf, reps=5):
        for i in range(nbuf):
            fn(i)
        torch.cuda.synchronize()
        ts = []
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for i in range(nbuf):
                fn(i)
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) / nbuf)
        return sorted(ts)[len(ts) // 2]

    res = {}
    # ---- SpatialConvolutionMM --------------------------------------------------------------
    for name, (N, C, K, HW, k, pad) in (("convmm_3x3_256to256_14x14_n128", (128, 256, 256, 14, 3, 1)),
                                         ("convmm_1x1_1024to256_14x14_n128", (128, 1024, 256, 14, 1, 0))):
        nbuf = 6
        xs = [torch.randn((N, C, HW, HW), device=dev, generator=gen) for _ in range(nbuf)]
        gys = [torch.randn((N, K, HW, HW), device=dev, generator=gen) for _ in range(nbuf)]
        ys = [torch.empty((N, K, HW, HW), device=dev) for _ in range(nbuf)]
        gxs = [torch.empty((N, C, HW, HW), device=dev) for _ in range(nbuf)]
        w = torch.randn((K, C, k, k), device=dev, generator=gen) * (2.0 / (C * k * k)) ** 0.5
        b = torch.rand((K,), device=dev, generator=gen)
        gw, gb = torch.zeros_like(w), torch.zeros_like(b)
        flop = 2.0 * N * K * C * k * k * HW * HW
        ops = {"fwd": lambda i: F.convmm_forward(xs[i], w, b, 1, 1, pad, pad, out=ys[i]),
               "dgrad": lambda i: F.convmm_grad_input(gys[i], w, HW, HW, 1, 1, pad, pad, out=gxs[i]),
               "wgrad": lambda i: F.convmm_acc_grad(xs[i], gys[i], gw, gb, 1, 1, pad, pad, 1.0)}
        for op, fn in ops.items():
            ms = timed(fn, nbuf)
            res["%s_%s" % (name, op)] = {"us": round(ms * 1e3, 1), "value": round(flop / (ms * 1e-3) / 1e12, 1),
                                         "unit": "TFLOP/s fp32-equivalent (3xTF32 tcgen05)"}
        del xs, gys, ys, gxs
    # ---- BatchNormalization and SpatialMaxPooling --------------------------------------------
    N, C, HW = 256, 64, 112
    x = torch.randn((N, C, HW, HW), device=dev, generator=gen) * 2 + 0.5
    y = torch.empty_like(x)
    gy = torch.randn((N, C, HW, HW), device=dev, generator=gen)
    gx = torch.empty_like(x)
    gamma = torch.rand((C,), device=dev, generator=gen)
    beta = torch.zeros((C,), device=dev)
    rm, rv = torch.zeros((C,), device=dev), torch.ones((C,), device=dev)
    ggam, gbet = torch.zeros((C,), device=dev), torch.zeros((C,), device=dev)
    S = x.numel() * 4
    _, sm, ss = F.batchnorm_forward(x, gamma, beta, rm, rv, True, out=y)

    def put(key, ms, nbytes):
        gbs = nbytes / (ms * 1e-3) / 1e9
        res[key] = {"us": round(ms * 1e3, 1), "value": round(gbs, 0), "unit": "GB/s algorithmic",
                    "frac_of_measured_peak": round(gbs / peak, 3)}

    put("batchnorm_train_fwd_256x64x112x112", timed(lambda i: F.batchnorm_forward(x, gamma, beta, rm, rv, True, out=y, save_mean=sm, save_std=ss), 1), 2 * S)
    put("batchnorm_eval_fwd_256x64x112x112", timed(lambda i: F.batchnorm_forward(x, gamma, beta, rm, rv, False, out=y, save_mean=sm, save_std=ss), 1), 2 * S)
    put("batchnorm_train_bwd_256x64x112x112", timed(lambda i: F.batchnorm_backward(x, gy, gamma, rm, rv, sm, ss, True, grad_weight=ggam, grad_bias=gbet, out=gx), 1), 3 * S)
    oHW = F.maxpool_out_size(HW, 3, 2, 1, False)
    py = torch.empty((N, C, oHW, oHW), device=dev)
    pidx = torch.empty((N, C, oHW, oHW), device=dev, dtype=torch.int64)
    pgy = torch.randn((N, C, oHW, oHW), device=dev, generator=gen)
    pool_bytes = S + py.numel() * 4 + pidx.numel() * 8
    put("maxpool_3x3s2p1_fwd_256x64x112x112", timed(lambda i: F.maxpool_forward(y, 3, 3, 2, 2, 1, 1, False, out=py, indices=pidx), 1), pool_bytes)
    put("maxpool_3x3s2p1_bwd_256x64x112x112", timed(lambda i: F.maxpool_backward(pgy, pidx, HW, HW, 3, 3, 2, 2, 1, 1, False, out=gx), 1), pool_bytes)
    return res


def mobilenet_bench(args, dev, world, rank, dist):
    """Full MobileNetV1 (1.0, 224x224, 1000 classes) training step: forward, loss, backward, all-reduce of the
    flat gradient buffer, SGD update; global batch sharded over the ranks with DataParallelTable's slice rule.
    Returns images/s of the whole job (device-resident inputs) and the same with the shard's images copied
    from pinned host memory and the loss read back every step."""
    import torch
    from cunn_b200 import mobilenet as mb
    gb = args.mobilenet_batch
    cfg = mb.Config(224, 1, 1000)
    start, count = mb.slice_range(gb, world, rank)
    torch.manual_seed(SEED + 17 * rank)
    images = torch.randn((count, 3, 224, 224), device=dev)
    labels = torch.randint(1, 1001, (count,), device=dev, dtype=torch.int64)
    rep = mb.MobileNetV1(cfg, dev, mb.init_params(cfg, SEED), max_batch=max(count, 1))
    step = mb.DataParallelStep(rep, dist, use_graph=not args.no_graph, native=not args.torch_allreduce)   # forward + backward replayed from a CUDA graph
    warm, timed = 3, max(3, min(args.steps, 8))
    for _ in range(warm):
        step.train_step(images, labels, gb, 0.01)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(timed):
        loss = step.train_step(images, labels, gb, 0.01)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / timed
    # end to end: images from pinned host memory, loss back to the host, every step.  Two device buffers: the
    # copy of step i + 1's images runs on a second stream under step i's kernels, as an input pipeline would do it.
    himg = images.cpu().pin_memory()
    hlab = labels.cpu().pin_memory()
    hloss = torch.zeros(1).pin_memory()
    bufs = [(images, labels), (torch.empty_like(images), torch.empty_like(labels))]
    s_cmp, s_in = torch.cuda.current_stream(), torch.cuda.Stream(device=dev)
    ready = [torch.cuda.Event(), torch.cuda.Event()]      # buffer filled
    freed = [torch.cuda.Event(), torch.cuda.Event()]      # buffer consumed by the step that used it

    def fetch(i):
        b = i & 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(freed[b])
            bufs[b][0].copy_(himg, non_blocking=True)
            bufs[b][1].copy_(hlab, non_blocking=True)
            ready[b].record(s_in)

    if step.use_graph:                                    # the second input buffer gets its own graph: capture it untimed
        bufs[1][0].copy_(images)
        bufs[1][1].copy_(labels)
        for _ in range(2):
            step.train_step(bufs[1][0], bufs[1][1], gb, 0.01)
    for e in freed:
        e.record(s_cmp)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    fetch(0)
    for i in range(timed):
        if i + 1 < timed:
            fetch(i + 1)
        b = i & 1
        s_cmp.wait_event(ready[b])
        loss = step.train_step(bufs[b][0], bufs[b][1], gb, 0.01)
        freed[b].record(s_cmp)
        hloss.copy_(loss, non_blocking=True)
        s_cmp.synchronize()
    ems = (time.perf_counter() - t0) * 1e3 / timed
    if dist is not None:
        dist.all_reduce(loss)                             # the shards' scaled loss sums add up to the batch mean
        hloss.copy_(loss)
    if dist is not None:
        tt = torch.tensor([ms, ems], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, ems = float(tt[0]), float(tt[1])
    return {"img_s": round(gb / (ms * 1e-3), 1), "e2e_img_s": round(gb / (ems * 1e-3), 1), "global_batch": gb,
            "per_gpu_batch": count, "ms_per_step": round(ms, 3), "e2e_ms_per_step": round(ems, 3), "steps": timed,
            "loss": float(hloss[0]), "params": rep.nparams, "allreduce_bytes_per_step": rep.nparams * 4 if world > 1 else 0,
            "h2d_bytes_per_step": himg.numel() * 4 + hlab.numel() * 8,
            "step": "fwd + NLL loss + bwd + gradient all-reduce + SGD, fp32, BN statistics per shard",
            "launch": "forward + loss + backward replayed from one CUDA graph" if step.use_graph else "direct launches"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--min-seconds", type=float, default=1.0,
                    help="the timed region repeats rounds of --steps steps until it has lasted about this long")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--graph-streams", type=int, default=2,
                    help="streams the launches of the depthwise stack alternate between inside the CUDA graph")
    ap.add_argument("--torch-allreduce", action="store_true",
                    help="exchange gradients with torch.distributed.all_reduce instead of the library's DataParallelTable")
    ap.add_argument("--no-mobilenet", action="store_true")
    ap.add_argument("--no-others", action="store_true", help="skip the single-kernel timings of the GEMM convolution, batch norm and pooling")
    ap.add_argument("--mobilenet-batch", type=int, default=1024, help="global batch of the MobileNetV1 step")
    args = ap.parse_args()
    # Libraries (NCCL's version banner) may write to stdout; the one JSON line must be alone there.  File descriptor 1
    # points at stderr while the benchmark runs and `emit` writes the line to the real stdout.
    real_stdout = os.dup(1)
    sys.stdout.flush()
    os.dup2(2, 1)

    def emit(obj):
        sys.stdout.flush()
        os.write(real_stdout, (json.dumps(obj) + "\n").encode())

    if args.impl == "reference":
        run_reference(args, emit)
        return

    import torch
    import torch.distributed as dist
    import cunn_b200.functional as F
    from cunn_b200 import device_status

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    warmup = max(args.warmup, 3)
    steps = max(args.steps, 1)

    # ---- device-resident tensors -------------------------------------------------------------------
    gen = torch.Generator(device=dev)
    gen.manual_seed(SEED + rank)
    nparams = sum(C * 10 for C, _, _ in LAYERS)
    flat_grad = torch.zeros(nparams, device=dev)       # [gw | gb] per layer, the DataParallelTable flat layout
    T, off = [], 0
    for C, HW, s in LAYERS:
        o = out_size(HW, s)
        t = dict(C=C, HW=HW, s=s, o=o,
                 x=torch.rand((BATCH, C, HW, HW), device=dev, generator=gen) * 2 - 1,
                 gy=torch.randn((BATCH, C, o, o), device=dev, generator=gen),
                 w=(torch.rand((1, C, 3, 3), device=dev, generator=gen) * 2 - 1) / 3,
                 b=(torch.rand((1, C), device=dev, generator=gen) * 2 - 1) / 3,
                 y=torch.empty((BATCH, C, o, o), device=dev),
                 gx=torch.empty((BATCH, C, HW, HW), device=dev),
                 gw=flat_grad[off:off + 9 * C].view(1, C, 3, 3),
                 gb=flat_grad[off + 9 * C:off + 10 * C].view(1, C))
        off += 10 * C
        T.append(t)

    def fwd(t):
        F.dwconv_forward(t["x"], t["w"], t["b"], t["s"], t["s"], 1, 1, out=t["y"])

    def dgrad(t):
        F.dwconv_grad_input(t["gy"], t["w"], t["HW"], t["HW"], t["s"], t["s"], 1, 1, out=t["gx"])

    def wgrad(t):
        F.dwconv_acc_grad(t["x"], t["gy"], t["gw"], t["gb"], t["s"], t["s"], 1, 1, 1.0)

    OPS = [("fwd", fwd), ("dgrad", dgrad), ("wgrad", wgrad)]

    def kernels():
        for _, op in OPS:
            for t in T:
                op(t)

    launches_per_step = len(OPS) * len(T)
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    kernels()                       # first call: workspace allocation, function attributes
    torch.cuda.synchronize()
    # The layers of the stack are independent of each other, so inside a graph consecutive launches alternate
    # between the capture stream and side streams: the ramp-up of one kernel overlaps the tail of the one before.
    # Every stream has its own scratch buffer (cunn_b200.functional.workspace), allocated here, outside the capture.
    side = [torch.cuda.Stream(device=dev) for _ in range(max(args.graph_streams, 1) - 1)]
    for s2 in side:
        with torch.cuda.stream(s2):
            kernels()
    torch.cuda.synchronize()
    # One CUDA graph per step on one GPU.  With several ranks the step is two graphs: forwards and
    # parameter gradients first, then the input gradients, so that the NCCL all-reduce of the flat
    # weight-gradient buffer (issued between them, on NCCL's own stream) overlaps the input-gradient kernels;
    # the step ends when both have finished.
    def part(names, streams=()):
        for s2 in streams:
            s2.wait_stream(stream)
        i = 0
        for name, op in OPS:
            if name in names:
                for t in T:
                    k = i % (len(streams) + 1)
                    i += 1
                    if k == 0:
                        op(t)
                    else:
                        with torch.cuda.stream(streams[k - 1]):
                            op(t)
        for s2 in streams:
            stream.wait_stream(s2)

    graphs = None
    table = None
    if world > 1 and not args.torch_allreduce:
        # The exchange runs in the library's DataParallelTable: ncclAllReduce of the local gradient buffer on a
        # communication stream behind an event, then visible += sum, local = 0 (DataParallelTable.lua:247-265).
        from cunn_b200 import dpt
        uid = torch.zeros(128, dtype=torch.uint8, device=dev)
        if rank == 0:
            uid.copy_(torch.frombuffer(bytearray(dpt.unique_id()), dtype=torch.uint8))
        dist.broadcast(uid, src=0)
        visible_grad = torch.zeros_like(flat_grad)
        scratch_params = torch.zeros_like(flat_grad)
        table = dpt.NativeDataParallelTable().add_rank(nparams, local_rank, rank, world, bytes(uid.cpu().numpy().tobytes()))
        table.set_buffers(0, scratch_params.data_ptr(), flat_grad.data_ptr(), visible_grad.data_ptr())
        table.set_stream(0, stream.cuda_stream)
        table.reduce()                  # creates the NCCL channels up front
        torch.cuda.synchronize()
    elif world > 1:
        dist.all_reduce(flat_grad)      # creates the NCCL communicator up front
        torch.cuda.synchronize()
    if not args.no_graph:
        parts = [("fwd", "dgrad", "wgrad")] if world == 1 else [("fwd", "wgrad"), ("dgrad",)]
        graphs = []
        for names in parts:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                part(names, side)
            graphs.append(g)

    def step():
        if world == 1:
            if graphs:
                graphs[0].replay()
            else:
                kernels()
            return
        if graphs:
            graphs[0].replay()
        else:
            part(("fwd", "wgrad"))
        if table is not None:
            table.bucketReady(0, 0)     # event on the compute stream; the all-reduce starts behind it on the comm stream
        else:
            work = dist.all_reduce(flat_grad, async_op=True)
        if graphs:
            graphs[1].replay()
        else:
            part(("dgrad",))
        if table is not None:
            table.reduce()              # compute stream waits for the collective, folds the sum into the visible buffer
        else:
            work.wait()                 # the compute stream waits for the collective; the host does not

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(str(torch.cuda.get_device_properties(dev).uuid)) if rank == 0 else None
    if sampler:
        sampler.uuid = "GPU-" + sampler.uuid if not sampler.uuid.startswith("GPU-") else sampler.uuid
        sampler.start()
    torch.cuda.synchronize()
    # The timed region is `rounds` back-to-back rounds of exactly `steps` steps each, enough rounds to last
    # about args.min_seconds, so that the clocks are sampled over a sustained run; CUDA events bracket every
    # round and the reported time per step is the mean over all of them.
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record()
    for _ in range(steps):
        step()
    p1.record()
    torch.cuda.synchronize()
    probe_ms = max(p0.elapsed_time(p1), 1e-3)
    rounds = int(max(1, min(2000, -(-args.min_seconds * 1e3 // probe_ms))))
    if world > 1:
        rt = torch.tensor([rounds], device=dev)
        dist.all_reduce(rt, op=dist.ReduceOp.MAX)
        rounds = int(rt.item())
        dist.barrier()
    torch.cuda.synchronize()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(rounds + 1)]
    marks[0].record()
    for r in range(rounds):
        for _ in range(steps):
            step()
        marks[r + 1].record()
    torch.cuda.synchronize()
    ms = marks[0].elapsed_time(marks[rounds])
    round_ms = sorted(marks[r].elapsed_time(marks[r + 1]) / steps for r in range(rounds))
    clocks = sampler.stop() if sampler else None
    if world > 1:
        dist.barrier()
        tt = torch.tensor([ms], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms = float(tt.item())
    ms_per_step = ms / (steps * rounds)
    timed = {"rounds": rounds, "steps_per_round": steps, "total_ms": round(ms, 2),
             "ms_per_step_best_round": round(round_ms[0], 4), "ms_per_step_median_round": round(round_ms[rounds // 2], 4),
             "ms_per_step_worst_round": round(round_ms[-1], 4)}
    value = step_bytes(BATCH) * world / (ms_per_step * 1e-3) / 1e9

    # ---- the graphs compute what direct launches on one stream compute ------------------------------
    verified = None
    single_stream = None
    if graphs:
        flat_grad.zero_()
        step()
        torch.cuda.synchronize()
        got = [(t["y"].clone(), t["gx"].clone()) for t in T]
        got_grad = flat_grad.clone()
        for t in T:
            t["y"].zero_()
            t["gx"].zero_()
        flat_grad.zero_()
        kernels()
        torch.cuda.synchronize()
        bad = [i + 1 for i, ((y, gx), t) in enumerate(zip(got, T)) if not (torch.equal(y, t["y"]) and torch.equal(gx, t["gx"]))]
        # parameter gradients are summed with atomics in some layers: compare against the largest gradient
        gerr = float((got_grad - flat_grad).abs().max() / flat_grad.abs().max()) if world == 1 else 0.0
        verified = not bad and gerr < 1e-5   # with several ranks the graph step also sums the gradients over the ranks
        del got, got_grad
        if not verified:
            raise SystemExit("bench: the graph replay and direct launches disagree (layers %s, gradient error %.3g)" % (bad, gerr))
        if side and world == 1:
            # the same step with every launch on one stream, for comparison
            g1 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g1, stream=stream):
                part(("fwd", "dgrad", "wgrad"))
            for _ in range(warmup):
                g1.replay()
            torch.cuda.synchronize()
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record()
            for _ in range(steps * rounds):
                g1.replay()
            s1.record()
            torch.cuda.synchronize()
            sms = s0.elapsed_time(s1) / (steps * rounds)
            peak1, _ = measured_peaks()
            single_stream = {"ms_per_step": round(sms, 4), "value": round(step_bytes(BATCH) / (sms * 1e-3) / 1e9, 1),
                             "unit": "GB/s", "frac_of_peak": round(step_bytes(BATCH) / (sms * 1e-3) / 1e9 / peak1, 4),
                             "note": "the same 39 launches replayed from a graph in ONE stream"}

    # ---- per-kernel durations ---------------------------------------------------------------------------
    # Every one of the 39 launches is timed on the device, apart from the others: a CUDA graph holds the launch repeated
    # over `nrot` rotating sets of the layer's tensors (enough sets that a set is touched again only after >= 400 MB of
    # other traffic, so the inputs come from HBM, not from L2), the graph is replayed back to back between two CUDA events
    # on the launching stream, and the duration is the mean per launch.  (Timing direct launches with an event after each
    # measures the host's launch rate for the kernels shorter than ~16 us, not the GPU.)
    per = []
    kreps = max(3, min(steps, 10))
    with torch.cuda.stream(stream):
        for name, op in OPS:
            for li, t in enumerate(T):
                nbytes = layer_bytes(t["C"], t["HW"], t["s"], BATCH)
                nrot = max(1, -(-400_000_000 // nbytes))
                sets = [t]
                for _ in range(nrot - 1):
                    r = dict(t)
                    r["x"], r["gy"] = t["x"].clone(), t["gy"].clone()
                    r["y"], r["gx"] = torch.empty_like(t["y"]), torch.empty_like(t["gx"])
                    sets.append(r)
                for r in sets:
                    op(r)
                torch.cuda.synchronize()
                if args.no_graph:
                    def run(sets=sets, op=op):
                        for r in sets:
                            op(r)
                else:
                    gk = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(gk, stream=stream):
                        for r in sets:
                            op(r)
                    run = gk.replay
                run()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                e0.record()
                for _ in range(kreps):
                    run()
                e1.record()
                torch.cuda.synchronize()
                d = e0.elapsed_time(e1) / (kreps * nrot)
                per.append(dict(op=name, layer=li + 1, C=t["C"], HW=t["HW"], stride=t["s"], ms=d, bytes=nbytes, sets=nrot))
                del sets
    peak, peak_kind = measured_peaks()
    top = max(per, key=lambda k: k["ms"])
    achieved = top["bytes"] / (top["ms"] * 1e-3) / 1e9
    key = "%s_%d" % (top["op"], top["layer"])
    traffic = NCU_TRAFFIC_MB.get(key)
    roofline = {"bound": "hbm", "kernel": "dwconv %s, layer %d (C=%d, %dx%d, stride %d)" %
                (top["op"], top["layer"], top["C"], top["HW"], top["HW"], top["stride"]),
                "achieved": round(achieved, 1), "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                "frac": round(achieved / peak, 4),
                "traffic": None if traffic is None else traffic * 1e6,
                "algorithmic_bytes": top["bytes"], "launch_ms": round(top["ms"], 5),
                "step": {"achieved": round(step_bytes(BATCH) / (ms_per_step * 1e-3) / 1e9 if world == 1 else
                                           value / world, 1),
                         "frac": round((value / world) / peak, 4),
                         "note": "all 39 launches: algorithmic bytes / graph-replay time per step; consecutive launches "
                                 "alternate between %d streams inside the graph" % (len(side) + 1),
                         "single_stream": single_stream, "matches_direct_launches": verified},
                "per_kernel_method": "each launch alone, replayed back to back from a CUDA graph over rotating tensor sets "
                                     "(>= 400 MB between two uses of a set), mean device time per launch",
                "per_kernel": [dict(op=k["op"], layer=k["layer"], us=round(k["ms"] * 1e3, 2),
                                    gbs=round(k["bytes"] / (k["ms"] * 1e-3) / 1e9, 0),
                                    frac=round(k["bytes"] / (k["ms"] * 1e-3) / 1e9 / peak, 3)) for k in per]}

    # ---- end to end through the THNN_Cuda* entry points with host buffers -----------------------------
    # The calls a Lua module makes: THNN_CudaSpatialDepthWiseConvolution_updateOutput / _updateGradInput /
    # _accGradParameters on tensor structs (lib/THCUNN/generic/THCUNN.h:667-702), outputs resized by the callee.
    e2e = None
    H = None
    if not args.no_e2e:
        import numpy as np
        from cunn_b200 import thnn
        nnb = thnn.THNN()
        esteps = max(1, min(steps, 3))
        H = []
        for t in T:
            H.append(dict(x=t["x"].cpu().pin_memory(), gy=t["gy"].cpu().pin_memory(),
                          y=torch.empty(t["y"].shape).pin_memory(), gx=torch.empty(t["gx"].shape).pin_memory()))
        hgrad = torch.empty(nparams).pin_memory()
        h2d = sum(h["x"].numel() + h["gy"].numel() for h in H) * 4
        d2h = sum(h["y"].numel() + h["gx"].numel() for h in H) * 4 + nparams * 4

        # Three streams: host->device copies, kernels, device->host copies.  PCIe is full duplex, so layer
        # i's results travel back while layer i+1's inputs travel in; events order copy -> compute -> copy.
        s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        s_cmp = torch.cuda.current_stream()

        def e2e_step():
            s_in.wait_stream(s_cmp)
            s_out.wait_stream(s_cmp)
            for t, h in zip(T, H):
                with torch.cuda.stream(s_in):
                    t["x"].copy_(h["x"], non_blocking=True)
                    t["gy"].copy_(h["gy"], non_blocking=True)
                    ev_in = torch.cuda.Event()
                    ev_in.record(s_in)
                s_cmp.wait_event(ev_in)
                st = t["s"]
                y = nnb.SpatialDepthWiseConvolution_updateOutput(t["x"], t["w"], t["b"], 3, 3, st, st, 1, 1)
                gx = nnb.SpatialDepthWiseConvolution_updateGradInput(t["x"], t["gy"], t["w"], 3, 3, st, st, 1, 1)
                nnb.SpatialDepthWiseConvolution_accGradParameters(t["x"], t["gy"], t["gw"], t["gb"], 3, 3, st, st, 1, 1, 1.0)
                ev_c = torch.cuda.Event()
                ev_c.record(s_cmp)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_c)
                    h["y"].copy_(y, non_blocking=True)
                    h["gx"].copy_(gx, non_blocking=True)
                    y.record_stream(s_out)
                    gx.record_stream(s_out)
            if world > 1:
                dist.all_reduce(flat_grad)
            hgrad.copy_(flat_grad, non_blocking=True)
            s_cmp.wait_stream(s_out)
            s_cmp.synchronize()

        e2e_step()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(esteps):
            e2e_step()
        a1.record()
        torch.cuda.synchronize()
        ems = max(a0.elapsed_time(a1), (time.perf_counter() - t0) * 1e3)
        if world > 1:
            tt = torch.tensor([ems], device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ems = float(tt.item())
        nnb.close()
        e2e = {"value": round(step_bytes(BATCH) * world / (ems / esteps * 1e-3) / 1e9, 2), "unit": "GB/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": esteps,
               "ms_per_step": round(ems / esteps, 3),
               "api": "THNN_CudaSpatialDepthWiseConvolution_updateOutput / _updateGradInput / _accGradParameters"}

    # ---- the benchmarked kernels against the fp64 oracle (checker only; part of the CPU leg) --------------
    parity = None
    if rank == 0 and world == 1 and not args.no_cpu:
        parity = parity_check(T, fwd, dgrad, wgrad)

    # ---- MobileNetV1 training step, batch-sharded over the ranks ------------------------------------
    mbn = None
    if not args.no_mobilenet:
        mbn = mobilenet_bench(args, dev, world, rank, dist if world > 1 else None)

    others = None
    if world == 1 and not args.no_others:
        del T, H
        torch.cuda.empty_cache()
        others = other_configs_bench(dev)

    status = device_status()
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        c = cpu_baseline(steps=3, warmup=1, budget_seconds=30.0)
        cpu = {k: (round(c[k], 3) if isinstance(c[k], float) else c[k]) for k in ("value", "unit", "cores", "kind", "sample")}
        pc = c.get("pytorch_cpu")
        if pc:
            cpu["pytorch_cpu"] = {k: (round(v, 3) if isinstance(v, float) else v) for k, v in pc.items()}

    if rank == 0:
        line = {"metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": steps,
                "warmup": warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_config(BATCH, world),
                "clocks": clocks, "timed": timed, "single_stream": single_stream, "e2e": e2e,
                "gpu_launches": launches_per_step * steps * rounds, "parity": parity,
                "roofline": roofline, "cpu_baseline": cpu, "mobilenet_v1": mbn, "other_configs": others, "device_status": status}
        emit(line)
    if table is not None:
        table.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
