"""MobileNetV1 replica step (libTHCUNN.so, C ABI) against the same network composed from the CPU oracle's
operators, on a reduced configuration (64x64 input, 1/8 width, 10 classes) that the oracle finishes in
seconds.  Checks loss, every parameter gradient and the BN running statistics."""
import numpy as np
import pytest

from conftest import rel_err

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def oracle_step(ref, cfg_layout, params, images, labels1, inv_gb, momentum=0.1, eps=1e-5):
    """Forward + loss + backward with the oracle's operators.  Returns loss, grads, bn running stats."""
    from cunn_b200.mobilenet import KIND_DW, KIND_PW, KIND_STEM
    layers, fc = cfg_layout[:-1], cfg_layout[-1]
    grads = np.zeros_like(params)
    nbn = sum(2 * L["cout"] for L in layers)
    bn = np.zeros(nbn, np.float32)
    x = images
    saved = []
    for L in layers:
        co, ci = L["cout"], L["cin"]
        b = params[L["b_off"]:L["b_off"] + co]
        g, beta = params[L["g_off"]:L["g_off"] + co], params[L["beta_off"]:L["beta_off"] + co]
        s = L["stride"]
        if L["kind"] == KIND_DW:
            w = params[L["w_off"]:L["w_off"] + L["wcount"]].reshape(1, ci, 3, 3)
            y = ref.dwconv_forward(x, w, b.reshape(1, ci), s, s, 1, 1)
        elif L["kind"] == KIND_PW:
            w = params[L["w_off"]:L["w_off"] + L["wcount"]].reshape(co, ci, 1, 1)
            y = ref.convmm_forward(x, w, b, 1, 1, 0, 0)
        else:
            w = params[L["w_off"]:L["w_off"] + L["wcount"]].reshape(co, ci, 3, 3)
            y = ref.convmm_forward(x, w, b, s, s, 1, 1)
        z, rm, rv, sm, ss = ref.bn_forward(y, g, beta, np.zeros(co, np.float32), np.ones(co, np.float32), True, momentum, eps)
        bn[L["bn_off"]:L["bn_off"] + co] = rm
        bn[L["bn_off"] + co:L["bn_off"] + 2 * co] = rv
        a = ref.threshold_forward(z)
        saved.append((x, w, y, a, rm, rv, sm, ss, g))
        x = a
    fh = layers[-1]["hout"]
    pooled = ref.avgpool_forward(x, fh, fh, 1, 1, 0, 0)
    B = images.shape[0]
    feat, classes = fc["cin"], fc["cout"]
    wfc = params[fc["w_off"]:fc["w_off"] + fc["wcount"]].reshape(classes, feat, 1, 1)
    logits = ref.convmm_forward(pooled, wfc, params[fc["b_off"]:fc["b_off"] + classes], 1, 1, 0, 0).reshape(B, classes)
    lp = ref.logsoftmax_forward(logits)
    loss_sum, _ = ref.classnll_forward(lp, labels1, None, False)
    loss = loss_sum * inv_gb
    glp = ref.classnll_backward(labels1, 1.0 / inv_gb, B, classes, None, True)
    glogits = ref.logsoftmax_backward(lp, glp).reshape(B, classes, 1, 1)
    gw, gb = ref.convmm_acc_grad(pooled, glogits, np.zeros_like(wfc), np.zeros(classes, np.float32), 1, 1, 0, 0, 1.0)
    grads[fc["w_off"]:fc["w_off"] + fc["wcount"]] = gw.ravel()
    grads[fc["b_off"]:fc["b_off"] + classes] = gb
    g = ref.avgpool_backward(ref.convmm_grad_input(glogits, wfc, 1, 1, 1, 1, 0, 0), fh, fh, fh, fh, 1, 1, 0, 0)
    for L, (xin, w, y, a, rm, rv, sm, ss, gam) in zip(reversed(layers), reversed(saved)):
        co, ci, s = L["cout"], L["cin"], L["stride"]
        g = ref.threshold_backward(a, g)
        g, ggam, gbeta = ref.bn_backward(y, g, gam, rm, rv, sm, ss, True, 1.0, eps, gw=np.zeros(co, np.float32),
                                         gb=np.zeros(co, np.float32))
        grads[L["g_off"]:L["g_off"] + co] = ggam
        grads[L["beta_off"]:L["beta_off"] + co] = gbeta
        H = xin.shape[2]
        if L["kind"] == KIND_DW:
            gw, gb = ref.dwconv_acc_grad(xin, g, np.zeros_like(w), np.zeros((1, ci), np.float32), s, s, 1, 1, 1.0)
            gnext = ref.dwconv_grad_input(g, w, H, H, s, s, 1, 1)
        else:
            k, pad = (1, 0) if L["kind"] == KIND_PW else (3, 1)
            gw, gb = ref.convmm_acc_grad(xin, g, np.zeros_like(w), np.zeros(co, np.float32), s, s, pad, pad, 1.0)
            gnext = ref.convmm_grad_input(g, w, H, H, s, s, pad, pad) if L is not layers[0] else None
        grads[L["w_off"]:L["w_off"] + L["wcount"]] = gw.ravel()
        grads[L["b_off"]:L["b_off"] + co] = gb.ravel()
        g = gnext
    return loss, grads, bn


def test_mobilenet_step_matches_oracle(ref64, ref32):
    from cunn_b200 import mobilenet as mb, device_status
    cfg = mb.Config(64, 8, 10)
    lay = mb.layout(cfg)
    params = mb.init_params(cfg, seed=7)
    rng = np.random.default_rng(3)
    B, GB = 4, 8                                          # 4 local rows of a global batch of 8
    images = rng.standard_normal((B, 3, 64, 64)).astype(np.float32)
    labels1 = rng.integers(1, 11, B).astype(np.int64)     # 1-based, like Lua targets
    rep = mb.MobileNetV1(cfg, torch.device("cuda"), params, max_batch=B)
    rep.grads.fill_(0.5)                                  # gradients are ACCUMULATED into the buffer
    loss = rep.step(torch.from_numpy(images).cuda(), torch.from_numpy(labels1).cuda(), GB)
    torch.cuda.synchronize()
    assert device_status() == 0
    rloss, rgrads, rbn = oracle_step(ref64, lay, params, images, labels1, 1.0 / GB)
    assert float(loss) == pytest.approx(rloss, rel=1e-4)
    got = rep.grads.cpu().numpy() - 0.5
    # A 27-layer ReLU/BN network with a handful of samples per BN channel amplifies rounding differences
    # chaotically (one ReLU flipping near zero changes upstream gradients by per cent): the reference
    # algorithm's own fp32 CPU port differs from the fp64 oracle by 5-10 % on most tensors here.  So the
    # per-tensor bars are: the classifier (no amplification) tight, the median tight, the worst tensor sane,
    # and the GPU no further from the fp64 truth than the fp32 CPU port is.
    _, g32, _ = oracle_step(ref32, lay, params, images, labels1, 1.0 / GB)
    err_gpu, err_cpu32 = [], []
    for L in lay:
        off, cnt = L["w_off"], L["wcount"]
        want = rgrads[off:off + cnt]
        scale = max(float(np.abs(want).max()), 1e-12)
        err_gpu.append(float(np.abs(got[off:off + cnt] - want).max()) / scale)
        err_cpu32.append(float(np.abs(g32[off:off + cnt] - want).max()) / scale)
    assert err_gpu[-1] < 1e-3                                       # classifier weights
    assert float(np.median(err_gpu)) < max(1e-3, float(np.median(err_cpu32)))
    assert max(err_gpu) < max(0.25, 2 * max(err_cpu32))
    fc = lay[-1]
    assert rel_err(got[fc["b_off"]:fc["b_off"] + fc["cout"]], rgrads[fc["b_off"]:fc["b_off"] + fc["cout"]]) < 1e-3
    assert rel_err(rep.bn_running.cpu().numpy(), rbn) < 1e-3
    # SGD update: p -= lr * g
    before = rep.params.clone()
    rep.sgd(0.1)
    # the kernel may contract p - lr * g into one fused multiply-add: allow one rounding of the result
    assert torch.allclose(rep.params, before - 0.1 * rep.grads, rtol=2e-7, atol=1e-7)


def test_mobilenet_layout_matches_reference_parameter_count():
    # 4,242,920 parameters for width 1.0, 1000 classes (convolutions with bias, BN affine, Linear)
    from cunn_b200 import mobilenet as mb
    from cunn_b200._lib import lib
    import ctypes
    cfg = mb.Config(224, 1, 1000)
    assert lib.cunn_b200_mobilenet_param_count(ctypes.byref(cfg)) == 4242920
    lay = mb.layout(cfg)
    assert len(lay) == 28 and lay[-1]["kind"] == mb.KIND_FC and lay[-1]["hin"] == 7
    assert [L["stride"] for L in lay if L["kind"] == mb.KIND_DW] == [1, 2, 1, 2, 1, 2, 1, 1, 1, 1, 1, 2, 1]


def test_graph_replay_equals_direct_launches():
    # DataParallelStep(use_graph=True): the first two uses of a buffer pair launch directly (the second also
    # captures), the third replays the graph.  With learning rate 0 every step sees the same parameters, so the
    # replayed step must reproduce the loss exactly (the forward pass is deterministic) and the gradients up to the
    # summation order of the layers that add with atomics.
    from cunn_b200 import mobilenet as mb, device_status
    cfg = mb.Config(64, 8, 10)
    params = mb.init_params(cfg, seed=11)
    g = torch.Generator(device="cuda").manual_seed(2)
    B = 6
    images = torch.randn((B, 3, 64, 64), device="cuda", generator=g)
    labels = torch.randint(1, 11, (B,), device="cuda", dtype=torch.int64, generator=g)
    rep = mb.MobileNetV1(cfg, torch.device("cuda"), params, max_batch=B)
    step = mb.DataParallelStep(rep, None, use_graph=True)
    losses, grads, bn = [], [], []
    for _ in range(4):
        losses.append(float(step.train_step(images, labels, B, 0.0)))
        grads.append(rep.grads.clone())
        bn.append(rep.bn_running.clone())
    torch.cuda.synchronize()
    assert device_status() == 0
    assert len(step._graphs) == 1
    assert losses[2] == losses[0] and losses[3] == losses[0]
    scale = float(grads[0].abs().max())
    assert float((grads[2] - grads[0]).abs().max()) < 1e-5 * scale
    assert float((grads[3] - grads[0]).abs().max()) < 1e-5 * scale
    # the running statistics keep moving towards the batch statistics: step 3 continues from step 2
    assert not torch.equal(bn[2], bn[1]) and float((bn[3] - bn[2]).abs().max()) < float((bn[1] - bn[0]).abs().max()) * 1.0001
    # and with a learning rate the replayed steps train the network
    first = float(step.train_step(images, labels, B, 0.05))
    for _ in range(5):
        last = float(step.train_step(images, labels, B, 0.05))
    assert last < first
