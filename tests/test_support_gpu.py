"""Support operators of the MobileNetV1 step (Threshold, SpatialAveragePooling, LogSoftMax, ClassNLLCriterion,
SGD update): CUDA kernels against the oracle and the committed fixtures."""
import numpy as np
import pytest

from conftest import golden, rel_err

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.detach().cpu().numpy()


@pytest.fixture(scope="module")
def F():
    import cunn_b200.functional as F
    return F


def test_threshold(F, ref64):
    rng = np.random.default_rng(0)
    for n in (1, 7, 1024, 100003):
        x = rng.standard_normal(n).astype(np.float32)
        gy = rng.standard_normal(n).astype(np.float32)
        assert np.array_equal(host(F.threshold_forward(dev(x))), ref64.threshold_forward(x))
        assert np.array_equal(host(F.threshold_backward(dev(x), dev(gy))), ref64.threshold_backward(x, gy))
        assert np.array_equal(host(F.threshold_forward(dev(x), 0.5, -2.0)), ref64.threshold_forward(x, 0.5, -2.0))
    xd = dev(x)
    F.threshold_forward(xd, out=xd)                       # in place, as nn.ReLU(true) does
    assert np.array_equal(host(xd), np.maximum(x, 0))


def test_support_golden(F, ref64):
    g = golden("support")
    lp = F.logsoftmax_forward(dev(g["x"]))
    assert rel_err(host(lp), g["lp"]) < 1e-5
    tgt = dev(g["target0"] + ref64.index_base)
    out = F.classnll_forward(lp, tgt)
    assert abs(float(out[0]) - float(g["loss"])) < 1e-5 * abs(float(g["loss"])) and float(out[1]) == 5.0
    gl = F.classnll_backward(tgt, out, 5, 1000)
    assert rel_err(host(F.logsoftmax_backward(lp, gl)), g["gx"]) < 1e-4
    assert rel_err(host(F.avgpool_forward(dev(g["a"]), 7, 7, 1, 1, 0, 0)), g["ap"]) < 1e-5
    assert rel_err(host(F.avgpool_backward(dev(g["gap"]), 7, 7, 7, 7, 1, 1, 0, 0)), g["ga"]) < 1e-5
    assert rel_err(host(F.avgpool_forward(dev(g["a2"]), 3, 3, 2, 2, 1, 1)), g["ap2"]) < 1e-5
    assert rel_err(host(F.avgpool_backward(dev(g["gap2"]), 9, 10, 3, 3, 2, 2, 1, 1)), g["ga2"]) < 1e-5


def test_avgpool_includepad_known_answer(F):
    # the reference's known-answer test (test.lua:2597-2616)
    x = torch.full((1, 1, 2, 2), 3.0, device="cuda")
    inc = host(F.avgpool_forward(x, 2, 2, 1, 1, 1, 1, count_include_pad=True))
    exc = host(F.avgpool_forward(x, 2, 2, 1, 1, 1, 1, count_include_pad=False))
    assert inc[0, 0, 0, 0] == pytest.approx(0.75) and exc[0, 0, 0, 0] == pytest.approx(3.0) and inc[0, 0, 1, 1] == pytest.approx(3.0)


def test_classnll_ignore_index_and_weights(F, ref64):
    rng = np.random.default_rng(5)
    B, D = 37, 11
    lp = np.log(rng.dirichlet(np.ones(D), B)).astype(np.float32)
    tgt = rng.integers(1, D + 1, B).astype(np.int64)
    w = rng.uniform(0.5, 2, D).astype(np.float32)
    for size_average in (True, False):
        for ign in (-100, 3):
            rl, rtw = ref64.classnll_forward(lp, tgt, w, size_average, ign)
            out = F.classnll_forward(dev(lp), dev(tgt), dev(w), size_average, ign)
            assert float(out[0]) == pytest.approx(rl, rel=1e-5) and float(out[1]) == pytest.approx(rtw, rel=1e-6)
            rg = ref64.classnll_backward(tgt, rtw, B, D, w, size_average, ign)
            g = F.classnll_backward(dev(tgt), out, B, D, dev(w), size_average, ign)
            assert rel_err(host(g), rg) < 1e-5


def test_sgd_update(F):
    p = torch.arange(10, dtype=torch.float32, device="cuda")
    g = torch.ones(10, device="cuda") * 2
    F.sgd_update(p, g, 0.25)
    assert torch.equal(p.cpu(), torch.arange(10, dtype=torch.float32) - 0.5)
