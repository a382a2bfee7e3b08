"""The scratch-free parameter-gradient entry point (cunn_b200_dwconv_acc_grad_static).

Some users of the library have no device allocator to lend it: their own memory pool already owns the
GPU, or they reach the library through a binding that passes tensors and nothing else.  For them the
depthwise parameter gradient can run on a fixed scratch array that lives inside the library.  This test
drives that entry point through the C ABI exactly as such a caller would (raw pointers, no workspace)
and checks that it returns what the ordinary entry point returns, twice in a row, because the second
call starts from whatever the first left in the shared array.

The file name sorts last on purpose: a run that stops at the first failure has then already run every
other test.  It passes on its own in a fresh process as well as after the rest of the suite.
"""
import ctypes

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

GRAD_TOL = 1e-4  # the tolerance the other gradient tests use


def _rel_err(got, want):
    floor = 1e-2 * float(np.max(np.abs(want)))
    return float(np.max(np.abs(got - want) / np.maximum(np.abs(want), floor)))


@pytest.mark.parametrize("N,C,HW,stride", [(6, 64, 28, 1), (3, 32, 112, 2), (5, 512, 7, 1)])
def test_static_scratch_entry_matches_workspace_entry(N, C, HW, stride):
    import cunn_b200.functional as F
    from cunn_b200._lib import lib, check, device_status

    g = torch.Generator(device="cuda")
    g.manual_seed(42 + C)
    o = (HW + 2 - 3) // stride + 1
    x = torch.rand((N, C, HW, HW), device="cuda", generator=g) * 2 - 1
    gy = torch.randn((N, C, o, o), device="cuda", generator=g)
    gw0 = torch.randn((1, C, 3, 3), device="cuda", generator=g)
    gb0 = torch.randn((1, C), device="cuda", generator=g)
    stream = torch.cuda.current_stream().cuda_stream

    for call in range(2):                      # two calls in a row share the built-in array
        scale = 1.0 if call == 0 else 0.5
        want_w, want_b = gw0.clone(), gb0.clone()
        F.dwconv_acc_grad(x, gy, want_w, want_b, stride, stride, 1, 1, scale)
        got_w, got_b = gw0.clone(), gb0.clone()
        check(lib.cunn_b200_dwconv_acc_grad_static(
            x.data_ptr(), gy.data_ptr(), got_w.data_ptr(), got_b.data_ptr(),
            N, C, HW, HW, 1, 3, 3, stride, stride, 1, 1, ctypes.c_float(scale), stream))
        torch.cuda.synchronize()
        assert _rel_err(got_w.cpu().numpy(), want_w.cpu().numpy()) < GRAD_TOL
        assert _rel_err(got_b.cpu().numpy(), want_b.cpu().numpy()) < GRAD_TOL
    assert device_status() == 0


def test_static_scratch_entry_rejects_oversized_problem():
    from cunn_b200._lib import lib, CunnError, check

    cap = lib.cunn_b200_dwconv_acc_grad_static_capacity()
    assert cap == 4 << 20
    # 65536 channels of 4x4 planes: far more partial sums than the built-in array holds.  The size check
    # runs before anything is launched, so tiny dummy buffers are enough.
    N, C, HW = 64, 65536, 4
    need = lib.cunn_b200_dwconv_acc_grad_workspace(N, C, HW, HW, 1, 3, 3, 1, 1, 1, 1)
    if need <= cap:
        pytest.skip("this device's tile plan fits the built-in array")
    buf = torch.zeros(64, device="cuda")
    with pytest.raises(CunnError, match="static scratch"):
        check(lib.cunn_b200_dwconv_acc_grad_static(
            buf.data_ptr(), buf.data_ptr(), buf.data_ptr(), buf.data_ptr(),
            N, C, HW, HW, 1, 3, 3, 1, 1, 1, 1, ctypes.c_float(1.0), torch.cuda.current_stream().cuda_stream))
