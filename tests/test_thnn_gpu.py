"""THNN_Cuda* entry points (the reference's C ABI, tensor structs, callee-resized outputs, error hook)
against the fp64 CPU oracle.  Mirrors what the reference's tests exercise at this level: strided inputs,
views that start inside their storage, 3-D (unbatched) inputs, bias / no bias, accumulate with scale.
Bars: forward 1e-5, gradients and GEMM-path results 1e-4 (conftest.rel_err), pooling indices identical."""
import numpy as np
import pytest

from conftest import rel_err

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nnb():
    from cunn_b200 import thnn
    b = thnn.THNN()
    yield b
    b.close()


def non_contiguous(t):
    """Same values, strided memory (the reference's makeNonContiguous, test.lua:62-83)."""
    big = torch.empty(t.shape + (2,), device=t.device, dtype=t.dtype)
    big[..., 0] = t
    return big[..., 0]


def offset_view(t):
    """Same values in a view that starts 3 elements into its storage (Lua tensors carry such offsets)."""
    buf = torch.empty(t.numel() + 3, device=t.device, dtype=t.dtype)
    v = buf[3:].view(t.shape)
    v.copy_(t)
    assert v.storage_offset() == 3
    return v


def H(t):
    return None if t is None else t.detach().cpu().numpy()


def close(a, b, tol=1e-5):
    """a: device tensor from the entry point; b: oracle array (or a device tensor)."""
    b = H(b) if isinstance(b, torch.Tensor) else np.asarray(b)
    return rel_err(H(a).reshape(b.shape), b) <= tol


def test_depthwise_entry_points(nnb, ref64):
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.rand((3, 6, 14, 14), device="cuda", generator=g)
    w = torch.rand((2, 6, 3, 3), device="cuda", generator=g) - 0.5
    b = torch.rand((2, 6), device="cuda", generator=g)
    ry = ref64.dwconv_forward(H(x), H(w), H(b), 1, 1, 1, 1)
    for xin in (x, non_contiguous(x), offset_view(x)):
        y = nnb.SpatialDepthWiseConvolution_updateOutput(xin, w, b, 3, 3, 1, 1, 1, 1)
        assert tuple(y.shape) == (3, 12, 14, 14)
        assert close(y, ry)
    # 2-D weight [M, C*kH*kW] is accepted; no bias
    y = nnb.SpatialDepthWiseConvolution_updateOutput(x, w.view(2, 54), None, 3, 3, 2, 2, 1, 1)
    assert close(y, ref64.dwconv_forward(H(x), H(w), None, 2, 2, 1, 1))
    # unbatched input gives a 3-D output
    y3 = nnb.SpatialDepthWiseConvolution_updateOutput(x[0], w, b, 3, 3, 1, 1, 1, 1)
    assert tuple(y3.shape) == (12, 14, 14) and close(y3, ry[0])
    # a strided gradOutput: the reference views it as if it were contiguous
    # (generic/SpatialDepthWiseConvolution.cu:285-297); here its values are used
    gy = torch.randn((3, 12, 14, 14), device="cuda", generator=g)
    gx = nnb.SpatialDepthWiseConvolution_updateGradInput(x, non_contiguous(gy), w, 3, 3, 1, 1, 1, 1)
    assert close(gx, ref64.dwconv_grad_input(H(gy), H(w), 14, 14, 1, 1, 1, 1), 1e-4)
    gw, gb = torch.ones_like(w), torch.ones_like(b)
    nnb.SpatialDepthWiseConvolution_accGradParameters(x, non_contiguous(gy), gw, gb, 3, 3, 1, 1, 1, 1, 0.5)
    rw, rb = ref64.dwconv_acc_grad(H(x), H(gy), np.ones(w.shape, np.float32), np.ones(b.shape, np.float32), 1, 1, 1, 1, 0.5)
    assert close(gw, rw, 1e-4) and close(gb, rb, 1e-4)


def test_convmm_entry_points(nnb, ref64):
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn((2, 8, 10, 9), device="cuda", generator=g)
    w = torch.randn((16, 8, 3, 3), device="cuda", generator=g) * 0.1
    b = torch.randn(16, device="cuda", generator=g)
    y = nnb.SpatialConvolutionMM_updateOutput(non_contiguous(x), w.view(16, 72), b, 3, 3, 1, 1, 1, 1)
    assert tuple(y.shape) == (2, 16, 10, 9) and close(y, ref64.convmm_forward(H(x), H(w), H(b), 1, 1, 1, 1), 1e-4)
    gy = torch.randn_like(y)
    gx = nnb.SpatialConvolutionMM_updateGradInput(offset_view(x), non_contiguous(gy), w, 3, 3, 1, 1, 1, 1)
    assert close(gx, ref64.convmm_grad_input(H(gy), H(w), 10, 9, 1, 1, 1, 1), 1e-4)
    gw, gb = torch.zeros_like(w), torch.zeros_like(b)
    nnb.SpatialConvolutionMM_accGradParameters(x, gy, gw, gb, 3, 3, 1, 1, 1, 1, 2.0)
    rw, rb = ref64.convmm_acc_grad(H(x), H(gy), np.zeros(w.shape, np.float32), np.zeros(16, np.float32), 1, 1, 1, 1, 2.0)
    assert close(gw, rw, 1e-4) and close(gb, rb, 1e-4)
    # no bias, unbatched
    y3 = nnb.SpatialConvolutionMM_updateOutput(x[1], w, None, 3, 3, 2, 2, 0, 0)
    assert y3.dim() == 3 and close(y3, ref64.convmm_forward(H(x[1:2]), H(w), None, 2, 2, 0, 0)[0], 1e-4)


def test_batchnorm_entry_points(nnb, ref64):
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn((4, 5, 6, 7), device="cuda", generator=g) * 2 + 0.5
    w, b = torch.rand(5, device="cuda", generator=g), torch.rand(5, device="cuda", generator=g)
    rm, rv = torch.zeros(5, device="cuda"), torch.ones(5, device="cuda")
    ry, rm2, rv2, rsm, rss = ref64.bn_forward(H(x), H(w), H(b), H(rm), H(rv), True, 0.1, 1e-5)
    y, sm, ss = nnb.BatchNormalization_updateOutput(non_contiguous(x), w, b, rm, rv, True, 0.1, 1e-5)
    assert tuple(y.shape) == tuple(x.shape) and close(y, ry) and close(sm, rsm) and close(ss, rss) and close(rm, rm2) and close(rv, rv2)
    gy = torch.randn_like(x)
    gw, gb = torch.zeros(5, device="cuda"), torch.zeros(5, device="cuda")
    gx = nnb.BatchNormalization_backward(offset_view(x), gy, gw, gb, w, rm, rv, sm, ss, True, 1.0, 1e-5)
    z = np.zeros(5, np.float32)
    rgx, rgw, rgb = ref64.bn_backward(H(x), H(gy), H(w), rm2, rv2, rsm, rss, True, 1.0, 1e-5, gw=z, gb=z)
    assert close(gx, rgx, 1e-4) and close(gw, rgw, 1e-4) and close(gb, rgb, 1e-4)
    # inference mode, no affine, parameters only
    y, _, _ = nnb.BatchNormalization_updateOutput(x, None, None, rm, rv, False, 0.1, 1e-5)
    assert close(y, ref64.bn_forward(H(x), None, None, rm2, rv2, False, 0.1, 1e-5)[0])
    assert nnb.BatchNormalization_backward(x, gy, gw, None, None, rm, rv, sm, ss, True, 1.0, 1e-5, want_gx=False) is None


def test_batchnorm_is_the_first_call_on_a_fresh_state(ref64):
    # A new state has no scratch yet; batch norm over 40 000 channels needs more than the 1 MiB a first
    # allocation rounds up to, and must size its own buffer rather than another operator's.
    from cunn_b200 import thnn
    b = thnn.THNN()
    try:
        g = torch.Generator(device="cuda").manual_seed(31)
        N, C = 2, 40000
        assert thnn.lib.cunn_b200_batchnorm_workspace(N, C) > (1 << 20)
        x = torch.randn((N, C, 3, 3), device="cuda", generator=g)
        rm, rv = torch.zeros(C, device="cuda"), torch.ones(C, device="cuda")
        ry, rrm, rrv, rsm, rss = ref64.bn_forward(H(x), None, None, H(rm), H(rv), True, 0.1, 1e-5)
        y, sm, ss = b.BatchNormalization_updateOutput(x, None, None, rm, rv, True, 0.1, 1e-5)
        assert close(y, ry) and close(sm, rsm) and close(ss, rss)
        gy = torch.randn_like(x)
        gx = b.BatchNormalization_backward(x, gy, None, None, None, rm, rv, sm, ss, True, 1.0, 1e-5)
        assert close(gx, ref64.bn_backward(H(x), H(gy), None, rrm, rrv, rsm, rss, True, 1.0, 1e-5)[0], 1e-4)
    finally:
        b.close()


def test_maxpool_entry_points(nnb, ref64):
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn((2, 3, 16, 24), device="cuda", generator=g)
    for ceil_mode in (False, True):
        y, ind = nnb.SpatialMaxPooling_updateOutput(non_contiguous(x), 3, 3, 2, 2, 1, 1, ceil_mode)
        ry, rind = ref64.maxpool_forward(H(x), 3, 3, 2, 2, 1, 1, ceil_mode)
        assert np.array_equal(H(y), ry) and np.array_equal(H(ind), rind)
        gy = torch.randn_like(y)
        gx = nnb.SpatialMaxPooling_updateGradInput(offset_view(x), gy, ind, 3, 3, 2, 2, 1, 1, ceil_mode)
        assert close(gx, ref64.maxpool_backward(H(gy), rind, 16, 24, 3, 3, 2, 2, 1, 1), 1e-5)
    y3, ind3 = nnb.SpatialMaxPooling_updateOutput(x[0], 2, 2, 2, 2, 0, 0, False)
    assert y3.dim() == 3 and ind3.dim() == 4          # indices stay 4-D, as in the reference


def test_errors_reach_the_hook_with_the_reference_messages(nnb):
    from cunn_b200.thnn import THNNError
    x = torch.zeros((1, 4, 2, 2), device="cuda")
    with pytest.raises(THNNError, match="Output size is too small"):
        nnb.SpatialConvolutionMM_updateOutput(x, torch.zeros((8, 4, 5, 5), device="cuda"), None, 5, 5, 1, 1, 0, 0)
    with pytest.raises(THNNError, match="Need input of dimension 4 and input.size\\[1\\] == 3"):
        nnb.SpatialDepthWiseConvolution_updateOutput(x, torch.zeros((1, 3, 3, 3), device="cuda"), None, 3, 3, 1, 1, 1, 1)
    with pytest.raises(THNNError, match="pad should be smaller than half of kernel size"):
        nnb.SpatialMaxPooling_updateOutput(torch.zeros((1, 1, 8, 8), device="cuda"), 2, 2, 2, 2, 2, 2, False)
    with pytest.raises(THNNError, match="weight tensor has to be contiguous"):
        w = torch.zeros((8, 4, 3, 6), device="cuda")[..., ::2]
        nnb.SpatialConvolutionMM_updateOutput(x, w, None, 3, 3, 1, 1, 1, 1)
