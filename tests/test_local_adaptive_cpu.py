"""Oracle routines of SpatialConvolutionLocal and the adaptive poolings against independent formulations built from
PyTorch's CPU operators (unfold + einsum; adaptive_*_pool2d).  No GPU needed."""
import numpy as np
import pytest

from conftest import rel_err

torch = pytest.importorskip("torch")
F = torch.nn.functional


@pytest.mark.parametrize("shape", [(2, 3, 8, 9, 4, 3, 3, 1, 1, 1, 1), (3, 2, 10, 7, 5, 3, 2, 2, 1, 1, 0), (1, 4, 6, 6, 2, 1, 1, 1, 1, 0, 0)])
def test_local_convolution_oracle_against_unfold_einsum(ref64, shape):
    N, C, H, W, K, kH, kW, dH, dW, padH, padW = shape
    rng = np.random.default_rng(1)
    oH, oW = (H + 2 * padH - kH) // dH + 1, (W + 2 * padW - kW) // dW + 1
    P, R = oH * oW, C * kH * kW
    x = rng.standard_normal((N, C, H, W)).astype(np.float32)
    w = rng.standard_normal((P, K, R)).astype(np.float32)
    b = rng.standard_normal((K, oH, oW)).astype(np.float32)
    xt = torch.from_numpy(x).double().requires_grad_(True)
    wt = torch.from_numpy(w).double().requires_grad_(True)
    bt = torch.from_numpy(b).double().requires_grad_(True)
    col = F.unfold(xt, (kH, kW), padding=(padH, padW), stride=(dH, dW))              # [N, R, P]
    y = torch.einsum("pkr,nrp->nkp", wt, col).view(N, K, oH, oW) + bt
    gy = rng.standard_normal((N, K, oH, oW)).astype(np.float32)
    y.backward(torch.from_numpy(gy).double())
    assert rel_err(ref64.localconv_forward(x, w, b, kH, kW, dH, dW, padH, padW), y.detach().numpy()) < 1e-6
    assert rel_err(ref64.localconv_grad_input(gy, w, C, H, W, kH, kW, dH, dW, padH, padW), xt.grad.numpy()) < 1e-6
    gw0, gb0 = rng.standard_normal(w.shape).astype(np.float32), rng.standard_normal(b.shape).astype(np.float32)
    gw, gb = ref64.localconv_acc_grad(x, gy, gw0, gb0, kH, kW, dH, dW, padH, padW, 0.5)
    assert rel_err(gw, gw0 + 0.5 * wt.grad.numpy()) < 1e-6
    assert rel_err(gb, gb0 + 0.5 * bt.grad.numpy()) < 1e-6


@pytest.mark.parametrize("shape", [(2, 3, 7, 7, 3, 3), (1, 4, 10, 13, 4, 5), (2, 2, 14, 14, 1, 1), (1, 2, 9, 6, 5, 4)])
def test_adaptive_pooling_oracle_against_pytorch(ref64, shape):
    N, C, H, W, oH, oW = shape
    rng = np.random.default_rng(2)
    x = rng.standard_normal((N, C, H, W)).astype(np.float32)
    xt = torch.from_numpy(x).double().requires_grad_(True)
    yt, it = F.adaptive_max_pool2d(xt, (oH, oW), return_indices=True)
    y, ind = ref64.adaptive_maxpool_forward(x, oH, oW)
    assert np.array_equal(y, yt.detach().numpy().astype(np.float32))
    # PyTorch stores the flat position in the plane; here: row / column inside the window + base
    for yy in range(oH):
        for xx in range(oW):
            y0 = int(np.floor(np.float32(yy) / np.float32(oH) * np.float32(H)))
            x0 = int(np.floor(np.float32(xx) / np.float32(oW) * np.float32(W)))
            flat = (y0 + ind[0, :, :, yy, xx] - ref64.index_base) * W + x0 + ind[1, :, :, yy, xx] - ref64.index_base
            assert np.array_equal(flat, it[:, :, yy, xx].numpy())
    gy = rng.standard_normal(y.shape).astype(np.float32)
    yt.backward(torch.from_numpy(gy).double())
    assert rel_err(ref64.adaptive_maxpool_backward(gy, ind, H, W), xt.grad.numpy()) < 1e-6
    xt.grad = None
    ya = F.adaptive_avg_pool2d(xt, (oH, oW))
    assert rel_err(ref64.adaptive_avgpool_forward(x, oH, oW), ya.detach().numpy()) < 1e-6
    ya.backward(torch.from_numpy(gy).double())
    assert rel_err(ref64.adaptive_avgpool_backward(gy, H, W), xt.grad.numpy()) < 1e-6
