"""DataParallelTable around a module made of the library's kernels, one replica on one GPU: forward and backward
go through the depthwise entry points, gradients accumulate in the visible buffer over two backward calls and
the update is p -= lr * g."""
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


class DepthwiseLayer:
    """SpatialDepthWiseConvolution 3x3 pad 1 with flat parameters [weight (C*9) | bias (C)]."""

    def __init__(self, F, C, stride, dev):
        g = torch.Generator(device=dev).manual_seed(11)
        self.F, self.C, self.s = F, C, stride
        self.params = (torch.rand(C * 10, device=dev, generator=g) * 2 - 1) / 3
        self.grads = torch.zeros_like(self.params)

    def _w(self, t):
        return t[:self.C * 9].view(1, self.C, 3, 3), t[self.C * 9:].view(1, self.C)

    def forward(self, x):
        w, b = self._w(self.params)
        return self.F.dwconv_forward(x, w, b, self.s, self.s, 1, 1)

    def backward(self, x, gy, scale=1.0):
        w, _ = self._w(self.params)
        gw, gb = self._w(self.grads)
        self.F.dwconv_acc_grad(x, gy, gw, gb, self.s, self.s, 1, 1, scale)
        return self.F.dwconv_grad_input(gy, w, x.shape[2], x.shape[3], self.s, self.s, 1, 1)


def test_table_over_depthwise_layer():
    import cunn_b200.functional as F
    from cunn_b200 import device_status
    from cunn_b200.data_parallel import DataParallelTable
    dev = torch.device("cuda")
    layer = DepthwiseLayer(F, 16, 2, dev)
    dpt = DataParallelTable().add(layer)
    g = torch.Generator(device=dev).manual_seed(3)
    x = torch.randn((6, 16, 14, 14), device=dev, generator=g)
    y = dpt.forward(x)
    gy = torch.randn(y.shape, device=dev, generator=g)
    gx = dpt.backward(x, gy, 0.5)
    dpt.backward(x, gy, 0.5)
    params, grads = dpt.getParameters()
    ref = DepthwiseLayer(F, 16, 2, dev)
    assert torch.equal(y, ref.forward(x)) and torch.equal(gx, ref.backward(x, gy, 1.0))
    # two half-scaled backward calls add up to the full gradient (fp32 atomics: compare with a tolerance)
    assert torch.allclose(grads, ref.grads, rtol=1e-4, atol=1e-5)
    assert torch.count_nonzero(layer.grads) == 0
    before = params.clone()
    dpt.updateParameters(0.1)
    assert torch.allclose(params, before - 0.1 * grads, rtol=2e-7, atol=1e-7)
    dpt.zeroGradParameters()
    assert torch.count_nonzero(grads) == 0 and device_status() == 0
