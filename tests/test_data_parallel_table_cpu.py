"""nn.DataParallelTable semantics on CPU ranks (gloo, world size 2), following the reference's own tests
(test_DataParallelTable.lua): outputs and input gradients equal the single-device module (:637-690),
an identity Linear returns its input on ragged and tiny batches (:692-741), Linear(10, 5) flattens to 55
parameters (:440-465), gradients accumulate over three micro-batches between zeroGradParameters (:531-576),
parameters stay identical on every replica, and syncParameters spreads replica 1's parameters.  The module is a
CPU Linear with the replica protocol; the DataParallelTable under test is the shipped class."""
import os
import socket

import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist
import torch.multiprocessing as mp


class Linear:
    """y = x W^T + b with flat parameters [W (out x in) | b (out)] and a flat local gradient buffer."""

    def __init__(self, nin, nout, seed=0):
        g = torch.Generator().manual_seed(seed)
        self.nin, self.nout = nin, nout
        self.params = torch.randn(nout * nin + nout, generator=g, dtype=torch.float64)
        self.grads = torch.zeros_like(self.params)

    def _wb(self, t):
        return t[:self.nout * self.nin].view(self.nout, self.nin), t[self.nout * self.nin:]

    def output_shape(self, in_tail):
        return (self.nout,)

    def forward(self, x):
        W, b = self._wb(self.params)
        return x @ W.t() + b

    def backward(self, x, gy, scale=1.0):
        W, _ = self._wb(self.params)
        gW, gb = self._wb(self.grads)
        gW += scale * (gy.t() @ x)
        gb += scale * gy.sum(0)
        return gy @ W


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _batch(n, nin, nout, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn((n, nin), generator=g, dtype=torch.float64),
            torch.randn((n, nout), generator=g, dtype=torch.float64))


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from cunn_b200.data_parallel import DataParallelTable
    res = {}

    # (1) forward / backward equal the single module; parameters differ per rank before the first sync
    dpt = DataParallelTable(1, True, True, dist=dist).add(Linear(10, 5, seed=rank), gpus=list(range(world)))
    assert dpt.size() == world and dpt.get(rank + 1) is dpt.module
    params, gparams = dpt.getParameters()
    res["nparams"] = params.numel()
    fwd = []
    for n in (4, 9, 15, 1):                       # 2 * nGPU, uneven, fewer rows than replicas
        x, gy = _batch(n, 10, 5, 100 + n)
        dpt.zeroGradParameters()
        y = dpt.forward(x)
        assert y.shape[0] == dpt.shard(n)[1]
        yall = dpt.gatherOutput(n)
        gx = dpt.backward(x, gy)
        dpt.output = gx                            # reuse the gather for the input gradient
        gxall = dpt.gatherOutput(n)
        fwd.append((n, yall.clone(), gxall.clone(), gparams.clone()))
    res["fwd"] = fwd

    # (2) gradient accumulation over three micro-batches, then one update
    dpt.zeroGradParameters()
    for k in range(3):
        x, gy = _batch(7, 10, 5, 200 + k)
        dpt.forward(x)
        dpt.backward(x, gy, 0.5)
    res["acc"] = gparams.clone()
    dpt.updateParameters(0.1)
    res["updated"] = params.clone()
    other = params.clone()
    dist.broadcast(other, src=0)
    assert torch.equal(other, params)              # identical without any broadcast after the update

    # (3) identity Linear on ragged / tiny batches returns its input exactly
    ident = Linear(6, 6)
    ident.params.zero_()
    ident.params[:36] = torch.eye(6, dtype=torch.float64).reshape(-1)
    dpi = DataParallelTable(dist=dist).add(ident)
    for n in (1, 2, 3, 5):
        x, _ = _batch(n, 6, 6, 300 + n)
        dpi.forward(x)
        assert torch.equal(dpi.gatherOutput(n), x)

    # (4) syncParameters: a change made on replica 1 only reaches every replica at the next forward
    if rank == 0:
        params.add_(1.0)
    dpt.needsSync = True
    x, _ = _batch(4, 10, 5, 400)
    dpt.forward(x)
    other = params.clone()
    dist.broadcast(other, src=0)
    assert torch.equal(other, params)

    if rank == 0:
        torch.save(res, out)
    dist.destroy_process_group()


def test_data_parallel_table_matches_single_module(tmp_path):
    out = str(tmp_path / "dpt.pt")
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    res = torch.load(out)
    assert res["nparams"] == 55                    # Linear(10, 5): 50 weights + 5 biases
    ref = Linear(10, 5, seed=0)                    # replica 1's parameters are the ones every rank used
    for n, yall, gxall, gsum in res["fwd"]:
        x, gy = _batch(n, 10, 5, 100 + n)
        ref.grads.zero_()
        # rows are independent; the CPU GEMM blocks differently for shards and for the full batch, hence 1e-13
        assert torch.allclose(yall, ref.forward(x), rtol=1e-13, atol=1e-13)
        assert torch.allclose(gxall, ref.backward(x, gy), rtol=1e-13, atol=1e-13)
        assert torch.allclose(gsum, ref.grads, rtol=1e-12, atol=1e-12)
    ref.grads.zero_()
    for k in range(3):
        x, gy = _batch(7, 10, 5, 200 + k)
        ref.backward(x, gy, 0.5)
    assert torch.allclose(res["acc"], ref.grads, rtol=1e-12, atol=1e-12)
    assert torch.allclose(res["updated"], ref.params - 0.1 * ref.grads, rtol=1e-12, atol=1e-12)


def test_single_process_table_is_the_module():
    from cunn_b200.data_parallel import DataParallelTable, sliceRange
    m = Linear(4, 3, seed=5)
    dpt = DataParallelTable().add(m)
    x, gy = _batch(6, 4, 3, 1)
    assert torch.equal(dpt.forward(x), m.forward(x))
    dpt.backward(x, gy)
    dpt.backward(x, gy)
    p, g = dpt.getParameters()
    ref = Linear(4, 3, seed=5)
    ref.backward(x, gy)
    ref.backward(x, gy)
    assert torch.allclose(g, ref.grads) and torch.count_nonzero(m.grads) == 0
    dpt.zeroGradParameters()
    assert torch.count_nonzero(g) == 0
    # the reference's rule, 1-based replica index: 7 rows over 3 replicas -> 3, 2, 2
    assert [sliceRange(7, i, 3) for i in (1, 2, 3)] == [(0, 3), (3, 2), (5, 2)]
    with pytest.raises(ValueError):
        DataParallelTable(dimension=2)
    with pytest.raises(RuntimeError):
        dpt.add(m)
