"""Host logic of the batch-sharded data-parallel step on CPU ranks (gloo, world size 2): the shard rule, the
gradient sum over replicas, identical updates on every rank, ragged and tiny batches.  The replica here is a
stand-in linear model on CPU tensors with the same interface as cunn_b200.mobilenet.MobileNetV1 (the real
replica needs a GPU); the DataParallelStep logic under test is the shipped one."""
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist
import torch.multiprocessing as mp


class LinearReplica:
    """y = x W^T, loss = sum((y - t)^2) / (2 * global_batch): same contract as the MobileNet replica —
    gradients of the locally summed, globally scaled loss are accumulated into a flat buffer."""

    def __init__(self, params):
        self.params = params.clone()
        self.grads = torch.zeros_like(self.params)
        self.loss = torch.zeros(1)

    def zero_grad(self):
        self.grads.zero_()

    def step(self, x, t, global_batch):
        W = self.params.view(3, 5)
        if x.shape[0] == 0:                      # a replica without rows takes no part (DataParallelTable.lua:531)
            self.loss.zero_()
            return self.loss
        r = x @ W.t() - t
        self.loss[0] = float((r * r).sum()) / (2 * global_batch)
        self.grads += ((r.t() @ x) / global_batch).reshape(-1)
        return self.loss

    def sgd(self, lr):
        self.params -= lr * self.grads


def _worker(rank, world, port, batches, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from cunn_b200.mobilenet import DataParallelStep, slice_range
    torch.manual_seed(0)
    params = torch.randn(15)
    step = DataParallelStep(LinearReplica(params), dist)
    results = []
    for n in batches:
        g = torch.Generator().manual_seed(100 + n)
        X, T = torch.randn((n, 5), generator=g), torch.randn((n, 3), generator=g)   # the full batch, same on all ranks
        s, c = step.shard(n)
        loss = step.train_step(X[s:s + c], T[s:s + c], n, 0.1)
        total = loss.clone()
        dist.all_reduce(total)
        results.append((float(total), step.replica.params.clone()))
    if rank == 0:
        torch.save(results, out)
    # every rank must hold identical parameters without any broadcast
    mine = step.replica.params.clone()
    other = mine.clone()
    dist.broadcast(other, src=0)
    assert torch.equal(mine, other)
    dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_rank_step_equals_single_replica(tmp_path):
    # batch sizes of the reference's DataParallelTable test: 2 * nGPU, 9, 15 (uneven), plus 1 (fewer rows
    # than replicas) — test_DataParallelTable.lua:126,263-293
    batches = [4, 9, 15, 1]
    out = str(tmp_path / "res.pt")
    mp.spawn(_worker, args=(2, _free_port(), batches, out), nprocs=2, join=True)
    got = torch.load(out)
    # single replica on the full batches
    from cunn_b200.mobilenet import DataParallelStep
    torch.manual_seed(0)
    single = DataParallelStep(LinearReplica(torch.randn(15)), None)
    for n, (loss2, params2) in zip(batches, got):
        g = torch.Generator().manual_seed(100 + n)
        X, T = torch.randn((n, 5), generator=g), torch.randn((n, 3), generator=g)
        loss1 = single.train_step(X, T, n, 0.1)
        assert float(loss1) == pytest.approx(loss2, rel=1e-6)
        assert torch.allclose(single.replica.params, params2, rtol=1e-6, atol=1e-7)


def test_slice_range_is_the_reference_rule():
    from cunn_b200.mobilenet import slice_range
    for n in (0, 1, 2, 7, 9, 15, 1024):
        for g in (1, 2, 3, 4, 8):
            pos = 0
            for i in range(g):
                s, c = slice_range(n, g, i)
                per, extra = divmod(n, g)
                assert (s, c) == (pos, per + 1 if i < extra else per)
                pos += c
            assert pos == n
