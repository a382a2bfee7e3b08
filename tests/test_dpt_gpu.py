"""The native DataParallelTable on GPUs.  One GPU: buffers, gradient folding and accumulation over several
backward passes (test_DataParallelTable.lua:531-576), update, serialisation.  Two GPUs (skipped on a one-GPU box):
replicas in one process with worker threads and a real NCCL all-reduce, ragged scatter / gather
(test_DataParallelTable.lua:692-741), parameter broadcast, one replica per process, and the reduced MobileNetV1
replica on two GPUs against the CPU oracle run shard by shard with the same shard rule."""
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def ngpus():
    return torch.cuda.device_count()


@pytest.fixture(scope="module")
def dpt():
    from cunn_b200 import dpt
    from cunn_b200._lib import lib, check
    check(lib.cunn_b200_dpt_nccl_load(b"libnccl.so.2"))     # the real library, whatever an earlier test loaded
    return dpt


def attach(t, i, n, dev):
    """Gives replica i torch-owned buffers so that the test can read and write them."""
    bufs = [torch.zeros(n, device=dev) for _ in range(3)]
    t.set_buffers(i, *[b.data_ptr() for b in bufs])
    return bufs


def sync_all():
    for d in range(ngpus()):
        torch.cuda.synchronize(d)


def test_single_replica_accumulates_updates_and_serialises(dpt, tmp_path):
    n = 1003
    t = dpt.NativeDataParallelTable().add(n, [0])
    try:
        params, local, visible = attach(t, 0, n, "cuda:0")
        assert t.size() == 1 and t.local_replicas() == 1 and t.param_count() == n
        for k in (1.0, 2.0, 3.0):                      # three micro-batches between zeroGradParameters
            sync_all()
            local.fill_(k)
            sync_all()
            t.reduce()
            sync_all()
            assert float(local.abs().max()) == 0.0
        assert torch.all(visible == 6.0)
        t.updateParameters(0.5)
        sync_all()
        assert torch.all(params == -3.0)
        path = str(tmp_path / "t.dpt")
        t.write(path, b"running-stats")
        t.zeroGradParameters()
        sync_all()
        assert float(visible.abs().max()) == 0.0
        params.fill_(7.0)
        sync_all()
        assert t.read(path, 13) == b"running-stats"
        sync_all()
        assert torch.all(params == -3.0)
        gpus, p, extra = dpt.file_read(path)
        assert gpus == [0] and np.all(p == -3.0) and extra == b"running-stats"
    finally:
        t.close()


@pytest.mark.skipif(ngpus() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("threads", [False, True])
def test_two_replicas_in_one_process(dpt, threads):
    n = 70001
    t = dpt.NativeDataParallelTable().add(n, [0, 1])
    try:
        if threads:
            t.threads()
        bufs = [attach(t, i, n, "cuda:%d" % i) for i in range(2)]
        t.setBuckets([n, n // 3])                      # two buckets: [n/3, n) becomes ready first, then [0, n/3)
        seen = []

        def backward(i, dev, stream):
            # what a module's accGradParameters does: write the local gradient on the replica's stream, then tell the
            # table which bucket is complete
            seen.append((i, dev))
            with torch.cuda.device(dev), torch.cuda.stream(torch.cuda.ExternalStream(stream, device="cuda:%d" % dev)):
                bufs[i][1][n // 3:] = float(i + 1)
                t.bucketReady(i, 0)
                bufs[i][1][:n // 3] = 10.0 * (i + 1)
            return 0

        for _ in range(2):
            t.exec(backward)
            t.reduce()
            t.watchdog(30.0)
        sync_all()
        assert sorted(seen) == [(0, 0), (0, 0), (1, 1), (1, 1)]
        for i in range(2):
            vis = bufs[i][2]
            assert torch.all(vis[n // 3:] == 6.0) and torch.all(vis[:n // 3] == 60.0)     # (1 + 2) and (10 + 20), twice
            assert float(bufs[i][1].abs().max()) == 0.0
        # parameters: replica 1 diverged; syncParameters brings back replica 0's
        bufs[0][0].fill_(1.5)
        bufs[1][0].fill_(-4.0)
        sync_all()
        t.syncParameters()
        t.updateParameters(0.25)
        sync_all()
        for i in range(2):
            assert torch.all(bufs[i][0][n // 3:] == 0.0) and torch.all(bufs[i][0][:n // 3] == -13.5)
        # ragged scatter / gather of a 5-row batch from and to host memory: rows 3 + 2
        src = torch.arange(5 * 7, dtype=torch.float32).view(5, 7).pin_memory()
        dst = [torch.zeros((3, 7), device="cuda:%d" % i) for i in range(2)]
        assert t.scatter(src.data_ptr(), 5, 28, [d.data_ptr() for d in dst]) == [3, 2]
        back = torch.zeros((5, 7)).pin_memory()
        t.gather([d.data_ptr() for d in dst], 5, 28, back.data_ptr())
        for i in range(2):
            torch.cuda.current_stream(i).synchronize()
        sync_all()
        # the table's own streams did the copies
        assert torch.equal(back, src) and torch.equal(dst[1][:2].cpu(), src[3:])
    finally:
        t.close()


RANK_SCRIPT = textwrap.dedent("""
    import os, sys, time
    sys.path.insert(0, %(root)r)
    import torch
    from cunn_b200 import dpt
    rank, world, path = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
    torch.cuda.set_device(rank)
    if rank == 0:
        uid = dpt.unique_id()
        open(path + ".tmp", "wb").write(uid)
        os.rename(path + ".tmp", path)
    else:
        for _ in range(600):
            if os.path.exists(path):
                break
            time.sleep(0.05)
        uid = open(path, "rb").read()
    n = 4099
    t = dpt.NativeDataParallelTable().add_rank(n, rank, rank, world, uid)
    bufs = [torch.zeros(n, device="cuda") for _ in range(3)]
    t.set_buffers(0, *[b.data_ptr() for b in bufs])
    t.set_stream(0, torch.cuda.current_stream().cuda_stream)
    bufs[1].fill_(rank + 1.0)
    bufs[0].fill_(float(rank))
    t.reduce()
    t.syncParameters()
    t.watchdog(30.0)
    torch.cuda.synchronize()
    assert torch.all(bufs[2] == world * (world + 1) / 2), bufs[2][:4]
    assert torch.all(bufs[0] == 0.0)
    t.close()
    print("rank", rank, "ok")
""")


@pytest.mark.skipif(ngpus() < 2, reason="needs two GPUs")
def test_one_replica_per_process(tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(RANK_SCRIPT % {"root": ROOT})
    uid = str(tmp_path / "uid")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, str(script), str(r), "2", uid], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                              env=env) for r in range(2)]
    outs = [p.communicate(timeout=180)[0].decode() for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and "rank %d ok" % r in o, o[-2000:]


@pytest.mark.skipif(ngpus() < 2, reason="needs two GPUs")
def test_mobilenet_on_two_replicas_matches_the_sharded_oracle(dpt, ref64):
    # The parity rule for g > 1: the oracle runs the same shards (BN statistics per shard, as in the reference) and the
    # gradients are summed; the table's visible gradient must equal that sum on every replica.
    from cunn_b200 import mobilenet as mb
    from test_mobilenet_gpu import oracle_step
    cfg = mb.Config(64, 8, 10)
    lay = mb.layout(cfg)
    params = mb.init_params(cfg, seed=11)
    rng = np.random.default_rng(5)
    GB = 7                                                         # shards of 4 and 3 rows
    images = rng.standard_normal((GB, 3, 64, 64)).astype(np.float32)
    labels = rng.integers(1, 11, GB).astype(np.int64)
    reps = [mb.MobileNetV1(cfg, torch.device("cuda", i), params, max_batch=4) for i in range(2)]
    n = reps[0].nparams
    t = dpt.NativeDataParallelTable().add(n, [0, 1])
    try:
        vis = []
        for i, r in enumerate(reps):
            v = torch.zeros(n, device="cuda:%d" % i)
            vis.append(v)
            t.set_buffers(i, r.params.data_ptr(), r.grads.data_ptr(), v.data_ptr())
            t.set_stream(i, torch.cuda.current_stream(i).cuda_stream)
        want = np.zeros(n, np.float64)
        loss_want = 0.0
        for i, r in enumerate(reps):
            s, c = dpt.slice_range(GB, 2, i)
            with torch.cuda.device(i):
                r.zero_grad()
                r.step(torch.from_numpy(images[s:s + c]).cuda(), torch.from_numpy(labels[s:s + c]).cuda(), GB)
            l, g, _ = oracle_step(ref64, lay, params, images[s:s + c], labels[s:s + c], 1.0 / GB)
            want += g
            loss_want += l
        t.reduce()
        sync_all()
        loss = sum(float(r.loss) for r in reps)
        assert loss == pytest.approx(loss_want, rel=1e-4)
        assert torch.equal(vis[0].cpu(), vis[1].cpu())                 # every replica holds the same sum
        got = vis[0].cpu().numpy()
        fc = lay[-1]
        sl = slice(fc["w_off"], fc["w_off"] + fc["wcount"])
        assert np.max(np.abs(got[sl] - want[sl])) < 1e-3 * np.max(np.abs(want[sl]))      # classifier: no chaotic amplification
        errs = [np.max(np.abs(got[L["w_off"]:L["w_off"] + L["wcount"]] - want[L["w_off"]:L["w_off"] + L["wcount"]])) /
                max(np.max(np.abs(want[L["w_off"]:L["w_off"] + L["wcount"]])), 1e-12) for L in lay]
        assert float(np.median(errs)) < 1e-2
    finally:
        t.close()
