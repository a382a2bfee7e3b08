"""Host side of the native DataParallelTable (include/cunn_b200_dpt.h), no GPU: the shard rule, the on-disk
format with the reference's deserializeNGPUs behaviour, and the communicator watchdog against a stand-in NCCL
whose asynchronous error state the test controls (failures are injected on the host only)."""
import ctypes
import os
import subprocess

import numpy as np
import pytest

from cunn_b200 import dpt
from cunn_b200._lib import CunnError

HERE = os.path.dirname(os.path.abspath(__file__))


def test_slice_range_is_the_reference_rule():
    # DataParallelTable.lua:469-479: the first n mod g replicas get one extra row; 0-based starts here
    for n in (0, 1, 2, 8, 9, 15, 1024):
        for g in (1, 2, 3, 4, 8):
            per, extra = divmod(n, g)
            pos = 0
            for i in range(g):
                s, c = dpt.slice_range(n, g, i)
                assert (s, c) == (pos, per + (1 if i < extra else 0))
                pos += c
            assert pos == n
    # a batch smaller than the GPU count leaves the last replicas without rows (:531)
    assert [dpt.slice_range(2, 4, i)[1] for i in range(4)] == [1, 1, 0, 0]


def test_slice_range_matches_the_oracle(ref64):
    for n, g in ((9, 4), (15, 8), (7, 7), (3, 5)):
        for i in range(g):
            assert dpt.slice_range(n, g, i) == ref64.slice_range(n, g, i)


def test_file_round_trip_and_gpu_reassignment(tmp_path):
    path = str(tmp_path / "table.dpt")
    params = np.random.default_rng(0).standard_normal(1000).astype(np.float32)
    extra = np.arange(12, dtype=np.float32).tobytes()
    dpt.file_write(path, [3, 1, 2, 0], params, extra)
    gpus, p, e = dpt.file_read(path)
    assert gpus == [3, 1, 2, 0] and np.array_equal(p, params) and e == extra
    # deserializeNGPUs = 2 (DataParallelTable.lua:373-381): replicas re-assigned to GPUs 0, 1
    gpus, p, _ = dpt.file_read(path, ngpus_wanted=2, gpus_available=2)
    assert gpus == [0, 1] and np.array_equal(p, params)
    # stored assignment kept, but this machine has only 2 GPUs (:383-393)
    with pytest.raises(CunnError, match="only 2 GPUs are available"):
        dpt.file_read(path, gpus_available=2)
    with pytest.raises(CunnError, match="Asked for 8 GPUs but only 2"):
        dpt.file_read(path, ngpus_wanted=8, gpus_available=2)
    with open(path, "r+b") as f:
        f.truncate(200)
    with pytest.raises(CunnError, match="truncated"):
        dpt.file_read(path)
    bad = str(tmp_path / "other.bin")
    open(bad, "wb").write(b"not a table at all")
    with pytest.raises(CunnError, match="not a DataParallelTable file"):
        dpt.file_read(bad)


@pytest.fixture
def fake_nccl(tmp_path):
    so = str(tmp_path / "libfakenccl.so")
    subprocess.check_call(["gcc", "-shared", "-fPIC", "-O1", "-o", so, os.path.join(HERE, "fake_nccl.c")])
    from cunn_b200._lib import lib, check
    check(lib.cunn_b200_dpt_nccl_load(so.encode()))
    fake = ctypes.CDLL(so)
    fake.fake_nccl_reset()
    yield fake
    fake.fake_nccl_reset()


def test_watchdog_aborts_on_an_asynchronous_error(fake_nccl):
    t = dpt.NativeDataParallelTable()
    try:
        t.adopt_comms([0x10, 0x11])
        t.watchdog(0.05)                                   # healthy communicators, nothing in flight
        fake_nccl.fake_nccl_set_async(2)                   # ncclSystemError
        with pytest.raises(CunnError, match="asynchronous error.*unhandled system error.*aborted"):
            t.watchdog(1.0)
        assert fake_nccl.fake_nccl_aborts() == 2           # both communicators were aborted
        with pytest.raises(CunnError, match="were aborted"):
            t.watchdog(1.0)                                # the table stays failed
    finally:
        t.close()


def test_watchdog_times_out_on_a_collective_that_never_finishes(fake_nccl):
    t = dpt.NativeDataParallelTable()
    try:
        t.adopt_comms([0x10])
        fake_nccl.fake_nccl_set_async(7)                   # ncclInProgress for ever: a peer that never joined
        with pytest.raises(CunnError, match="did not finish within 0.050 s"):
            t.watchdog(0.05)
        assert fake_nccl.fake_nccl_aborts() == 1
    finally:
        t.close()


def test_unique_id_comes_from_the_loaded_nccl(fake_nccl):
    assert dpt.unique_id() == bytes(range(128))
