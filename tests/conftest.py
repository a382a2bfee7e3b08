import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def golden(name):
    return dict(np.load(os.path.join(GOLDEN, name + ".npz")))


@pytest.fixture(scope="session")
def ref64():
    from oracle.thnn_ref import Ref
    return Ref("ref64_")


@pytest.fixture(scope="session")
def ref32():
    from oracle.thnn_ref import Ref
    return Ref("ref32_")


def rel_err(got, want, floor_frac=1e-2):
    """Element-wise relative error  max_i |got_i - want_i| / max(|want_i|, floor)  with
    floor = floor_frac * max_j |want_j|.  The floor keeps outputs that are small only
    because large terms cancelled (where no fp32 summation order can hold a relative
    bound) from dominating; everywhere else this is the plain relative error."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    if want.size == 0:
        return 0.0
    floor = floor_frac * max(float(np.max(np.abs(want))), 1e-30)
    return float(np.max(np.abs(got - want) / np.maximum(np.abs(want), floor)))


def norm_err(got, want):
    """Tensor-normalised error  max_i |got_i - want_i| / max_j |want_j|."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    if want.size == 0:
        return 0.0
    return float(np.max(np.abs(got - want)) / max(float(np.max(np.abs(want))), 1e-30))
