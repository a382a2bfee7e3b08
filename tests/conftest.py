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
def refd():
    """The oracle built for fp64 tensors (the CudaDouble entry points)."""
    from oracle.thnn_ref import Ref
    return Ref("refd_")


@pytest.fixture(scope="session")
def ref32():
    from oracle.thnn_ref import Ref
    return Ref("ref32_")


_CHUNK = 1 << 24


def _flat_pair(got, want):
    got, want = np.asarray(got), np.asarray(want)
    assert got.shape == want.shape, (got.shape, want.shape)
    return got.reshape(-1), want.reshape(-1)


def _absmax(a):
    m = 0.0
    for i in range(0, a.size, _CHUNK):
        c = a[i:i + _CHUNK]
        if c.size:
            m = max(m, float(np.max(np.abs(c))))
    return m


def rel_err(got, want, floor_frac=1e-2):
    """Element-wise relative error  max_i |got_i - want_i| / max(|want_i|, floor)  with
    floor = floor_frac * max_j |want_j|.  The floor keeps outputs that are small only
    because large terms cancelled (where no fp32 summation order can hold a relative
    bound) from dominating; everywhere else this is the plain relative error.
    assert_parity() below evaluates the same quantity with the stricter 1e-3 floor.
    Differences are taken in fp64, a block at a time so that large tensors need no fp64 copy."""
    got, want = _flat_pair(got, want)
    if want.size == 0:
        return 0.0
    floor = floor_frac * max(_absmax(want), 1e-30)
    worst = 0.0
    for i in range(0, want.size, _CHUNK):
        g = got[i:i + _CHUNK].astype(np.float64)
        w = want[i:i + _CHUNK].astype(np.float64)
        e = np.abs(g - w) / np.maximum(np.abs(w), floor)
        if np.isnan(e).any():
            return float("nan")
        worst = max(worst, float(np.max(e)))
    return worst


def norm_err(got, want):
    """Tensor-normalised error  max_i |got_i - want_i| / max_j |want_j|."""
    got, want = _flat_pair(got, want)
    if want.size == 0:
        return 0.0
    worst = 0.0
    for i in range(0, want.size, _CHUNK):
        e = np.abs(got[i:i + _CHUNK].astype(np.float64) - want[i:i + _CHUNK].astype(np.float64))
        if np.isnan(e).any():
            return float("nan")
        worst = max(worst, float(np.max(e)))
    return worst / max(_absmax(want), 1e-30)


# ---------------------------------------------------------------------------------------------
# Parity bookkeeping: every assert_parity() call records both error figures; the table is printed
# at the end of the run and written as JSON to the file the CUNN_PARITY_REPORT variable names, if set.
_PARITY = []


def assert_parity(name, got, want, tol, port=None):
    """Checks one tensor of the CUDA path against the fp64 oracle and records the figures.

    Two numbers are computed: the tensor-normalised error  max|got-want| / max|want|  and the
    element-wise relative error with a floor of 1e-3 * max|want|.  The first must be <= tol.  The
    second must be <= tol as well, unless fp32 arithmetic itself cannot reach it on this tensor:
    `port` (the same routine of the fp32 CPU port of the oracle, an array or a callable returning
    one, evaluated only when needed) shows what plain fp32 achieves, and the CUDA result may then
    be at most 1.5x as far from the oracle as the port is.
    """
    n, r = norm_err(got, want), rel_err(got, want, 1e-3)
    rec = {"name": name, "tol": tol, "norm_err": n, "rel_err_floor_1e-3": r, "fp32_port_rel_err_floor_1e-3": None}
    _PARITY.append(rec)
    assert n <= tol, "%s: tensor-normalised error %.3g > %.3g" % (name, n, tol)
    if r <= tol:
        return rec
    assert port is not None, "%s: element-wise error (floor 1e-3) %.3g > %.3g" % (name, r, tol)
    p = rel_err(port() if callable(port) else port, want, 1e-3)
    rec["fp32_port_rel_err_floor_1e-3"] = p
    assert r <= 1.5 * p, "%s: element-wise error (floor 1e-3) %.3g > %.3g and > 1.5 x the fp32 port's %.3g" % (name, r, tol, p)
    return rec


def pytest_terminal_summary(terminalreporter):
    if not _PARITY:
        return
    tr = terminalreporter
    tr.write_sep("-", "parity against the fp64 oracle (tensor-normalised | element-wise, floor 1e-3 | fp32 CPU port)")
    for rec in _PARITY:
        p = rec["fp32_port_rel_err_floor_1e-3"]
        tr.write_line("%-58s tol %.0e  %.2e  %.2e  %s" % (rec["name"][:58], rec["tol"], rec["norm_err"],
                                                         rec["rel_err_floor_1e-3"], "-" if p is None else "%.2e" % p))
    out = os.environ.get("CUNN_PARITY_REPORT")
    if out:
        import json
        with open(out, "w") as f:
            json.dump(_PARITY, f, indent=1)
