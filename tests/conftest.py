import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests", "golden"), os.path.join(ROOT, "oracle")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


_GOLDEN = {}


def load_golden(family):
    """{case name: ({input name: array}, {output name: array})} of one fixture file."""
    if family not in _GOLDEN:
        path = os.path.join(ROOT, "tests", "golden", f"{family}.npz")
        data = np.load(path)
        cases = {}
        for key in data.files:
            name, kind, arr = key.split("/")
            ins, outs = cases.setdefault(name, ({}, {}))
            (ins if kind == "in" else outs)[arr] = data[key]
        _GOLDEN[family] = cases
    return _GOLDEN[family]


def ulp_diff(a, b):
    """Distance in units in the last place between two float32 arrays (same shape)."""
    a = np.ascontiguousarray(a, np.float32).view(np.int32).astype(np.int64)
    b = np.ascontiguousarray(b, np.float32).view(np.int32).astype(np.int64)
    a = np.where(a < 0, -(a & 0x7FFFFFFF), a)
    b = np.where(b < 0, -(b & 0x7FFFFFFF), b)
    return np.abs(a - b)


def assert_bit_exact(got, want, what=""):
    got, want = np.asarray(got, np.float32), np.asarray(want, np.float32)
    assert got.shape == want.shape, f"{what}: shape {got.shape} != {want.shape}"
    same = (got.view(np.int32) == want.view(np.int32)) | ((got == 0) & (want == 0)) | (np.isnan(got) & np.isnan(want))
    if not same.all():
        bad = np.argwhere(~same)[0]
        raise AssertionError(f"{what}: {int((~same).sum())} of {same.size} elements differ, first at {tuple(bad)}: "
                             f"{got[tuple(bad)]!r} vs {want[tuple(bad)]!r}")


def assert_contraction_close(got, want, k, what=""):
    """The tolerance stated for conv/matmul: rel 1e-4 per element OR 1e-3 max-abs after
    normalising by sqrt(K)."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} != {want.shape}"
    err = np.abs(got - want)
    rel_ok = err <= 1e-4 * np.abs(want)
    norm_ok = err / np.sqrt(max(k, 1)) <= 1e-3
    ok = rel_ok | norm_ok
    assert ok.all(), f"{what}: max abs err {err.max():.3e} (K={k}), {int((~ok).sum())} elements out of tolerance"


@pytest.fixture(scope="session")
def nn_gpu():
    """The product namespace on device 0 (GPU tests only)."""
    import litenn_b200 as nn
    devs = nn.devices.get_all()
    if not devs:
        pytest.fail("no CUDA device visible: GPU tests must run on the B200 box")
    nn.devices.set_current(devs[0])
    yield nn
