import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))  # the oracle is test infrastructure
GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


class GraphArrays:
    """graphs.npz and graphs_tp.npz (inputs and reference results of the small memgraph fixtures) as one
    read-only mapping with the `.files` of an npz."""

    def __init__(self):
        self._d = {}
        for name in ("graphs.npz", "graphs_tp.npz"):
            a = np.load(os.path.join(GOLDEN_DIR, "graphs", name))
            for k in a.files:
                self._d[k] = a[k]
        self.files = list(self._d)

    def __getitem__(self, k):
        return self._d[k]


class Golden:
    def __init__(self):
        with open(os.path.join(GOLDEN_DIR, "golden.json")) as f:
            self.meta = json.load(f)
        self.arrays = np.load(os.path.join(GOLDEN_DIR, "golden.npz"))

    def es_inputs(self, case):
        return [self.arrays["es/%s/in%d" % (case["name"], k)] for k in range(len(case["inns"]))]

    def es_output(self, case):
        return self.arrays["es/%s/out" % case["name"]]


_golden = None


def golden():
    global _golden
    if _golden is None:
        _golden = Golden()
    return _golden


@pytest.fixture(scope="session", name="golden")
def golden_fixture():
    return golden()


def ulp_distance(a, b):
    """Distance in units in the last place between two same-dtype float arrays."""
    a, b = np.asarray(a), np.asarray(b)
    assert a.dtype == b.dtype
    if a.dtype == np.complex64:
        return max(ulp_distance(a.real.copy(), b.real.copy()), ulp_distance(a.imag.copy(), b.imag.copy()))
    it = {2: np.int16, 4: np.int32, 8: np.int64}[a.dtype.itemsize]
    ai, bi = a.view(it).astype(np.int64), b.view(it).astype(np.int64)
    sign = np.int64(1) << (8 * a.dtype.itemsize - 1)
    ai = np.where(ai < 0, -(ai + sign), ai)  # sign-magnitude -> monotone integers
    bi = np.where(bi < 0, -(bi + sign), bi)
    both_nan = np.isnan(a) & np.isnan(b)
    d = np.abs(ai - bi)
    d[both_nan] = 0
    return int(d.max()) if d.size else 0
