import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU; run with `-m gpu`")


@pytest.fixture
def rng():
    return np.random.default_rng(20251125)


def bits(a):
    """Bit pattern view for bit-exact float comparisons (distinguishes -0/+0 and NaN payloads)."""
    a = np.ascontiguousarray(a)
    return a.view({4: np.uint32, 1: np.uint8, 2: np.uint16, 8: np.uint64}[a.dtype.itemsize])


def _canonical_nan(a):
    """NaN payloads are the one thing that legitimately differs between processors: x86 SSE returns the
    first NaN operand quieted, the GPU returns the canonical NaN 0x7fffffff. Both are "NaN"; every
    other bit pattern (including the sign of zero and infinities) must match exactly."""
    a = np.array(a, copy=True)
    if a.dtype.kind == "f":
        a[np.isnan(a)] = np.nan
    return a


def assert_bit_exact(actual, expected, what=""):
    actual, expected = _canonical_nan(actual), _canonical_nan(expected)
    assert actual.shape == expected.shape, f"{what}: shape {actual.shape} vs {expected.shape}"
    ba, be = bits(actual), bits(expected)
    if not np.array_equal(ba, be):
        bad = np.flatnonzero(ba.ravel() != be.ravel())
        i = bad[0]
        raise AssertionError(f"{what}: {bad.size} of {ba.size} elements differ; first at {i}: "
                             f"{actual.ravel()[i]!r} vs {expected.ravel()[i]!r}")


def ref_metric(actual, expected):
    """The reference's own acceptance metric (test/onnx_importer_test.cpp:161-177):
    max_abs and max(|a-r| / max(1,|r|))."""
    a = np.asarray(actual, dtype=np.float64)
    r = np.asarray(expected, dtype=np.float64)
    diff = np.abs(a - r)
    return float(diff.max(initial=0.0)), float((diff / np.maximum(1.0, np.abs(r))).max(initial=0.0))


def assert_close(actual, expected, tol, what=""):
    assert np.asarray(actual).shape == np.asarray(expected).shape, what
    max_abs, max_rel = ref_metric(actual, expected)
    assert np.isfinite(max_abs) and (max_abs <= tol or max_rel <= tol), \
        f"{what}: max_abs={max_abs:.3e} max_rel={max_rel:.3e} tol={tol}"
