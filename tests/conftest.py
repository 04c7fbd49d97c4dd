import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def pkg():
    return entry.load_package()


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as o
    o.build()
    return o


@pytest.fixture(scope="session")
def ctx(pkg):
    """A library context on cuda:0. Only GPU tests may request it: there is no CPU path."""
    c = pkg.Context(0)
    yield c
    c.close()


def f16_normal(rng, shape, std=1.0):
    return (rng.standard_normal(shape) * std).astype(np.float16)


def assert_close_ref(got, ref, what="", rel=1e-2):
    """The parity bar: max|got - ref| <= 1e-2 * max|ref| per output tensor."""
    got = np.asarray(got, np.float32)
    ref = np.asarray(ref, np.float32)
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    err = float(np.abs(got - ref).max()) if got.size else 0.0
    tol = rel * float(np.abs(ref).max()) if ref.size else 0.0
    assert err <= tol, f"{what}: max abs err {err:.4e} > {tol:.4e}"


def compare_results_f16(expected, actual, eps):
    """compareResultsF16 of the reference's matmul tests (matmul_test.zig:108-152):
    relative error where |expected| > 1 (threshold eps), absolute otherwise (threshold 0.1*eps)."""
    e = np.asarray(expected, np.float32)
    a = np.asarray(actual, np.float32)
    assert e.shape == a.shape
    diff = np.abs(e - a)
    big = np.abs(e) > 1.0
    err = np.where(big, diff / np.where(big, np.abs(e), 1.0), diff)
    thr = np.where(big, eps, eps * 0.1)
    bad = int((err > thr).sum())
    assert bad == 0, f"{bad} elements differ, max diff {float(diff.max())}"
