import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


def rel_l2(a, b):
    a = np.asarray(a).astype(np.complex128 if np.iscomplexobj(a) or np.iscomplexobj(b) else np.float64)
    b = np.asarray(b).astype(a.dtype)
    den = np.linalg.norm(b.reshape(-1))
    return float(np.linalg.norm((a - b).reshape(-1)) / (den if den > 0 else 1.0))


def max_rel(a, b):
    """Max over elements of |a-b| / max(|b|, rms(b)): the elementwise relative error, where
    entries smaller than the tensor's RMS are judged on the RMS scale. (A float32 dot product is
    only accurate relative to the size of its terms, so entries that are small through
    cancellation cannot be compared on their own magnitude; the reference's metric also floors the
    denominator, array_conversions.mojo:63-135.)"""
    a = np.asarray(a, dtype=np.float64).reshape(-1)
    b = np.asarray(b, dtype=np.float64).reshape(-1)
    assert a.shape == b.shape, (a.shape, b.shape)
    if b.size == 0:
        return 0.0
    if not (np.all(np.isfinite(a)) and np.all(np.isfinite(b))):
        return float("inf") if not np.array_equal(np.isfinite(a), np.isfinite(b)) else \
            max_rel(np.where(np.isfinite(a), a, 0), np.where(np.isfinite(b), b, 0))
    floor = max(float(np.sqrt(np.mean(b * b))), 1e-30)
    return float((np.abs(a - b) / np.maximum(np.abs(b), floor)).max())


@pytest.fixture(scope="session")
def oracle():
    from oracle import endia_oracle as eo
    eo.build()
    return eo


@pytest.fixture(scope="session")
def nd():
    import endia_b200
    endia_b200._array.device()
    return endia_b200


def rng(seed=0):
    return np.random.Generator(np.random.PCG64(seed))
