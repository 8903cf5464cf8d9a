import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


class Golden:
    """Access to one committed `.npz` of reference-generated vectors: g["case.key"]."""

    def __init__(self, name):
        self._z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))

    def __getitem__(self, key):
        return self._z[key]

    def __contains__(self, key):
        return key in self._z.files

    def cases(self):
        return sorted({k.split(".", 1)[0] for k in self._z.files})


@pytest.fixture(scope="session")
def golden():
    cache = {}

    def get(name):
        if name not in cache:
            cache[name] = Golden(name)
        return cache[name]

    return get


def norm_rel_err(got, ref):
    """max|got-ref| / rms(ref): reported next to failures; strict form of the criterion."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    if ref.size == 0:
        return 0.0
    rms = np.sqrt(np.mean(ref * ref))
    err = np.max(np.abs(got - ref))
    return float(err / rms) if rms > 0 else float(err)


def mixed_rel_err(got, ref):
    """max over elements of |got-ref| / (rms(ref) + |ref|).

    This is the reference's own acceptance form |got-ref| <= atol + rtol*|ref|
    (check_tiny_gpt2_kernel.py:80) with atol = rtol * rms(ref): element-wise relative error is
    meaningless for outputs that cross zero, and a pure norm-relative bound is meaningless for
    heavy-tailed or mostly-zero outputs (a scatter-add gradient, a bf16-rounded product)."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    if ref.size == 0:
        return 0.0
    rms = np.sqrt(np.mean(ref * ref))
    if rms == 0:
        return float(np.max(np.abs(got - ref)))
    return float(np.max(np.abs(got - ref) / (rms + np.abs(ref))))


def assert_close(got, ref, tol, what=""):
    assert np.all(np.isfinite(np.asarray(got, dtype=np.float64))), f"{what}: non-finite values"
    e = mixed_rel_err(got, ref)
    assert e <= tol, (f"{what}: max |d|/(rms+|ref|) = {e:.3e} > {tol:.1e} "
                      f"(max_abs/rms = {norm_rel_err(got, ref):.3e})")


# tolerances of the parity contract
TOL_FWD = 1e-5      # fp32 forward
TOL_BWD = 1e-4      # fp32 backward reductions
TOL_BF16 = 2e-2     # bf16 storage mode
