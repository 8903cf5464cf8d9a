"""The pybind11 form of the binding on the GPU.

The package calls the C ABI through ctypes by default; `AG_B200_BINDING=pybind11` routes every call
through the compiled module `autograd_b200.cuda_ext` instead (csrc/cuda_ext.cpp - the counterpart of the
reference's pybind11 module, metal_ext.mm:770-796).  The binding is chosen when the package is imported, so
the check runs in a child interpreter: the parity tests against the reference-generated golden vectors
(every kernel family, forward and backward) must pass unchanged through the other binding.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def test_pybind11_binding_passes_the_golden_parity_tests():
    from autograd_b200 import build as agbuild
    if agbuild.build_pybind() is None:
        pytest.skip("pybind11 or the Python headers are not installed")
    env = dict(os.environ, AG_B200_BINDING="pybind11")
    probe = subprocess.run([sys.executable, "-c", "import autograd_b200._native as N; print(N.BINDING)"], env=env,
                           cwd=os.path.dirname(HERE), capture_output=True, text=True, timeout=300)
    assert probe.returncode == 0 and probe.stdout.strip() == "pybind11", probe.stdout + probe.stderr
    run = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu", "-p", "no:cacheprovider",
                          os.path.join(HERE, "test_gpu_parity.py"), "-k", "golden"], env=env,
                         cwd=os.path.dirname(HERE), capture_output=True, text=True, timeout=900)
    tail = (run.stdout + run.stderr)[-3000:]
    assert run.returncode == 0, tail
    assert " passed" in run.stdout and "failed" not in run.stdout, tail
