"""Build entry point in the style of the reference's own native extension (its setup.py builds
metal_ext.mm): `python setup.py build_ext --inplace` compiles the CUDA sources for sm_100a into
autograd_b200/libautograd_b200.so with nvcc, and csrc/cuda_ext.cpp into the pybind11 module
autograd_b200/cuda_ext*.so with g++.  The library is a plain C-ABI shared object (no Python or torch
symbols); the package binds it with ctypes by default (no per-Python-version artefact needed) and
through the pybind11 module with AG_B200_BINDING=pybind11."""
import importlib.util
import os

from setuptools import Command, setup

HERE = os.path.dirname(os.path.abspath(__file__))


def _load_builder():
    spec = importlib.util.spec_from_file_location("_ag_b200_build", os.path.join(HERE, "autograd_b200", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class BuildCuda(Command):
    description = "compile the sm_100a kernels and the C ABI with nvcc"
    user_options = [("force", "f", "rebuild even if the library is up to date"), ("inplace", "i", "accepted for familiarity")]
    boolean_options = ["force", "inplace"]

    def initialize_options(self):
        self.force = False
        self.inplace = True

    def finalize_options(self):
        pass

    def run(self):
        builder = _load_builder()
        print(builder.build(force=bool(self.force), verbose=True))
        print(builder.build_pybind(force=bool(self.force), verbose=True) or "pybind11 module skipped (pybind11 or Python.h absent)")


setup(
    name="autograd_b200",
    version="0.1.0",
    description="B200-native CUDA backend for the fused layer kernels of tuzbing/autograd",
    packages=["autograd_b200"],
    package_data={"autograd_b200": ["libautograd_b200.so", "cuda_ext*.so", "csrc/*"]},
    cmdclass={"build_ext": BuildCuda},
)
