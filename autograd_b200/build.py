"""Build the C-ABI library `libautograd_b200.so` from csrc/*.cu with nvcc for sm_100a.

The library is built in-tree (next to this file) so that it travels with a source snapshot;
it links only against the CUDA runtime (no torch, no Python).  `python -m autograd_b200.build`
rebuilds when a source is newer than the library.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
LIB = os.path.join(HERE, "libautograd_b200.so")
OBJ_DIR = os.path.join(HERE, "build")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
    "-I", INCLUDE, "-I", CSRC,
]


def _nvcc():
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    return hs


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(p) > t for p in sources() + _headers() + [__file__])


def build(force=False, verbose=False, ptxas_info=False):
    if not force and not needs_build():
        return LIB
    os.makedirs(OBJ_DIR, exist_ok=True)
    hdr_time = max(os.path.getmtime(p) for p in _headers() + [__file__])

    def compile_one(src):
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        if not force and os.path.exists(obj) and os.path.getmtime(obj) > max(os.path.getmtime(src), hdr_time):
            return obj, ""
        cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + ["-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        return obj, r.stderr

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        results = list(ex.map(compile_one, sources()))
    objs = [o for o, _ in results]
    if verbose or ptxas_info:
        for _, log in results:
            if log:
                sys.stderr.write(log)
    cmd = [_nvcc(), "-shared", "-o", LIB] + objs + ["-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


def pybind_module_path():
    import sysconfig
    return os.path.join(HERE, "cuda_ext" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))


def build_pybind(force=False, verbose=False):
    """Compile csrc/cuda_ext.cpp (the pybind11 form of the binding; host C++ only, links against the library
    next to it).  Returns the module path, or None where pybind11 or the Python headers are absent - the ctypes
    binding, which needs neither, is the default."""
    import sysconfig
    try:
        import pybind11
    except ImportError:
        return None
    py_inc = sysconfig.get_paths()["include"]
    if not os.path.exists(os.path.join(py_inc, "Python.h")):
        return None
    src = os.path.join(CSRC, "cuda_ext.cpp")
    out = pybind_module_path()
    deps = [src, LIB] + [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    if not force and os.path.exists(out) and all(os.path.getmtime(out) >= os.path.getmtime(d) for d in deps):
        return out
    cmd = [shutil.which("g++") or "g++", "-O2", "-shared", "-fPIC", "-std=c++17", "-fvisibility=hidden",
           "-I", py_inc, "-I", pybind11.get_include(), "-I", INCLUDE, src, "-o", out,
           "-L", HERE, "-lautograd_b200", "-Wl,-rpath,$ORIGIN"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"g++ failed for {src}:\n{r.stdout}\n{r.stderr}")
    if verbose and r.stderr:
        sys.stderr.write(r.stderr)
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv))
    print(build_pybind(force="--force" in sys.argv, verbose=True) or "pybind11 module skipped (pybind11 or Python.h absent)")
