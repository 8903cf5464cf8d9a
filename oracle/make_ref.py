"""Recipe: place an UNMODIFIED copy of the reference's Python modules under `oracle/_ref/`.

TEST INFRASTRUCTURE ONLY.  The reference (tuzbing/autograd) is pure Python + numpy on its CPU
path, so "building" it means copying the handful of flat top-level modules its
`Runtime(device="cpu")` needs, byte for byte, into a folder that source control ignores and
that travels with a snapshot of the tree the way a built library does.  With that folder
present the checker can run the reference's own CPU backend - and the reference's own
`Runtime(device="cuda")` hot loop in front of this package's backend - on a machine that has
no reference checkout.

    python oracle/make_ref.py [--reference /path/to/autograd]

The reference imports `metal_ext` (its Apple-only native extension) at import time
(storage.py:4, backend.py:16); the only file written here that is not a copy is a stub of
that name whose `MetalContext` raises on use.  A MANIFEST lists the SHA-256 of every copied
file so that a stale or edited copy shows.

Nothing in the shipped package imports `oracle/_ref`: tests, the smoke check and the CPU arm
of the benchmark do.
"""
from __future__ import annotations

import argparse
import hashlib
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")

# What `Runtime(device="cpu")`, the op/tensor IR, the models and the optimizer import, transitively.
MODULES = ("backend.py", "device.py", "gemm.py", "module.py", "op.py", "optimizer.py", "runtime.py", "scratch.py",
           "storage.py", "tensor.py", "utils.py")

STUB = '''"""Stand-in for the reference's Apple-only native extension: importable, unusable."""


class MetalContext:
    def __init__(self, *args, **kwargs):
        raise RuntimeError("metal_ext is not available on this host")
'''


def default_reference():
    return os.environ.get("AUTOGRAD_REFERENCE", "")


def _sha(path):
    h = hashlib.sha256()
    with open(path, "rb") as f:
        h.update(f.read())
    return h.hexdigest()


def is_current(reference):
    """True when every module under DEST is byte-identical to the checkout's."""
    for name in MODULES:
        src, dst = os.path.join(reference, name), os.path.join(DEST, name)
        if not os.path.exists(dst) or _sha(src) != _sha(dst):
            return False
    return os.path.exists(os.path.join(DEST, "metal_ext.py"))


def make_ref(reference=None, force=False):
    """Copy the modules; returns DEST, or None when no checkout is available (the folder
    made on a machine that has one is then used as it is)."""
    reference = reference or default_reference()
    if not reference or not os.path.exists(os.path.join(reference, "runtime.py")):
        return None
    if not force and is_current(reference):
        return DEST
    os.makedirs(DEST, exist_ok=True)
    lines = []
    for name in MODULES:
        src = os.path.join(reference, name)
        shutil.copyfile(src, os.path.join(DEST, name))
        lines.append(f"{_sha(src)}  {name}")
    with open(os.path.join(DEST, "metal_ext.py"), "w") as f:
        f.write(STUB)
    with open(os.path.join(DEST, "MANIFEST"), "w") as f:
        f.write("unmodified copies of the reference's modules (sha256  name); metal_ext.py is a stub\n")
        f.write("\n".join(lines) + "\n")
    return DEST


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=default_reference())
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    out = make_ref(a.reference, a.force)
    if out is None:
        sys.exit("no reference checkout: pass --reference or set AUTOGRAD_REFERENCE")
    print(out)
