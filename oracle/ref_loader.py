"""Import the reference's own modules from `oracle/_ref/` (see make_ref.py).

TEST INFRASTRUCTURE ONLY.  The reference is a flat set of top-level modules (`runtime`,
`backend`, `op`, `tensor`, `device`, ...), so loading it means putting that folder first on
`sys.path`; the names then live in `sys.modules` for the rest of the process.
"""
from __future__ import annotations

import importlib
import os
import sys
from types import SimpleNamespace

REF_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")

_NAMES = ("utils", "tensor", "op", "gemm", "scratch", "storage", "backend", "device", "runtime", "module", "optimizer")


def available() -> bool:
    return os.path.exists(os.path.join(REF_DIR, "runtime.py"))


def load():
    """Namespace of the reference's modules.  Raises when the folder has not been made."""
    if not available():
        raise RuntimeError(f"{REF_DIR} is missing: run `python oracle/make_ref.py --reference <checkout>` on a "
                           "machine that has the reference")
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    mods = {}
    for n in _NAMES:
        m = importlib.import_module(n)
        where = os.path.dirname(os.path.abspath(getattr(m, "__file__", "")))
        if where != REF_DIR:
            raise RuntimeError(f"module {n!r} was already imported from {where}, not from {REF_DIR}")
        mods[n] = m
    return SimpleNamespace(**mods)


def blas_info() -> str:
    """numpy version and the BLAS it links, for the parity / timing reports (the reference pins neither)."""
    import numpy as np
    try:
        cfg = np.show_config(mode="dicts")
        blas = cfg.get("Build Dependencies", {}).get("blas", {})
        return f"numpy {np.__version__}, BLAS {blas.get('name', '?')} {blas.get('version', '')}".strip()
    except Exception:
        return f"numpy {np.__version__}"
