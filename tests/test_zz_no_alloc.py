"""The allocation-free LayerNorm backward (ag_layernorm_backward_noalloc).

Some callers of the library cannot supply the partial-sum workspace that
ag_layernorm_backward asks for: they were handed only the op's tensors, or they run where
device allocation is not allowed.  For them the library keeps a fixed workspace in its own
image.  This test calls that entry point through the C ABI twice in a row, with different
shapes so that the second call runs on top of the first call's leftovers in the shared
workspace, and checks dx, dgamma and dbeta against the regular entry point AND against the
numpy oracle (backend.py:435-487) within the backward tolerance of the parity suite.  Further
cases reach the one piece of logic that only this entry point has - the clip of the grid to the
partial rows that fit the fixed workspace - and the calls that ask for only one of dgamma /
dbeta.  It lives in a file that sorts last so that a run stopping at the first failure has
already gone through every other test.
"""
import numpy as np
import pytest

import gpu_util as G
from conftest import TOL_BWD, assert_close
from oracle import fused_layers as O

pytestmark = pytest.mark.gpu


def _case(ctx, N, C, seed, with_resid, want=("dgamma", "dbeta")):
    rng = np.random.default_rng(seed)
    x_ = rng.standard_normal((N, C), dtype=np.float32)
    dy_ = rng.standard_normal((N, C), dtype=np.float32)
    g_ = (1 + 0.02 * rng.standard_normal(C)).astype(np.float32)
    resid_ = rng.standard_normal((N, C), dtype=np.float32) if with_resid else np.zeros((N, C), np.float32)
    eps = 1e-5
    out = {}
    for which in ("regular", "noalloc"):
        x, dy, gamma = G.up(x_), G.up(dy_), G.up(g_)
        dx = G.up(resid_)
        dgamma, dbeta = G.up(np.full(C, 0.5, np.float32)), G.up(np.full(C, -0.25, np.float32))
        a = lambda t: t.storage.ptr.address  # noqa: E731
        pg = a(dgamma) if "dgamma" in want else 0
        pb = a(dbeta) if "dbeta" in want else 0
        if which == "regular":
            nbytes = ctx.norm_partials_bytes(C)
            ws = G.empty((nbytes,), np.uint8)
            ctx.layernorm_backward(a(dy), a(x), a(gamma), a(dx), a(dx), pg, pb, a(ws), nbytes, N, C, eps)
        else:
            ws = None
            ctx.layernorm_backward_noalloc(a(dy), a(x), a(gamma), a(dx), a(dx), pg, pb, N, C, eps)
        out[which] = (G.down(dx), G.down(dgamma), G.down(dbeta))
        assert ctx.status() == 0
        G.free(x, dy, gamma, dx, dgamma, dbeta, ws)
    # the oracle, with the same pre-loaded gradients; a gradient that was not asked for keeps its value
    g0, b0 = np.full(C, 0.5, np.float32), np.full(C, -0.25, np.float32)
    dx_ref, dg_ref, db_ref = O.layernorm_backward(x_, g_, dy_, eps, resid_, g0, b0)
    oracle = (dx_ref, dg_ref if "dgamma" in want else g0, db_ref if "dbeta" in want else b0)
    for name, got, ref, orc in zip(("dx", "dgamma", "dbeta"), out["noalloc"], out["regular"], oracle):
        assert_close(got, ref, TOL_BWD, f"noalloc {name} vs the regular entry point N={N} C={C}")
        assert_close(got, orc, TOL_BWD, f"noalloc {name} vs the oracle N={N} C={C}")


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    ctx, alloc, be = G.env()
    _case(ctx, 4096, 1280, seed=11, with_resid=True)     # first call on this device resolves the symbol
    _case(ctx, 1500, 384, seed=12, with_resid=False)     # second call reuses the workspace as left behind
    _case(ctx, 33, 101, seed=13, with_resid=True)        # ragged width: scalar kernels, same workspace
    assert ctx.status() == 0


def test_noalloc_grid_is_clipped_to_the_fixed_workspace():
    """8 MiB hold 8 MiB / (2 * C * 4) partial rows: 512 at C 2048 (row-in-registers kernel, which would
    otherwise launch more CTAs for 8192 rows) and 256 at C 4096 (the widest row the entry point takes;
    the generic kernel would use 592).  Then the calls that want only one of the two column sums."""
    ctx, alloc, be = G.env()
    _case(ctx, 8192, 2048, seed=14, with_resid=True)
    _case(ctx, 4096, 4096, seed=15, with_resid=False)
    _case(ctx, 2048, 1280, seed=16, with_resid=True, want=("dgamma",))
    _case(ctx, 2048, 384, seed=17, with_resid=False, want=("dbeta",))
    assert ctx.status() == 0


def test_noalloc_rejects_rows_beyond_its_limit():
    import autograd_b200 as ag
    ctx, alloc, be = G.env()
    C = 4096 + 4
    t = G.up(np.zeros((2, C), np.float32))
    g = G.up(np.ones(C, np.float32))
    a = lambda s: s.storage.ptr.address  # noqa: E731
    with pytest.raises(ag.AgError, match="exceeds the built-in workspace limit"):
        ctx.layernorm_backward_noalloc(a(t), a(t), a(g), 0, a(t), a(g), a(g), 2, C, 1e-5)
    ctx.synchronize()
    G.free(t, g)
