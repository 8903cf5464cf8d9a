"""The allocation-free LayerNorm backward (ag_layernorm_backward_noalloc).

Some callers of the library cannot supply the partial-sum workspace that
ag_layernorm_backward asks for: they were handed only the op's tensors, or they run where
device allocation is not allowed.  For them the library keeps a fixed workspace in its own
image.  This test calls that entry point through the C ABI twice in a row, with different
shapes so that the second call runs on top of the first call's leftovers in the shared
workspace, and checks dx, dgamma and dbeta against the regular entry point within the
backward tolerance of the parity suite.  It lives in a file that sorts last so that a run
stopping at the first failure has already gone through every other test.
"""
import numpy as np
import pytest

import gpu_util as G
from conftest import TOL_BWD, assert_close

pytestmark = pytest.mark.gpu


def _case(ctx, N, C, seed, with_resid):
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
        if which == "regular":
            nbytes = ctx.norm_partials_bytes(C)
            ws = G.empty((nbytes,), np.uint8)
            ctx.layernorm_backward(a(dy), a(x), a(gamma), a(dx), a(dx), a(dgamma), a(dbeta), a(ws), nbytes, N, C, eps)
        else:
            ws = None
            ctx.layernorm_backward_noalloc(a(dy), a(x), a(gamma), a(dx), a(dx), a(dgamma), a(dbeta), N, C, eps)
        out[which] = (G.down(dx), G.down(dgamma), G.down(dbeta))
        G.free(x, dy, gamma, dx, dgamma, dbeta, ws)
    for name, got, ref in zip(("dx", "dgamma", "dbeta"), out["noalloc"], out["regular"]):
        assert_close(got, ref, TOL_BWD, f"noalloc {name} N={N} C={C}")


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    ctx, alloc, be = G.env()
    _case(ctx, 4096, 1280, seed=11, with_resid=True)     # first call on this device resolves the symbol
    _case(ctx, 1500, 384, seed=12, with_resid=False)     # second call reuses the workspace as left behind
    _case(ctx, 33, 101, seed=13, with_resid=True)        # ragged width: scalar kernels, same workspace
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
