"""GPU parity: CUDA kernels (through the backend callables -> C ABI) against the committed
reference-generated golden vectors and, at larger sizes, against the numpy oracle."""
import numpy as np
import pytest

import gpu_util as G
from conftest import TOL_BF16, TOL_BWD, TOL_FWD, assert_close, mixed_rel_err
from oracle import fused_layers as O

pytestmark = pytest.mark.gpu


# ------------------------------------------------------------------------------ context
def test_context_reports_b200():
    ctx, _, _ = G.env()
    assert ctx.compute_capability[0] == 10
    assert ctx.sm_count > 0 and ctx.l2_bytes > 0


def test_fill_and_copy_roundtrip():
    ctx, alloc, be = G.env()
    rng = np.random.default_rng(0)
    for n in (1, 3, 4, 5, 1023, 4096 + 7):
        a = rng.standard_normal(n).astype(np.float32)
        t = G.up(a)
        assert np.array_equal(G.down(t), a)
        be.fill(t, 2.5)
        assert np.array_equal(G.down(t), np.full(n, 2.5, np.float32))
        be.fill(t, 0.0)
        assert np.array_equal(G.down(t), np.zeros(n, np.float32))
        G.free(t)
    # odd alignment of a view: fill must not touch neighbours
    base = G.up(np.zeros(64, np.float32))
    view = type(base)((13,), np.float32)
    view.storage = alloc.view(base.storage, 4 * 3, (13,), np.float32)
    be.fill(view, 7.0)
    got = G.down(base)
    exp = np.zeros(64, np.float32)
    exp[3:16] = 7.0
    assert np.array_equal(got, exp)
    # int32 and bf16 storages
    ti = G.up(np.arange(10, dtype=np.int32), requires_grad=False)
    be.fill_storage2(ti.storage, 0)
    assert np.array_equal(G.down(ti), np.zeros(10, np.int32))
    tb = G.empty((9,), np.uint16)
    be.fill_storage2(tb.storage, 1.0)
    assert np.array_equal(G.down(tb), np.ones(9, np.float32))
    G.free(base, ti, tb)


# ------------------------------------------------------------------------------ add + layernorm
def _ln_case(g, c):
    return {k: g[f"{c}.{k}"] for k in ("x", "r", "gamma", "beta", "dy", "y", "dx", "dr", "dgamma", "dbeta", "resid",
                                       "dh_with_resid")}, float(g[f"{c}.eps"])


@pytest.mark.parametrize("case", ["probe", "c384", "ragged", "c100", "c1280"])
def test_add_layernorm_golden_unfused(golden, case):
    """AddOp node then LayerNormOp node, as the reference graph runs them."""
    ctx, alloc, be = G.env()
    d, eps = _ln_case(golden("add_layernorm"), case)
    x, r = G.up(d["x"], grad=0), G.up(d["r"], grad=0)
    gamma, beta = G.up(d["gamma"], grad=0), G.up(d["beta"], grad=0)
    h = G.empty(d["x"].shape, grad=0)
    y = G.empty(d["x"].shape, grad=d["dy"])
    add = G.node("AddOp", (x, r), (h,))
    ln = G.node("LayerNormOp", (h, gamma, beta), (y,), eps=eps, normalized_dim=-1)
    be.bind_add_forward(add)(add.inputs, add.outputs)
    G.run_forward(ln)
    assert_close(G.down(y), d["y"], TOL_FWD, "y")
    G.run_backward(ln)
    be.bind_add_backward(add)(add.inputs, add.outputs)
    assert_close(G.down(x.grad), d["dx"], TOL_BWD, "dx")
    assert_close(G.down(r.grad), d["dr"], TOL_BWD, "dr")
    assert_close(G.down(gamma.grad), d["dgamma"], TOL_BWD, "dgamma")
    assert_close(G.down(beta.grad), d["dbeta"], TOL_BWD, "dbeta")
    G.check_clean_status()
    G.free(x, r, gamma, beta, h, y)


@pytest.mark.parametrize("case", ["probe", "c384", "ragged", "c100", "c1280"])
def test_add_layernorm_golden_fused(golden, case):
    """One fused kernel for add + LayerNorm; backward with a pre-loaded residual gradient
    (the reference's own test of the fused residual-grad add, debug/check_qwen_kernel.py:471-487)."""
    ctx, alloc, be = G.env()
    d, eps = _ln_case(golden("add_layernorm"), case)
    shape = d["x"].shape
    rows = int(np.prod(shape[:-1]))
    x, r = G.up(d["x"]), G.up(d["r"])
    gamma, beta = G.up(d["gamma"], grad=0), G.up(d["beta"], grad=0)
    h = G.empty(shape, grad=d["resid"])
    y = G.empty(shape, grad=d["dy"])
    mean, rstd = G.empty((rows,)), G.empty((rows,))
    be.fused_add_layernorm_forward(x, r, gamma, beta, h, y, eps, mean, rstd)
    h_ref, y_ref, mean_ref, rstd_ref = O.add_layernorm_forward(d["x"], d["r"], d["gamma"], d["beta"], eps)
    assert np.array_equal(G.down(h), h_ref)
    assert_close(G.down(y), d["y"], TOL_FWD, "y")
    assert_close(G.down(mean).reshape(mean_ref.shape), mean_ref, TOL_FWD, "mean")
    assert_close(G.down(rstd).reshape(rstd_ref.shape), rstd_ref, TOL_FWD, "rstd")
    ln = G.node("LayerNormOp", (h, gamma, beta), (y,), eps=eps, normalized_dim=-1)
    G.run_backward(ln)
    assert_close(G.down(h.grad), d["dh_with_resid"], TOL_BWD, "dh")
    assert_close(G.down(gamma.grad), d["dgamma"], TOL_BWD, "dgamma")
    assert_close(G.down(beta.grad), d["dbeta"], TOL_BWD, "dbeta")
    # accumulation into dgamma/dbeta: a second backward doubles them
    be.fill(h.grad, 0.0)
    G.run_backward(ln)
    assert_close(G.down(gamma.grad), 2 * d["dgamma"], TOL_BWD, "dgamma x2")
    G.check_clean_status()
    G.free(x, r, gamma, beta, h, y, mean, rstd)


def _cfg1_inputs(N=16384, C=384, seed=1234):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((N, C), dtype=np.float32)
    r = rng.standard_normal((N, C), dtype=np.float32)
    gamma = (1 + 0.02 * rng.standard_normal(C)).astype(np.float32)
    beta = (0.02 * rng.standard_normal(C)).astype(np.float32)
    dy = rng.standard_normal((N, C), dtype=np.float32)
    return x, r, gamma, beta, dy


@pytest.mark.parametrize("N,C", [(16384, 384), (4096, 1280), (1000, 1536), (777, 2048), (300, 4100), (32768, 1280),
                                 (8192, 1536), (1, 384), (9, 1280)])
def test_add_layernorm_full_size_vs_oracle(N, C):
    """Config 1 (16384 x 384, eps 1e-5), the benchmark step's shape (32768 x 1280: every CTA walks
    many rows, the grid is one resident wave) and the other row widths of the path."""
    ctx, alloc, be = G.env()
    eps = 1e-5
    x_, r_, g_, b_, dy_ = _cfg1_inputs(N, C)
    x, r = G.up(x_), G.up(r_)
    gamma, beta = G.up(g_, grad=0), G.up(b_, grad=0)
    h, y = G.empty((N, C), grad=0), G.empty((N, C), grad=dy_)
    mean, rstd = G.empty((N,)), G.empty((N,))
    be.fused_add_layernorm_forward(x, r, gamma, beta, h, y, eps, mean, rstd)
    h_ref, y_ref, mean_ref, rstd_ref = O.add_layernorm_forward(x_, r_, g_, b_, eps)
    assert np.array_equal(G.down(h), h_ref)
    assert_close(G.down(y), y_ref, TOL_FWD, "y")
    assert_close(G.down(mean), mean_ref, TOL_FWD, "mean")
    assert_close(G.down(rstd), rstd_ref, TOL_FWD, "rstd")
    ln = G.node("LayerNormOp", (h, gamma, beta), (y,), eps=eps, normalized_dim=-1)
    G.run_backward(ln)
    z = np.zeros_like(x_)
    dh_ref, dg_ref, db_ref = O.layernorm_backward(h_ref, g_, dy_, eps, z, np.zeros_like(g_), np.zeros_like(b_))
    assert_close(G.down(h.grad), dh_ref, TOL_BWD, "dh")
    assert_close(G.down(gamma.grad), dg_ref, TOL_BWD, "dgamma")
    assert_close(G.down(beta.grad), db_ref, TOL_BWD, "dbeta")
    # fixed summation order: a repeat gives identical bits
    first = G.down(gamma.grad).copy()
    be.fill(gamma.grad, 0.0)
    be.fill(beta.grad, 0.0)
    be.fill(h.grad, 0.0)
    G.run_backward(ln)
    assert np.array_equal(G.down(gamma.grad), first)
    G.check_clean_status()
    G.free(x, r, gamma, beta, h, y, mean, rstd)


# ------------------------------------------------------------------------------ GELU
@pytest.mark.parametrize("case", ["probe", "ragged", "wide"])
def test_gelu_golden(golden, case):
    g = golden("gelu")
    x_, dy_, pre_ = g[f"{case}.x"], g[f"{case}.dy"], g[f"{case}.pre"]
    x = G.up(x_, grad=pre_)
    y = G.empty(x_.shape, grad=dy_)
    n = G.node("GELUOp", (x,), (y,))
    G.run_forward(n)
    assert_close(G.down(y), g[f"{case}.y"], TOL_FWD, "y")
    G.run_backward(n)
    assert_close(G.down(x.grad), g[f"{case}.dx"], TOL_BWD, "dx")
    G.free(x, y)


@pytest.mark.parametrize("rows,cols", [(16384, 1536), (32768, 5120)])
def test_gelu_full_size_vs_oracle(rows, cols):
    """16384 x 1536, and the MLP activation of the benchmark step (32768 x 5120)."""
    rng = np.random.default_rng(1239)
    x_ = (2.0 * rng.standard_normal((rows, cols), dtype=np.float32)).astype(np.float32)
    x_[0, :8] = [0.0, -0.0, 30.0, -30.0, 1e-20, -1e-20, 9.0, -9.0]
    dy_ = rng.standard_normal(x_.shape, dtype=np.float32)
    x = G.up(x_, grad=0)
    y = G.empty(x_.shape, grad=dy_)
    n = G.node("GELUOp", (x,), (y,))
    G.run_forward(n)
    assert_close(G.down(y), O.gelu_forward(x_), TOL_FWD, "y")
    G.run_backward(n)
    assert_close(G.down(x.grad), O.gelu_backward(x_, dy_, np.zeros_like(x_)), TOL_BWD, "dx")
    G.free(x, y)


# ------------------------------------------------------------------------------ RMSNorm / SwiGLU
@pytest.mark.parametrize("case", ["qwenish", "nogamma", "ragged"])
def test_rmsnorm_swiglu_golden(golden, case):
    ctx, alloc, be = G.env()
    g = golden("rmsnorm_swiglu")
    x_, eps = g[f"{case}.x"], float(g[f"{case}.eps"])
    has_gamma = f"{case}.gamma" in g
    x = G.up(x_, grad=g[f"{case}.resid"])
    gamma = G.up(g[f"{case}.gamma"], grad=0) if has_gamma else None
    y = G.empty(x_.shape)
    inv = G.empty((x_.shape[0],))
    be.rmsnorm_forward(x, gamma, y, eps, inv)
    assert_close(G.down(inv), g[f"{case}.inv_rms"], TOL_FWD, "inv_rms")
    assert_close(G.down(y), g[f"{case}.x_norm"], TOL_FWD, "x_norm")
    dz = G.up(g[f"{case}.dz"])
    be.rmsnorm_backward(dz, x, gamma, eps, x.grad, gamma.grad if has_gamma else None, dres=x.grad)
    assert_close(G.down(x.grad), g[f"{case}.dx_with_resid"], TOL_BWD, "dx")
    if has_gamma:
        assert_close(G.down(gamma.grad), g[f"{case}.dgamma"], TOL_BWD, "dgamma")
    gu = G.up(g[f"{case}.gu"])
    hidden = G.empty(g[f"{case}.hidden"].shape)
    be.swiglu_forward(gu, hidden)
    assert_close(G.down(hidden), g[f"{case}.hidden"], TOL_FWD, "hidden")
    dh = G.up(g[f"{case}.dhidden"])
    be.swiglu_backward(gu, dh)
    assert_close(G.down(gu), g[f"{case}.dgu"], TOL_BWD, "dgu")
    G.check_clean_status()
    G.free(x, gamma, y, inv, dz, gu, hidden, dh)


def _bf16(a):
    return O.round_to_bf16(a)


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_qwen_path_config3_reduced(dtype):
    """Config 3 shapes (C 1536, 12/2 heads x 128, I 8960, eps 1e-6, theta 1e6) at a reduced
    token count, fp32 and bf16 storage, against the fp32 oracle."""
    _qwen_path(dtype, 2, 192)


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_qwen_path_config3_full_size(dtype):
    """Config 3 at its stated size: batch 4 x seq 2048 = 8192 token rows, positions 0..2047."""
    _qwen_path(dtype, 4, 2048)


def _qwen_path(dtype, B, T):
    ctx, alloc, be = G.env()
    C, H, HKV, D, I, eps = 1536, 12, 2, 128, 8960, 1e-6
    N = B * T
    rng = np.random.default_rng(1236)
    bf = dtype == "bf16"
    tol_f, tol_b = (TOL_BF16, TOL_BF16) if bf else (TOL_FWD, TOL_BWD)
    st = np.uint16 if bf else np.float32

    def dev(a):
        if not bf:
            return G.up(a)
        t = G.empty(a.shape, np.uint16)
        be.copy_from_host(t, a)
        return t

    def prep(a):
        return _bf16(a) if bf else a

    x_ = prep(rng.standard_normal((N, C), dtype=np.float32))
    gamma_ = (1 + 0.02 * rng.standard_normal(C)).astype(np.float32)
    dz_ = prep(rng.standard_normal((N, C), dtype=np.float32))
    resid_ = prep(rng.standard_normal((N, C), dtype=np.float32))
    # RMSNorm
    x, dz, dxt = dev(x_), dev(dz_), dev(resid_)
    gamma = G.up(gamma_, grad=0)
    y = G.empty((N, C), st)
    inv = G.empty((N,))
    be.rmsnorm_forward(x, gamma, y, eps, inv)
    z_ref, inv_ref = O.rmsnorm_forward(x_, gamma_, eps)
    assert_close(G.down(inv), inv_ref, TOL_FWD, "inv_rms")
    assert_close(G.down(y), z_ref, tol_f, "rmsnorm y")
    be.rmsnorm_backward(dz, x, gamma, eps, dxt, gamma.grad, dres=dxt)
    dx_ref, dg_ref = O.rmsnorm_backward(x_, gamma_, dz_, eps, resid_, np.zeros_like(gamma_))
    assert_close(G.down(dxt), dx_ref, tol_b, "rmsnorm dx")
    assert_close(G.down(gamma.grad), dg_ref, TOL_BWD if not bf else TOL_BF16, "rmsnorm dgamma")
    G.free(x, dz, dxt, gamma, y, inv)
    # RoPE, rope_sign=+1 forward then its transpose as backward
    q_ = prep(rng.standard_normal((B, T, H, D), dtype=np.float32))
    k_ = prep(rng.standard_normal((B, T, HKV, D), dtype=np.float32))
    cos_, sin_ = O.rope_tables(T, D, 1e6)
    q, k, cos, sin = dev(q_), dev(k_), G.up(cos_), G.up(sin_)
    be.rope_qk(q, k, cos, sin, sin_sign=+1)
    q_ref, k_ref = O.rope_apply(q_, cos_, sin_, +1), O.rope_apply(k_, cos_, sin_, +1)
    assert_close(G.down(q), q_ref, tol_f, "rope q")
    assert_close(G.down(k), k_ref, tol_f, "rope k")
    be.rope_qk(q, k, cos, sin, sin_sign=-1)
    assert_close(G.down(q), q_, 2 * tol_f, "rope q roundtrip")
    G.free(q, k, cos, sin)
    # SwiGLU
    gu_ = prep(rng.standard_normal((N, 2 * I), dtype=np.float32))
    dh_ = prep(rng.standard_normal((N, I), dtype=np.float32))
    gu, dh = dev(gu_), dev(dh_)
    hidden = G.empty((N, I), st)
    be.swiglu_forward(gu, hidden)
    assert_close(G.down(hidden), O.swiglu_forward(gu_), tol_f, "swiglu hidden")
    be.swiglu_backward(gu, dh)
    assert_close(G.down(gu), O.swiglu_backward(gu_, dh_), tol_b, "swiglu dgu")
    G.check_clean_status()
    G.free(gu, dh, hidden)


# ------------------------------------------------------------------------------ RoPE
@pytest.mark.parametrize("case", ["qwen", "gpt", "tiny"])
def test_rope_golden(golden, case):
    ctx, alloc, be = G.env()
    g = golden("rope")
    q_, k_, cos_, sin_ = (g[f"{case}.{n}"] for n in ("q", "k", "cos", "sin"))
    for sign, tag in ((+1, "pos"), (-1, "neg")):
        q, k, cos, sin = G.up(q_), G.up(k_), G.up(cos_), G.up(sin_)
        be.rope_qk(q, k, cos, sin, sin_sign=sign)
        assert_close(G.down(q), g[f"{case}.q_{tag}"], TOL_FWD, f"q {tag}")
        assert_close(G.down(k), g[f"{case}.k_{tag}"], TOL_FWD, f"k {tag}")
        G.free(q, k, cos, sin)
    # q only
    q, cos, sin = G.up(q_), G.up(cos_), G.up(sin_)
    be.rope_qk(q, None, cos, sin, sin_sign=+1)
    assert_close(G.down(q), g[f"{case}.q_pos"], TOL_FWD, "q only")
    G.check_clean_status()
    G.free(q, cos, sin)


# ------------------------------------------------------------------------------ gather / scatter-add
@pytest.mark.parametrize("case", ["small", "collide", "wide"])
def test_gather_golden(golden, case):
    g = golden("gather")
    ids_, table_, dout_ = g[f"{case}.ids"], g[f"{case}.table"], g[f"{case}.dout"]
    ids = G.up(ids_, requires_grad=False)
    table = G.up(table_, grad=0)
    out = G.empty(dout_.shape, grad=dout_)
    n = G.node("GatherOp", (ids, table), (out,))
    G.run_forward(n)
    assert np.array_equal(G.down(out), g[f"{case}.out"])  # bit-exact
    G.run_backward(n)
    got = G.down(table.grad)
    assert_close(got, g[f"{case}.dtable"], TOL_BWD, "dtable")
    # rows nobody indexed stay exactly zero
    untouched = np.setdiff1d(np.arange(table_.shape[0]), ids_.ravel())
    assert not got[untouched].any()
    G.check_clean_status()
    G.free(ids, table, out)


def _assert_rows_close(got, ref, tol, what):
    """Every table row is an independent sum with its own scale (a hot row collects thousands
    of addends, most rows none): |got-ref| <= tol * (rms(row of ref) + |ref|), rows that
    received nothing must be exactly equal."""
    ref64, got64 = ref.astype(np.float64), got.astype(np.float64)
    row_rms = np.sqrt(np.mean(ref64 * ref64, axis=1, keepdims=True))
    quiet = row_rms[:, 0] == 0
    assert np.array_equal(got[quiet], ref[quiet]), f"{what}: untouched rows differ"
    e = np.max(np.abs(got64 - ref64)[~quiet] / (row_rms[~quiet] + np.abs(ref64[~quiet])))
    assert e <= tol, f"{what}: per-row max |d|/(rms_row+|ref|) = {e:.3e} > {tol:.1e}"


def _zipf_ids(rng, V, n, s=1.1):
    p = 1.0 / np.arange(1, V + 1) ** s
    p /= p.sum()
    return rng.choice(V, size=n, p=p).astype(np.int32)


@pytest.mark.parametrize("V,C,n", [(151936, 1536, 65536), (5000, 100, 4099), (32768, 1280, 32768), (300, 64, 5000),
                                   (700000, 8, 3000), (20000, 64, 300000)])
def test_gather_scatter_full_size(V, C, n):
    """Config 4: 65536 Zipf(1.1) ids over a 151936 x 1536 table; forward bit-exact, backward
    within tolerance of np.add.at, bit-reproducible, and bit-exact for rows whose occurrences
    fall inside one summation group.  The other shapes cover the sort's pass counts (a table of 300
    rows sorts in one 9-bit pass, 700000 rows need three) and the unfused sort that takes over
    beyond 262144 ids."""
    ctx, alloc, be = G.env()
    rng = np.random.default_rng(1237)
    ids_ = _zipf_ids(rng, V, n).reshape(1, n) if V != 32768 else rng.integers(0, V, size=(1, n)).astype(np.int32)
    table_ = (0.02 * rng.standard_normal((V, C), dtype=np.float32)).astype(np.float32)
    dout_ = rng.standard_normal((1, n, C), dtype=np.float32)
    ids = G.up(ids_, requires_grad=False)
    table = G.up(table_, grad=0)
    out = G.empty(dout_.shape, grad=dout_)
    node = G.node("GatherOp", (ids, table), (out,))
    G.run_forward(node)
    assert np.array_equal(G.down(out), O.gather_forward(ids_, table_))
    G.run_backward(node)
    got = G.down(table.grad)
    ref = O.gather_backward(ids_, dout_, np.zeros_like(table_))
    _assert_rows_close(got, ref, TOL_BWD, "dtable")
    # distance to the fp64 sum: the fixed-order grouped sum is no further from it than
    # numpy's sequential fp32 np.add.at (hot rows collect thousands of addends)
    truth = np.zeros(table_.shape, np.float64)
    np.add.at(truth, ids_.ravel().astype(np.int64), dout_.reshape(-1, C).astype(np.float64))
    assert np.max(np.abs(got - truth)) <= 2.0 * np.max(np.abs(ref - truth)) + 1e-12
    counts = np.bincount(ids_.ravel(), minlength=V)
    assert not got[counts == 0].any()
    singles = counts == 1
    assert np.array_equal(got[singles], ref[singles])
    be.fill(table.grad, 0.0)
    G.run_backward(node)
    assert np.array_equal(G.down(table.grad), got)  # deterministic
    # accumulate on top of an existing gradient
    G.run_backward(node)
    _assert_rows_close(G.down(table.grad), 2 * ref, TOL_BWD, "dtable x2")
    G.check_clean_status()
    G.free(ids, table, out)


@pytest.mark.parametrize("group", [32, 64, 128])
def test_scatter_add_group_sizes_agree(group, monkeypatch):
    """The segmented sum cuts the sorted ids into groups of 32 entries, or 64 from 49152 ids on;
    AG_B200_SCATTER_GROUP (read when a context is created) forces 32, 64 or 128.  Every size must give
    the np.add.at result: Zipf ids (segments that span many groups), a ragged last group, the scalar
    path (odd C), accumulation on top of an existing gradient."""
    import autograd_b200 as ag
    from autograd_b200 import hostgraph as hg
    monkeypatch.setenv("AG_B200_SCATTER_GROUP", str(group))
    ctx, alloc, be = ag.create(0)
    try:
        rng = np.random.default_rng(1251)

        def dev(a, requires_grad=False):
            t = hg.HostTensor(a.shape, a.dtype.type, requires_grad=requires_grad)
            t.storage = alloc.alloc(t.shape, t.dtype)
            be.copy_from_host(t, np.ascontiguousarray(a))
            return t

        for V, C, n in ((3000, 256, 20011), (50, 101, 777), (100000, 64, 60000)):
            ids_ = _zipf_ids(rng, V, n).reshape(1, n)
            dout_ = rng.standard_normal((1, n, C), dtype=np.float32)
            base_ = (0.01 * rng.standard_normal((V, C), dtype=np.float32)).astype(np.float32)
            ids, table = dev(ids_), dev(base_, requires_grad=True)
            table.grad = dev(base_)
            out = dev(np.zeros((1, n, C), np.float32), requires_grad=True)
            out.grad = dev(dout_)
            node = hg.make_node(hg.make_op("GatherOp"), (ids, table), (out,))
            be.get_backward_kernel(node.op)(node.inputs, node.outputs)
            got = be.copy_to_host(table.grad)
            ref = O.gather_backward(ids_, dout_, base_.copy())
            _assert_rows_close(got, ref, TOL_BWD, f"dtable group={group} V={V} C={C} n={n}")
            counts = np.bincount(ids_.ravel(), minlength=V)
            assert np.array_equal(got[counts == 0], base_[counts == 0])
            assert ctx.status() == 0
            for t in (ids, table, table.grad, out, out.grad):
                alloc.free(t.storage)
    finally:
        ctx.synchronize()
        alloc.free()
        ctx.close()


def test_gather_bad_index_sets_status_not_fault():
    ctx, alloc, be = G.env()
    table_ = np.arange(12, dtype=np.float32).reshape(3, 4)
    ids = G.up(np.array([[0, 5, -1, 2]], np.int32), requires_grad=False)
    table = G.up(table_, grad=0)
    out = G.empty((1, 4, 4), grad=np.ones((1, 4, 4), np.float32))
    n = G.node("GatherOp", (ids, table), (out,))
    G.run_forward(n)
    got = G.down(out)
    assert np.array_equal(got[0, 0], table_[0]) and np.array_equal(got[0, 3], table_[2])
    assert not got[0, 1].any() and not got[0, 2].any()
    assert ctx.status() & 1
    G.run_backward(n)
    assert ctx.status() & 1
    exp = np.zeros_like(table_)
    exp[0] = 1
    exp[2] = 1
    assert np.array_equal(G.down(table.grad), exp)
    assert ctx.status() == 0
    G.free(ids, table, out)


# ------------------------------------------------------------------------------ fused linear + CE
def _run_flce(be, X_, W_, Y_, precision, ignore_mode, reduction=0, chunk=4096, dloss=1.0):
    import autograd_b200 as ag
    be.ce_precision, be.ce_ignore_mode, be.ce_reduction, be.ce_vocab_chunk = precision, ignore_mode, reduction, chunk
    x = G.up(X_, grad=0)
    w = G.up(W_, grad=0)
    y = G.up(Y_, requires_grad=False)
    loss = G.empty((1,), grad=np.array([dloss], np.float32))
    n = G.node("FusedLinearCrossEntropyOp", (x, w, y), (loss,), ignore_index=-1)
    G.run_forward(n)
    G.run_backward(n)
    res = float(G.down(loss)[0]), G.down(x.grad), G.down(w.grad)
    G.free(x, w, y, loss)
    be.ce_precision, be.ce_ignore_mode, be.ce_reduction, be.ce_vocab_chunk = ag.AG_CE_3XTF32, 0, 0, 4096
    return res


@pytest.mark.parametrize("case", ["small", "ragged", "multi_chunk"])
@pytest.mark.parametrize("precision", [0, 1])
def test_flce_golden(golden, case, precision):
    ctx, alloc, be = G.env()
    g = golden("flce")
    X_, W_, Y_ = g[f"{case}.X"], g[f"{case}.W"], g[f"{case}.Y"]
    N = Y_.size
    # (1) verbatim reference semantics: ignored rows still contribute softmax*scale
    loss, dX, dW = _run_flce(be, X_, W_, Y_, precision, ignore_mode=1, chunk=128)
    assert abs(loss - float(g[f"{case}.loss"][0])) <= TOL_FWD * abs(loss)
    assert_close(dX, g[f"{case}.dX"], TOL_BWD, "dX compat")
    assert_close(dW, g[f"{case}.dW"], TOL_BWD, "dW compat")
    # (2) masked default == the reference run on the valid rows, rescaled by N_valid/N
    keep = g[f"{case}.valid_rows"]
    f = len(keep) / N
    loss, dX, dW = _run_flce(be, X_, W_, Y_, precision, ignore_mode=0, chunk=128)
    assert abs(loss - f * float(g[f"{case}.loss_valid_only"][0])) <= TOL_FWD * abs(loss)
    exp_dX = np.zeros((N, X_.shape[-1]), np.float32)
    exp_dX[keep] = f * g[f"{case}.dX_valid_only"].reshape(len(keep), -1)
    assert_close(dX.reshape(exp_dX.shape), exp_dX, TOL_BWD, "dX masked")
    assert_close(dW, f * g[f"{case}.dW_valid_only"], TOL_BWD, "dW masked")
    assert not dX.reshape(exp_dX.shape)[np.setdiff1d(np.arange(N), keep)].any()  # ignore handling is exact
    # (3) mean over valid rows
    loss_v, dXv, _ = _run_flce(be, X_, W_, Y_, precision, ignore_mode=0, reduction=1, chunk=128)
    assert abs(loss_v - float(g[f"{case}.loss_valid_only"][0])) <= TOL_FWD * abs(loss_v)
    G.check_clean_status()


@pytest.mark.parametrize("N,C,V,precision", [(2048, 384, 8192, 0), (2048, 384, 8192, 1), (1024, 1280, 8192, 1),
                                             (1000, 388, 4104, 1),   # ragged: rows, width and last panel (8 columns)
                                             (2048, 384, 8192, 3), (1024, 1280, 8192, 3), (1000, 392, 4104, 3)])
def test_flce_mid_size_vs_oracle(N, C, V, precision):
    """Config 2 shapes at a reduced token / vocab count, vocab chunk 4096 (two panels)."""
    ctx, alloc, be = G.env()
    rng = np.random.default_rng(1235)
    X_ = (rng.standard_normal((1, N, C)) / np.sqrt(C)).astype(np.float32)
    W_ = (0.02 * rng.standard_normal((V, C))).astype(np.float32)
    Y_ = rng.integers(0, V, size=(1, N)).astype(np.int32)
    Y_[rng.random((1, N)) < 0.05] = -1
    ref = O.flce_masked(X_[0], W_, Y_[0], dloss=0.5)
    loss, dX, dW = _run_flce(be, X_, W_, Y_, precision, ignore_mode=0, chunk=4096, dloss=0.5)
    assert abs(loss - float(ref["loss"])) <= TOL_FWD * abs(loss)
    assert_close(dX[0], ref["dX"], TOL_BWD, "dX")
    assert_close(dW, ref["dW"], TOL_BWD, "dW")
    G.check_clean_status()


@pytest.mark.parametrize("precision", [0, 1, 2, 3])
def test_flce_more_rows_than_one_row_tile(precision):
    """Token rows are taken in tiles of 18944 (one 128-row GEMM tile per SM); 19244 rows = a full tile and
    a ragged one of 300, with a ragged last vocabulary panel."""
    ctx, alloc, be = G.env()
    N, C, V = 18944 + 300, 64, 1000
    rng = np.random.default_rng(1240)
    X_ = (rng.standard_normal((1, N, C)) / np.sqrt(C)).astype(np.float32)
    W_ = (0.02 * rng.standard_normal((V, C))).astype(np.float32)
    Y_ = rng.integers(0, V, size=(1, N)).astype(np.int32)
    Y_[rng.random((1, N)) < 0.05] = -1
    Xo, Wo = (O.round_to_bf16(X_[0]), O.round_to_bf16(W_)) if precision == 2 else (X_[0], W_)
    ref = O.flce_masked(Xo, Wo, Y_[0], dloss=1.0)
    loss, dX, dW = _run_flce(be, X_, W_, Y_, precision, ignore_mode=0, chunk=512, dloss=1.0)
    tol_f, tol_b = (TOL_BF16, TOL_BF16) if precision == 2 else (TOL_FWD, TOL_BWD)
    assert abs(loss - float(ref["loss"])) <= tol_f * abs(loss)
    assert_close(dX[0], ref["dX"], tol_b, "dX")
    assert_close(dW, ref["dW"], tol_b, "dW")
    G.check_clean_status()


@pytest.mark.parametrize("precision", [1, 3])
def test_flce_wide_vocab_panel(precision):
    """Vocabulary panels wider than 4096 columns: the dX contraction is taken in pieces of 4096."""
    ctx, alloc, be = G.env()
    N, C, V = 768, 256, 8192 + 40
    rng = np.random.default_rng(4321)
    X_ = (rng.standard_normal((1, N, C)) / np.sqrt(C)).astype(np.float32)
    W_ = (0.02 * rng.standard_normal((V, C))).astype(np.float32)
    Y_ = rng.integers(0, V, size=(1, N)).astype(np.int32)
    Y_[rng.random((1, N)) < 0.05] = -1
    ref = O.flce_masked(X_[0], W_, Y_[0])
    loss, dX, dW = _run_flce(be, X_, W_, Y_, precision, ignore_mode=0, chunk=8192)
    assert abs(loss - float(ref["loss"])) <= TOL_FWD * abs(loss)
    assert_close(dX[0], ref["dX"], TOL_BWD, "dX")
    assert_close(dW, ref["dW"], TOL_BWD, "dW")
    G.check_clean_status()


@pytest.mark.parametrize("C", [384, 1280])
def test_flce_config2_full_size(C):
    """Config 2 at full size: 16384 tokens, vocab 32768, chunk 4096, 5 % ignored, 3xTF32 tensor-core
    panels against the numpy oracle on the same seeded inputs; plus size-independent properties:
    rows of dX for ignored tokens are exactly zero, every dlogits row sums to zero so that
    sum_v dW[v,:] equals -sum over nothing (checked as column sums of dW against X^T . rowsum = 0)."""
    ctx, alloc, be = G.env()
    N, V = 16384, 32768
    rng = np.random.default_rng(1235 + C)
    X_ = (rng.standard_normal((1, N, C)) / np.sqrt(C)).astype(np.float32)
    W_ = (0.02 * rng.standard_normal((V, C))).astype(np.float32)
    Y_ = rng.integers(0, V, size=(1, N)).astype(np.int32)
    Y_[rng.random((1, N)) < 0.05] = -1
    ref = O.flce_masked(X_[0], W_, Y_[0])
    loss, dX, dW = _run_flce(be, X_, W_, Y_, 1, ignore_mode=0, chunk=4096)
    assert abs(loss - float(ref["loss"])) <= TOL_FWD * abs(loss)
    assert_close(dX[0], ref["dX"], TOL_BWD, "dX")
    assert_close(dW, ref["dW"], TOL_BWD, "dW")
    ignored = Y_[0] < 0
    assert ignored.sum() > 500 and not dX[0][ignored].any()
    # softmax - onehot sums to zero over the vocabulary for every valid row: the column sums of dW vanish
    col = dW.astype(np.float64).sum(axis=0)
    assert np.max(np.abs(col)) <= 1e-4 * np.sqrt(np.mean(dW.astype(np.float64) ** 2)) * np.sqrt(V)
    # mean over valid rows = mean over all rows * N / N_valid (integer bookkeeping of the ignore mask)
    loss_v, _, _ = _run_flce(be, X_, W_, Y_, 1, ignore_mode=0, reduction=1, chunk=4096)
    assert abs(loss_v - loss * N / int((~ignored).sum())) <= 1e-5 * abs(loss_v)
    G.check_clean_status()


@pytest.mark.parametrize("C", [384, 1280])
def test_flce_bf16x3_config2_full_size(C):
    """The bf16 (hi, lo) pair mode (three MMAs at the bf16 rate) at the full config-2 size against the
    fp32 tolerances of the path: loss 1e-5, dX and dW 1e-4 (measured 3e-5 to 5e-5, like 3xTF32, once
    the accumulation chains of dW are bounded by split-K); the measured errors are printed."""
    ctx, alloc, be = G.env()
    N, V = 16384, 32768
    rng = np.random.default_rng(1235 + C)
    X_ = (rng.standard_normal((1, N, C)) / np.sqrt(C)).astype(np.float32)
    W_ = (0.02 * rng.standard_normal((V, C))).astype(np.float32)
    Y_ = rng.integers(0, V, size=(1, N)).astype(np.int32)
    Y_[rng.random((1, N)) < 0.05] = -1
    ref = O.flce_masked(X_[0], W_, Y_[0])
    loss, dX, dW = _run_flce(be, X_, W_, Y_, 3, ignore_mode=0, chunk=4096)
    print(f"bf16x3 C={C}: loss rel {abs(loss - float(ref['loss'])) / abs(loss):.2e}, "
          f"dX {mixed_rel_err(dX[0], ref['dX']):.2e}, dW {mixed_rel_err(dW, ref['dW']):.2e}")
    assert abs(loss - float(ref["loss"])) <= TOL_FWD * abs(loss)
    assert_close(dX[0], ref["dX"], TOL_BWD, "dX")
    assert_close(dW, ref["dW"], TOL_BWD, "dW")
    ignored = Y_[0] < 0
    assert not dX[0][ignored].any()
    G.check_clean_status()


@pytest.mark.parametrize("precision", [1, 3])
def test_flce_wide_hidden_keeps_accumulation_chains_short(precision):
    """16384 rows x hidden 4096: the dW panel has enough tiles to fill the GPU without split-K, and one
    accumulation chain over 16384 rows inside the tensor core is measurably biased (2.7e-4 of the rms
    at hidden 384).  The plan must split K for accuracy, not only for occupancy."""
    ctx, alloc, be = G.env()
    N, C, V = 16384, 4096, 4096
    rng = np.random.default_rng(99)
    X_ = (rng.standard_normal((1, N, C)) / np.sqrt(C)).astype(np.float32)
    W_ = (0.02 * rng.standard_normal((V, C))).astype(np.float32)
    Y_ = rng.integers(0, V, size=(1, N)).astype(np.int32)
    ref = O.flce_masked(X_[0], W_, Y_[0])
    loss, dX, dW = _run_flce(be, X_, W_, Y_, precision, ignore_mode=0, chunk=4096)
    print(f"precision {precision}: dX {mixed_rel_err(dX[0], ref['dX']):.2e}, dW {mixed_rel_err(dW, ref['dW']):.2e}")
    assert abs(loss - float(ref["loss"])) <= TOL_FWD * abs(loss)
    assert_close(dX[0], ref["dX"], TOL_BWD, "dX")
    assert_close(dW, ref["dW"], TOL_BWD, "dW")
    G.check_clean_status()


@pytest.mark.parametrize("N,C,V", [(2048, 384, 8192), (1000, 1280, 4104), (1000, 392, 4104)])
def test_flce_bf16_mode_vs_oracle(N, C, V):
    """The stated bf16 tensor-core mode of the CE GEMMs: 2e-2 against the fp32 oracle run on the
    same bf16-rounded operands (the rounding of X and W is the mode's definition; an element of
    dW that is a near-cancelling sum of two rounded activations cannot be held to 2e-2 of the
    unrounded result by any bf16 implementation), and 2e-2 in rms against the unrounded oracle."""
    ctx, alloc, be = G.env()
    rng = np.random.default_rng(1240)
    X_ = (rng.standard_normal((1, N, C)) / np.sqrt(C)).astype(np.float32)
    W_ = (0.02 * rng.standard_normal((V, C))).astype(np.float32)
    Y_ = rng.integers(0, V, size=(1, N)).astype(np.int32)
    Y_[rng.random((1, N)) < 0.05] = -1
    ref = O.flce_masked(O.round_to_bf16(X_[0]), O.round_to_bf16(W_), Y_[0])
    exact = O.flce_masked(X_[0], W_, Y_[0])
    loss, dX, dW = _run_flce(be, X_, W_, Y_, 2, ignore_mode=0, chunk=4096)
    assert abs(loss - float(ref["loss"])) <= TOL_BF16 * abs(loss)
    assert abs(loss - float(exact["loss"])) <= TOL_BF16 * abs(loss)
    assert_close(dX[0], ref["dX"], TOL_BF16, "dX")
    assert_close(dW, ref["dW"], TOL_BF16, "dW")
    for got, want in ((dX[0], exact["dX"]), (dW, exact["dW"])):
        rel_rms = np.sqrt(np.mean((got.astype(np.float64) - want) ** 2) / np.mean(want.astype(np.float64) ** 2))
        assert rel_rms <= TOL_BF16, rel_rms
    assert not dX[0][Y_[0] < 0].any()
    G.check_clean_status()


def test_flce_tensor_core_path_is_taken_and_deterministic():
    """3xTF32 panels: identical bits on a repeat, and different bits from the exact-fp32 FFMA
    panels (which proves the tensor-core kernel, not the FFMA one, produced them)."""
    ctx, alloc, be = G.env()
    rng = np.random.default_rng(1241)
    N, C, V = 1536, 256, 4096
    X_ = (rng.standard_normal((1, N, C)) / np.sqrt(C)).astype(np.float32)
    W_ = (0.02 * rng.standard_normal((V, C))).astype(np.float32)
    Y_ = rng.integers(0, V, size=(1, N)).astype(np.int32)
    a = _run_flce(be, X_, W_, Y_, 1, ignore_mode=0, chunk=2048)
    b = _run_flce(be, X_, W_, Y_, 1, ignore_mode=0, chunk=2048)
    c = _run_flce(be, X_, W_, Y_, 0, ignore_mode=0, chunk=2048)
    assert a[0] == b[0] and np.array_equal(a[1], b[1]) and np.array_equal(a[2], b[2])
    assert not np.array_equal(a[2], c[2])
    assert_close(a[2], c[2], TOL_BWD, "dW 3xtf32 vs fp32")
    G.check_clean_status()


@pytest.mark.parametrize("case", ["plain", "row_scaled"])
def test_rmsnorm_flce_golden(golden, case):
    ctx, alloc, be = G.env()
    g = golden("rmsnorm_flce")
    be.ce_precision, be.ce_vocab_chunk = 0, 64
    x = G.up(g[f"{case}.X"], grad=0)
    w = G.up(g[f"{case}.W"], grad=0)
    gam = G.up(g[f"{case}.G"], grad=0)
    y = G.up(g[f"{case}.Y"], requires_grad=False)
    inputs = [x, w, gam, y]
    if f"{case}.row_scale" in g:
        inputs.append(G.up(g[f"{case}.row_scale"], requires_grad=False))
    loss = G.empty((1,), grad=np.array([1.0], np.float32))
    n = G.node("FusedRMSNormLinearCrossEntropyOp", inputs, (loss,), eps=float(g[f"{case}.eps"]))
    G.run_forward(n)
    G.run_backward(n)
    got = float(G.down(loss)[0])
    assert abs(got - float(g[f"{case}.loss"][0])) <= TOL_FWD * abs(got)
    assert_close(G.down(x.grad), g[f"{case}.dX"], TOL_BWD, "dX")
    assert_close(G.down(w.grad), g[f"{case}.dW"], TOL_BWD, "dW")
    assert_close(G.down(gam.grad), g[f"{case}.dG"], TOL_BWD, "dG")
    be.ce_precision, be.ce_vocab_chunk = 1, 4096
    G.check_clean_status()
    G.free(*inputs, loss)


# ------------------------------------------------------------------------------ linear + bias + residual
@pytest.mark.parametrize("case", ["square", "wide", "mlp_down"])
def test_linear_add_golden(golden, case):
    """FusedLinearAddOp on the tcgen05 GEMM (3xTF32): forward with the output aliasing the residual
    input, backward accumulating on pre-loaded gradients, against the reference's CPU kernels."""
    ctx, alloc, be = G.env()
    g = golden("linear_add")
    x = G.up(g[f"{case}.x"], grad=g[f"{case}.pre_x"])
    act = G.up(g[f"{case}.act"], grad=g[f"{case}.pre_act"])
    w = G.up(g[f"{case}.w"], grad=g[f"{case}.pre_w"])
    b = G.up(g[f"{case}.b"], grad=g[f"{case}.pre_b"])
    out = G.empty(g[f"{case}.out"].shape, grad=g[f"{case}.dout"])
    n = G.node("FusedLinearAddOp", (x, act, w, b), (out,))
    G.run_forward(n)
    assert_close(G.down(out), g[f"{case}.out"], TOL_FWD, "out")
    G.run_backward(n)
    assert_close(G.down(x.grad), g[f"{case}.dx"], TOL_BWD, "dx")
    assert_close(G.down(act.grad), g[f"{case}.dact"], TOL_BWD, "dact")
    assert_close(G.down(w.grad), g[f"{case}.dw"], TOL_BWD, "dw")
    assert_close(G.down(b.grad), g[f"{case}.db"], TOL_BWD, "db")
    # in place: out aliases x (the reference aliases them when x dies at this node)
    x2 = G.up(g[f"{case}.x"])
    n2 = G.node("FusedLinearAddOp", (x2, act, w, b), (x2,))
    G.run_forward(n2)
    assert_close(G.down(x2), g[f"{case}.out"], TOL_FWD, "out in place")
    G.check_clean_status()
    G.free(x, act, w, b, out, x2)


@pytest.mark.parametrize("K", [1280, 5120])
def test_linear_add_projection_size_vs_oracle(K):
    """The attention-output projection (1280 -> 1280) and the MLP down-projection (5120 -> 1280) of the
    depth-20 model on 4096 token rows."""
    ctx, alloc, be = G.env()
    rng = np.random.default_rng(1242)
    N, C = 4096, 1280
    x_ = rng.standard_normal((N, C), dtype=np.float32)
    act_ = rng.standard_normal((N, K), dtype=np.float32)
    w_ = (rng.standard_normal((K, C)) / np.sqrt(K)).astype(np.float32)
    b_ = (0.1 * rng.standard_normal(C)).astype(np.float32)
    dout_ = rng.standard_normal((N, C), dtype=np.float32)
    x, act, w, b = G.up(x_, grad=0), G.up(act_, grad=0), G.up(w_, grad=0), G.up(b_, grad=0)
    out = G.empty((N, C), grad=dout_)
    n = G.node("FusedLinearAddOp", (x, act, w, b), (out,))
    G.run_forward(n)
    # The tensor core's fp32 adder truncates, so the error of an accumulation chain grows with its length
    # (2.5e-5 with one chain over K 1280).  The forward cuts K into equal pieces of at most 384 elements
    # whose results are added with round-to-nearest, which holds the fp32-forward bound of 1e-5.
    ref_out = O.linear_add_forward(x_, act_, w_, b_)
    got_out = G.down(out)
    print(f"linear_add forward K={K}: {mixed_rel_err(got_out, ref_out):.2e}")
    assert_close(got_out, ref_out, TOL_FWD, "out")
    G.run_backward(n)
    z = np.zeros
    dx, dact, dw, db = O.linear_add_backward(dout_, act_, w_, z((N, C), np.float32), z((N, K), np.float32),
                                             z((K, C), np.float32), z(C, np.float32))
    assert_close(G.down(x.grad), dx, TOL_BWD, "dx")
    assert_close(G.down(act.grad), dact, TOL_BWD, "dact")
    assert_close(G.down(w.grad), dw, TOL_BWD, "dw")
    assert_close(G.down(b.grad), db, TOL_BWD, "db")
    G.check_clean_status()
    G.free(x, act, w, b, out)


# ------------------------------------------------------------------------------ AdamW
def test_adamw_golden(golden):
    ctx, alloc, be = G.env()
    g = golden("adamw_bf16")
    lr, lr_t, b1, b2, eps, wd = (float(v) for v in g["hp"])
    p, gr, m, v = G.up(g["p"]), G.up(g["g"]), G.up(g["m"]), G.up(g["v"])
    be.adamw_step(p.storage, gr.storage, m.storage, v.storage, None, lr, lr_t, b1, b2, eps, wd, grad_scale=1.0)
    assert_close(G.down(p), g["p_out"], TOL_FWD, "p")
    assert_close(G.down(m), g["m_out"], TOL_FWD, "m")
    assert_close(G.down(v), g["v_out"], TOL_FWD, "v")
    G.free(p, gr, m, v)


# ------------------------------------------------------------------------------ bf16 gradient storage
def _bits_close(got_bits, ref_bits, what, max_off=0.01):
    """Stored bf16 words: equal, except that a sum formed in another order may land on the neighbouring
    bf16 value for a few elements (never further)."""
    got = O.bf16_bits_to_f32(got_bits).astype(np.float64)
    ref = O.bf16_bits_to_f32(ref_bits).astype(np.float64)
    off = got_bits != ref_bits
    assert off.mean() <= max_off, f"{what}: {off.mean():.3%} of the stored words differ"
    if off.any():
        assert np.max(np.abs(got[off] - ref[off]) / np.maximum(np.abs(ref[off]), 1e-30)) <= 2.0 ** -7, what


def test_grad_bf16_conversion_bit_exact(golden):
    """fp32 -> bf16 storage with and without accumulate, Inf / NaN / signed zero included, and back."""
    ctx, alloc, be = G.env()
    g = golden("grad_bf16")
    cases = [(g["src"], g["dst0"], g["conv_plain"], g["conv_acc"])]
    rng = np.random.default_rng(11)
    n = (1 << 20) + 5
    src = (rng.standard_normal(n) * 4).astype(np.float32)
    dst0 = O.f32_to_bf16_bits(rng.standard_normal(n).astype(np.float32))
    cases.append((src, dst0, O.f32_to_bf16_store(src, dst0, False), O.f32_to_bf16_store(src, dst0, True)))
    for src, dst0, plain, acc in cases:
        s = G.up(src, requires_grad=False)
        d = G.up(dst0, requires_grad=False)
        ctx.f32_to_bf16(s.storage.ptr.address, d.storage.ptr.address, src.size, accumulate=True)
        got = G.down_bits(d)
        # the sum of a NaN and a number is a NaN whose payload is the adder's choice: NaN-ness must agree
        nan = np.isnan(O.bf16_bits_to_f32(acc))
        assert np.array_equal(got[~nan], acc[~nan]) and np.all(np.isnan(O.bf16_bits_to_f32(got[nan])))
        ctx.f32_to_bf16(s.storage.ptr.address, d.storage.ptr.address, src.size, accumulate=False)
        assert np.array_equal(G.down_bits(d), plain)
        back = G.empty(src.shape, requires_grad=False)
        ctx.bf16_to_f32(d.storage.ptr.address, back.storage.ptr.address, src.size)
        assert np.array_equal(G.down(back).view(np.uint32), O.bf16_bits_to_f32(plain).view(np.uint32))
        G.free(s, d, back)
    G.check_clean_status()


def test_grad_bf16_edge_cases():
    """Empty input is a no-op, fewer elements than one packet take the scalar tail, a pointer that is not
    16-byte aligned is an error (never a fault); C not a multiple of 4 takes the scalar scatter-add."""
    import autograd_b200 as ag
    ctx, alloc, be = G.env()
    rng = np.random.default_rng(12)
    src = rng.standard_normal(13).astype(np.float32)
    old = O.f32_to_bf16_bits(rng.standard_normal(13).astype(np.float32))
    s, d = G.up(src, requires_grad=False), G.up(old, requires_grad=False)
    ctx.f32_to_bf16(s.storage.ptr.address, d.storage.ptr.address, 0)
    assert np.array_equal(G.down_bits(d), old)
    ctx.f32_to_bf16(s.storage.ptr.address, d.storage.ptr.address, 5, accumulate=True)
    want = old.copy()
    want[:5] = O.f32_to_bf16_store(src[:5], old[:5], True)
    assert np.array_equal(G.down_bits(d), want)
    ctx.f32_to_bf16(s.storage.ptr.address, d.storage.ptr.address, 13)
    assert np.array_equal(G.down_bits(d), O.f32_to_bf16_bits(src))
    with pytest.raises(ag.AgError):
        ctx.f32_to_bf16(s.storage.ptr.address + 4, d.storage.ptr.address, 4)
    with pytest.raises(ag.AgError):
        ctx.bf16_to_f32(d.storage.ptr.address + 2, s.storage.ptr.address, 4)
    G.free(s, d)
    # ragged width: 30 columns
    V, C, n = 40, 30, 200
    ids_ = rng.integers(0, V // 2, size=(1, n)).astype(np.int32)
    dout_ = rng.standard_normal((1, n, C), dtype=np.float32)
    t0 = O.f32_to_bf16_bits(rng.standard_normal((V, C)).astype(np.float32))
    ids, out = G.up(ids_, requires_grad=False), G.empty(dout_.shape, grad=dout_)
    table = G.empty((V, C))
    G.bf16_grad(table, t0)
    G.run_backward(G.node("GatherOp", (ids, table), (out,)))
    _bits_close(G.down_bits(table.grad), O.gather_backward_bf16(ids_, dout_, t0), "ragged dtable bits", max_off=0.02)
    G.check_clean_status()
    G.free(ids, out, table)


def test_gather_backward_bf16_golden(golden):
    ctx, alloc, be = G.env()
    g = golden("grad_bf16")
    ids = G.up(g["ids"], requires_grad=False)
    table = G.up(O.bf16_bits_to_f32(g["table0"]).reshape(g["table0"].shape))
    G.bf16_grad(table, g["table0"])
    out = G.empty(g["dout"].shape, grad=g["dout"])
    n = G.node("GatherOp", (ids, table), (out,))
    G.run_backward(n)
    got = G.down_bits(table.grad)
    _bits_close(got, g["table1"], "dtable bits")
    untouched = np.setdiff1d(np.arange(g["table0"].shape[0]), g["ids"].ravel())
    assert np.array_equal(got[untouched], g["table0"][untouched])
    G.check_clean_status()
    G.free(ids, table, out)


@pytest.mark.parametrize("V,C,n", [(32768, 1280, 32768), (5000, 100, 4099)])
def test_gather_backward_bf16_vs_oracle(V, C, n):
    """Zipf ids (hot rows spanning many groups), table gradient preloaded: stored words equal to the
    position-ordered oracle except for the odd neighbouring value; rows of a single short run and
    untouched rows exactly equal; run-to-run identical."""
    ctx, alloc, be = G.env()
    rng = np.random.default_rng(4321)
    ids_ = _zipf_ids(rng, V, n).reshape(1, n)
    dout_ = rng.standard_normal((1, n, C), dtype=np.float32)
    t0 = O.f32_to_bf16_bits((0.5 * rng.standard_normal((V, C))).astype(np.float32))
    ref = O.gather_backward_bf16(ids_, dout_, t0)
    ids = G.up(ids_, requires_grad=False)
    out = G.empty(dout_.shape, grad=dout_)
    runs = []
    for _ in range(2):
        table = G.empty((V, C))
        G.bf16_grad(table, t0)
        G.run_backward(G.node("GatherOp", (ids, table), (out,)))
        runs.append(G.down_bits(table.grad))
        G.free(table)
    assert np.array_equal(runs[0], runs[1])
    _bits_close(runs[0], ref, "dtable bits", max_off=0.002)
    counts = np.bincount(ids_.ravel(), minlength=V)
    assert np.array_equal(runs[0][counts == 0], t0[counts == 0])
    assert np.array_equal(runs[0][counts == 1], ref[counts == 1])
    G.check_clean_status()
    G.free(ids, out)


def test_adamw_bf16grad_golden(golden):
    ctx, alloc, be = G.env()
    g = golden("grad_bf16")
    lr, lr_t, b1, b2, eps, wd = (float(v) for v in g["hp"])
    p, gr, m, v = G.up(g["p"]), G.up(g["g_bits"], requires_grad=False), G.up(g["m"]), G.up(g["v"])
    be.adamw_step(p.storage, gr.storage, m.storage, v.storage, None, lr, lr_t, b1, b2, eps, wd,
                  grad_scale=float(g["grad_scale"]))
    assert_close(G.down(p), g["p_out"], TOL_FWD, "p")
    assert_close(G.down(m), g["m_out"], TOL_FWD, "m")
    assert_close(G.down(v), g["v_out"], TOL_FWD, "v")
    G.free(p, gr, m, v)


def test_parameter_grads_stored_as_bf16(golden):
    """LayerNorm dgamma/dbeta and the projection's dw/db land in bf16 gradient storage as
    bf16(stored + fp32 gradient): the kernels accumulate into zeroed fp32 staging, one rounding follows."""
    ctx, alloc, be = G.env()
    rng = np.random.default_rng(3)
    d, eps = _ln_case(golden("add_layernorm"), "c384")
    x = G.up(np.add(d["x"], d["r"]), grad=0)
    gamma, beta = G.up(d["gamma"]), G.up(d["beta"])
    pre_g = O.f32_to_bf16_bits(rng.standard_normal(d["gamma"].shape).astype(np.float32))
    pre_b = O.f32_to_bf16_bits(rng.standard_normal(d["beta"].shape).astype(np.float32))
    G.bf16_grad(gamma, pre_g)
    G.bf16_grad(beta, pre_b)
    y = G.empty(d["x"].shape, grad=d["dy"])
    ln = G.node("LayerNormOp", (x, gamma, beta), (y,), eps=eps, normalized_dim=-1)
    G.run_forward(ln)
    G.run_backward(ln)
    _bits_close(G.down_bits(gamma.grad), O.f32_to_bf16_store(d["dgamma"], pre_g, True), "dgamma bits")
    _bits_close(G.down_bits(beta.grad), O.f32_to_bf16_store(d["dbeta"], pre_b, True), "dbeta bits")
    G.free(x, gamma, beta, y)

    g = golden("linear_add")
    case = "wide"
    xw = G.up(g[f"{case}.x"], grad=g[f"{case}.pre_x"])
    act = G.up(g[f"{case}.act"], grad=g[f"{case}.pre_act"])
    w, b = G.up(g[f"{case}.w"]), G.up(g[f"{case}.b"])
    pre_w, pre_bb = O.f32_to_bf16_bits(g[f"{case}.pre_w"]), O.f32_to_bf16_bits(g[f"{case}.pre_b"])
    G.bf16_grad(w, pre_w)
    G.bf16_grad(b, pre_bb)
    out = G.empty(g[f"{case}.out"].shape, grad=g[f"{case}.dout"])
    n = G.node("FusedLinearAddOp", (xw, act, w, b), (out,))
    G.run_backward(n)
    # the golden dw/db include the fp32 preload; take it out again, then add onto the bf16 preload
    dw_only = np.subtract(g[f"{case}.dw"], g[f"{case}.pre_w"])
    db_only = np.subtract(g[f"{case}.db"], g[f"{case}.pre_b"])
    assert_close(G.down(w.grad), np.add(O.bf16_bits_to_f32(pre_w).reshape(dw_only.shape), dw_only), TOL_BF16, "dw")
    assert_close(G.down(b.grad), np.add(O.bf16_bits_to_f32(pre_bb).reshape(db_only.shape), db_only), TOL_BF16, "db")
    assert_close(G.down(xw.grad), g[f"{case}.dx"], TOL_BWD, "dx")
    G.check_clean_status()
    G.free(xw, act, w, b, out)


def test_errors_are_exceptions_not_aborts():
    import autograd_b200 as ag
    ctx, alloc, be = G.env()
    x = G.up(np.zeros((4, 8), np.float32))
    with pytest.raises(ag.AgError):  # workspace too small
        ctx.layernorm_backward(x.storage.ptr.address, x.storage.ptr.address, x.storage.ptr.address, 0,
                               x.storage.ptr.address, x.storage.ptr.address, x.storage.ptr.address,
                               x.storage.ptr.address, 16, 4, 8, 1e-5)
    with pytest.raises(ag.AgError):  # null input
        ctx.gelu_forward(0, x.storage.ptr.address, 32)
    ctx.synchronize()
    G.free(x)


def test_fused_layer_step_matches_oracle():
    """The kernel sequence that bench.py times (gather, add+LayerNorm, RoPE, GELU, fused linear+CE,
    their backward passes with the fused residual-gradient add, scatter-add into the tied table), at a
    small size, replayed with the oracle on the same buffers: loss, every dgamma/dbeta, the tied
    table gradient, the residual-stream gradient and the in-place rotated q/k must agree."""
    from autograd_b200.step import StepConfig
    _step_vs_oracle(StepConfig(n_layer=2, n_embd=128, n_head=1, head_dim=128, seq_len=64, batch=3, vocab=640))


def test_fused_layer_step_bench_width_matches_oracle():
    """The same replay at the width bench.py runs: n_embd 1280, 10 heads x 128, seq 2048, vocab 32768,
    MLP 5120, two layers, 10 sequences = 20480 token rows (more than one 18944-row tile of the CE head,
    so both row tiles occur; every norm / RoPE / GELU kernel takes its persistent multi-row path)."""
    from autograd_b200.step import StepConfig
    _step_vs_oracle(StepConfig(n_layer=2, n_embd=1280, n_head=10, head_dim=128, seq_len=2048, batch=10, vocab=32768))


def _step_vs_oracle(cfg):
    from autograd_b200.step import FusedLayerStep
    ctx, alloc, be = G.env()
    st = FusedLayerStep(ctx, alloc, be, cfg, seed=77)
    Nn, C, V, L, I = st.N, st.C, st.V, st.L, st.I
    B, T, H, D = cfg.batch, cfg.seq_len, cfg.n_head, cfg.head_dim
    rng = np.random.default_rng(5)
    ids = rng.integers(0, V, size=Nn).astype(np.int32)
    ids[:40] = 7                                   # a hot row for the scatter-add
    tg = rng.integers(0, V, size=Nn).astype(np.int32)
    tg[rng.random(Nn) < 0.1] = -1
    ctx.copy_from_host(st.ids, ids)
    ctx.copy_from_host(st.targets, tg)
    f = np.float32
    get = lambda addr, shape: ctx.copy_to_host(addr, shape, f).copy()
    table = get(st.table, (V, C))
    gam, bet = get(st.gamma, (st.n_norms, C)), get(st.beta, (st.n_norms, C))
    branch = [get(a, (Nn, C)) for a in st.branch]
    u = [get(a, (Nn, I)) for a in st.u]
    dy = [get(st.dy[0], (Nn, C)), get(st.dy[1], (Nn, C))]
    dg = get(st.dg, (Nn, I))
    q0, k0 = get(st.q, (B, T, H, D)), get(st.k, (B, T, H, D))
    cos, sin = get(st.cos, (T, D // 2)), get(st.sin, (T, D // 2))

    st.step()
    ctx.synchronize()
    G.check_clean_status()

    # ---- the same sequence with the oracle
    x = O.gather_forward(ids.reshape(B, T), table).reshape(Nn, C)
    q, k = q0.copy(), k0.copy()
    h1s, h2s = [], []
    for l in range(L):
        h1, _, _, _ = O.add_layernorm_forward(x, branch[(2 * l) % 4], gam[2 * l], bet[2 * l], cfg.eps)
        O.rope_apply(q, cos, sin, -1); O.rope_apply(k, cos, sin, -1)
        h2, _, _, _ = O.add_layernorm_forward(h1, branch[(2 * l + 1) % 4], gam[2 * l + 1], bet[2 * l + 1], cfg.eps)
        h1s.append(h1); h2s.append(h2)
        x = h2
    hf, yf, _, _ = O.add_layernorm_forward(x, branch[0], gam[2 * L], bet[2 * L], cfg.eps)
    res = O.flce_masked(yf, table, tg)
    zc = np.zeros(C, f)
    dgam, dbet = np.zeros((st.n_norms, C), f), np.zeros((st.n_norms, C), f)
    dh, dgam[2 * L], dbet[2 * L] = O.layernorm_backward(hf, gam[2 * L], res["dX"], cfg.eps, np.zeros_like(hf), zc, zc)
    du_last = None
    for l in reversed(range(L)):
        du_last = O.gelu_backward(u[l], dg, np.zeros_like(dg))
        dh, dgam[2 * l + 1], dbet[2 * l + 1] = O.layernorm_backward(h2s[l], gam[2 * l + 1], dy[1], cfg.eps, dh, zc, zc)
        O.rope_apply(q, cos, sin, +1); O.rope_apply(k, cos, sin, +1)
        # dy[0] was overwritten by the head's dX before the layer loop read it
        dyl = res["dX"] if l % 2 == 0 else dy[1]
        dh, dgam[2 * l], dbet[2 * l] = O.layernorm_backward(h1s[l], gam[2 * l], dyl, cfg.eps, dh, zc, zc)
    dtable = O.gather_backward(ids.reshape(B, T), dh.reshape(B, T, C), res["dW"])

    loss = st.read_loss()
    assert abs(loss - float(res["loss"])) <= TOL_FWD * abs(loss)
    small = get(st.small_bucket, (st.n_norms, 2, C))
    assert_close(small[:, 0], dgam, TOL_BWD, "dgamma of every norm")
    assert_close(small[:, 1], dbet, TOL_BWD, "dbeta of every norm")
    assert_close(get(st.dh, (Nn, C)), dh, TOL_BWD, "residual-stream gradient")
    assert_close(get(st.dtable, (V, C)), dtable, TOL_BWD, "tied table gradient")
    assert_close(get(st.du, (Nn, I)), du_last, TOL_BWD, "GELU input gradient")
    # forward rotation followed by the transposed rotation L times: back to the start within rounding
    assert_close(get(st.q, (B, T, H, D)), q, TOL_FWD * 4, "q after the step")
    assert_close(get(st.h_final, (Nn, C)), hf, TOL_FWD, "final residual stream")
    st.close()


# ------------------------------------------------------------------------------ shapes of the benchmark step
def test_rope_step_shape_vs_oracle():
    """RoPE as the benchmark step runs it: 16 sequences x 2048 positions, q and k with 10 heads x 128,
    theta 1e5, the nanochat sign forward and its transpose backward (flat work distribution, several
    packet pairs per thread)."""
    ctx, alloc, be = G.env()
    B, T, H, D = 16, 2048, 10, 128
    rng = np.random.default_rng(1243)
    q_ = rng.standard_normal((B, T, H, D), dtype=np.float32)
    k_ = rng.standard_normal((B, T, H, D), dtype=np.float32)
    cos_, sin_ = O.rope_tables(T, D, 1e5)
    q, k, cos, sin = G.up(q_), G.up(k_), G.up(cos_), G.up(sin_)
    be.rope_qk(q, k, cos, sin, sin_sign=-1)
    q1, k1 = O.rope_apply(q_, cos_, sin_, -1), O.rope_apply(k_, cos_, sin_, -1)
    assert_close(G.down(q), q1, TOL_FWD, "q forward")
    assert_close(G.down(k), k1, TOL_FWD, "k forward")
    be.rope_qk(q, k, cos, sin, sin_sign=+1)
    assert_close(G.down(q), O.rope_apply(q1, cos_, sin_, +1), TOL_FWD, "q backward")
    assert_close(G.down(k), O.rope_apply(k1, cos_, sin_, +1), TOL_FWD, "k backward")
    G.check_clean_status()
    G.free(q, k, cos, sin)


def test_rmsnorm_flce_qwen_shape_tensor_core():
    """FusedRMSNormLinearCrossEntropyOp (backend.py:716-886) on the tensor-core path (3xTF32) at the
    Qwen shape - hidden 1536, vocabulary 151936 (38 panels of 4096), eps 1e-6 - with row_scale
    (rl_autograd.py:518-524), targets of -1 and targets >= V (both ignored, backend.py:768;
    debug/check_qwen_kernel.py:872-874), on 2048 token rows."""
    ctx, alloc, be = G.env()
    rng = np.random.default_rng(1244)
    B, T, C, V, eps = 1, 2048, 1536, 151936, 1e-6
    N = B * T
    X_ = rng.standard_normal((B, T, C), dtype=np.float32)
    W_ = (0.02 * rng.standard_normal((V, C), dtype=np.float32)).astype(np.float32)
    G_ = (1 + 0.02 * rng.standard_normal(C)).astype(np.float32)
    Y_ = rng.integers(0, V, size=(B, T)).astype(np.int32)
    Y_[0, ::19] = -1
    Y_[0, 5::23] = V
    Y_[0, 7] = V + 1000
    rs_ = (rng.random((B, T)).astype(np.float32) * (2.0 / N)).astype(np.float32)
    assert be.ce_precision == 1 and be.ce_vocab_chunk == 4096
    x, w, gam = G.up(X_, grad=0), G.up(W_, grad=0), G.up(G_, grad=0)
    y, rs = G.up(Y_, requires_grad=False), G.up(rs_, requires_grad=False)
    loss = G.empty((1,), grad=np.array([1.0], np.float32))
    n = G.node("FusedRMSNormLinearCrossEntropyOp", [x, w, gam, y, rs], (loss,), eps=eps)
    G.run_forward(n)
    G.run_backward(n)
    ref = O.rmsnorm_flce(X_[0], W_, G_, Y_[0], eps, row_scale=rs_[0])
    got = float(G.down(loss)[0])
    assert abs(got - float(ref["loss"])) <= TOL_FWD * abs(got), (got, float(ref["loss"]))
    dX = G.down(x.grad)[0]
    assert_close(dX, ref["dX"], TOL_BWD, "dX")
    assert_close(G.down(w.grad), ref["dW"], TOL_BWD, "dW")
    assert_close(G.down(gam.grad), ref["dG"], TOL_BWD, "dG")
    ignored = (Y_[0] < 0) | (Y_[0] >= V)
    assert ignored.sum() > 150 and not dX[ignored].any()          # ignored rows: exactly zero gradient
    # out-of-range targets are reported through the status word and are otherwise treated as ignored
    ctx.synchronize()
    flags = ctx.status()
    assert flags in (0, 1), flags
    G.free(x, w, gam, y, rs, loss)


def test_staging_wait_that_gives_up_takes_the_plain_load_path():
    """A bounded wait run to expiry, safely: with the test hook the next norm kernel treats its wait for
    the bulk-copied gamma/beta as expired at once.  The kernel must set AG_STATUS_STAGE_FALLBACK, let the
    copy land, fill the vectors with plain loads, return by itself and still produce correct results."""
    import autograd_b200 as ag
    ctx, alloc, be = G.env()
    N, C, eps = 3000, 1280, 1e-5
    x_, r_, g_, b_, dy_ = _cfg1_inputs(N, C, seed=1245)
    x, r, gamma, beta = G.up(x_), G.up(r_), G.up(g_, grad=0), G.up(b_, grad=0)
    h, y = G.empty((N, C), grad=0), G.empty((N, C), grad=dy_)
    assert ctx.status() == 0
    ctx.debug_expire_staging()
    be.fused_add_layernorm_forward(x, r, gamma, beta, h, y, eps)
    ctx.synchronize()
    assert ctx.status() == ag.AG_STATUS_STAGE_FALLBACK
    h_ref, y_ref, _, _ = O.add_layernorm_forward(x_, r_, g_, b_, eps)
    assert_close(G.down(y), y_ref, TOL_FWD, "y after the fallback")
    ctx.debug_expire_staging()
    ln = G.node("LayerNormOp", (h, gamma, beta), (y,), eps=eps, normalized_dim=-1)
    G.run_backward(ln)
    ctx.synchronize()
    assert ctx.status() == ag.AG_STATUS_STAGE_FALLBACK
    dh_ref, dg_ref, db_ref = O.layernorm_backward(h_ref, g_, dy_, eps, np.zeros_like(x_), np.zeros_like(g_), np.zeros_like(b_))
    assert_close(G.down(h.grad), dh_ref, TOL_BWD, "dh after the fallback")
    assert_close(G.down(gamma.grad), dg_ref, TOL_BWD, "dgamma after the fallback")
    # the hook is one-shot: the next launch stages normally
    be.fused_add_layernorm_forward(x, r, gamma, beta, h, y, eps)
    ctx.synchronize()
    assert ctx.status() == 0
    G.free(x, r, gamma, beta, h, y)


@pytest.mark.parametrize("design", ["registers", "ring", "pair"])
def test_norm_kernels_with_one_design_forced(design, monkeypatch):
    """By default the norm kernels choose per shape between a row per warp in registers, the shared-memory
    row ring, and (backward) a row per pair of warps; AG_B200_NORM_RING / AG_B200_NORM_PAIR (read when a
    context is created) force one of them wherever the shape fits.  Every design must agree with the oracle
    on the same shapes: fp32 and bf16 storage, with and without gamma, a single row, fewer rows than warps,
    many rows per warp, the residual-gradient add."""
    import autograd_b200 as ag
    from autograd_b200 import hostgraph as hg
    monkeypatch.setenv("AG_B200_NORM_RING", "1" if design == "ring" else "0")
    monkeypatch.setenv("AG_B200_NORM_PAIR", "1" if design == "pair" else "0")
    ctx, alloc, be = ag.create(0)
    try:
        rng = np.random.default_rng(1246)

        def dev(a, dtype=np.float32):
            t = hg.HostTensor(a.shape, dtype, requires_grad=False)
            t.storage = alloc.alloc(t.shape, dtype)
            be.copy_from_host(t, a)
            return t

        for N, C, bf, with_gamma in ((1, 384, False, True), (5, 1280, False, True), (4097, 1536, False, True),
                                     (3001, 256, True, True), (7, 1536, True, False), (2500, 640, False, False)):
            st = np.uint16 if bf else np.float32
            tol_f, tol_b = (TOL_BF16, TOL_BF16) if bf else (TOL_FWD, TOL_BWD)
            prep = _bf16 if bf else (lambda a: a)
            x_, dz_, res_ = (prep(rng.standard_normal((N, C), dtype=np.float32)) for _ in range(3))
            g_ = (1 + 0.02 * rng.standard_normal(C)).astype(np.float32) if with_gamma else None
            x, dz, dx = dev(x_, st), dev(dz_, st), dev(res_, st)
            gamma = dev(g_) if with_gamma else None
            dgam = dev(np.zeros(C, np.float32)) if with_gamma else None
            y, inv = dev(np.zeros((N, C), np.float32), st), dev(np.zeros(N, np.float32))
            be.rmsnorm_forward(x, gamma, y, 1e-6, inv)
            z_ref, inv_ref = O.rmsnorm_forward(x_, g_, 1e-6)
            assert_close(be.copy_to_host(inv), inv_ref, TOL_FWD, f"inv_rms N={N} C={C} bf16={bf}")
            assert_close(be.copy_to_host(y), z_ref, tol_f, f"rmsnorm y N={N} C={C} bf16={bf}")
            be.rmsnorm_backward(dz, x, gamma, 1e-6, dx, dgam, dres=dx)
            dx_ref, dg_ref = O.rmsnorm_backward(x_, g_, dz_, 1e-6, res_, np.zeros(C, np.float32) if with_gamma else None)
            assert_close(be.copy_to_host(dx), dx_ref, tol_b, f"rmsnorm dx N={N} C={C} bf16={bf}")
            if with_gamma:
                assert_close(be.copy_to_host(dgam), dg_ref, tol_b, f"rmsnorm dgamma N={N} C={C} bf16={bf}")
            if not bf and with_gamma:      # LayerNorm with the fused residual add, same shape
                r_, b_ = rng.standard_normal((N, C), dtype=np.float32), (0.02 * rng.standard_normal(C)).astype(np.float32)
                r, beta, h = dev(r_), dev(b_), dev(np.zeros((N, C), np.float32))
                be.fused_add_layernorm_forward(x, r, gamma, beta, h, y, 1e-5)
                h_ref, y_ref, _, _ = O.add_layernorm_forward(x_, r_, g_, b_, 1e-5)
                assert np.array_equal(be.copy_to_host(h), h_ref)
                assert_close(be.copy_to_host(y), y_ref, TOL_FWD, f"layernorm y N={N} C={C}")
                for t in (r, beta, h):
                    alloc.free(t.storage)
            ctx.synchronize()
            for t in (x, dz, dx, gamma, dgam, y, inv):
                if t is not None:
                    alloc.free(t.storage)
        assert ctx.status() == 0
    finally:
        ctx.synchronize()
        alloc.free()
        ctx.close()
