"""The numpy oracle against the vectors produced by the reference's CPU backend
(tests/golden/make_golden.py).  CPU only."""
import numpy as np
import pytest

from conftest import assert_close
from oracle import fused_layers as O

TIGHT = 2e-6  # same numpy statements on the same machine class; allows BLAS/summation drift


def test_add_layernorm(golden):
    g = golden("add_layernorm")
    for c in g.cases():
        x, r, gamma, beta, dy = (g[f"{c}.{k}"] for k in ("x", "r", "gamma", "beta", "dy"))
        eps = float(g[f"{c}.eps"])
        h, y, mean, rstd = O.add_layernorm_forward(x, r, gamma, beta, eps)
        assert_close(y, g[f"{c}.y"], TIGHT, f"{c}.y")
        z = np.zeros_like(x)
        dh, dgamma, dbeta = O.layernorm_backward(h, gamma, dy, eps, z, np.zeros_like(gamma), np.zeros_like(beta))
        dx, dr = O.add_backward(dh, z, z)
        assert_close(dx, g[f"{c}.dx"], TIGHT, f"{c}.dx")
        assert_close(dr, g[f"{c}.dr"], TIGHT, f"{c}.dr")
        assert np.array_equal(g[f"{c}.dx"], g[f"{c}.dr"])
        assert_close(dgamma, g[f"{c}.dgamma"], 1e-5, f"{c}.dgamma")
        assert_close(dbeta, g[f"{c}.dbeta"], 1e-5, f"{c}.dbeta")
        dh2, _, _ = O.layernorm_backward(h, gamma, dy, eps, g[f"{c}.resid"], np.zeros_like(gamma), np.zeros_like(beta))
        assert_close(dh2, g[f"{c}.dh_with_resid"], TIGHT, f"{c}.dh_with_resid")


def test_gelu(golden):
    g = golden("gelu")
    for c in g.cases():
        x, dy, pre = g[f"{c}.x"], g[f"{c}.dy"], g[f"{c}.pre"]
        assert_close(O.gelu_forward(x), g[f"{c}.y"], TIGHT, f"{c}.y")
        assert_close(O.gelu_backward(x, dy, pre), g[f"{c}.dx"], TIGHT, f"{c}.dx")


def test_gather(golden):
    g = golden("gather")
    for c in g.cases():
        ids, table, dout = g[f"{c}.ids"], g[f"{c}.table"], g[f"{c}.dout"]
        assert np.array_equal(O.gather_forward(ids, table), g[f"{c}.out"])
        got = O.gather_backward(ids, dout, np.zeros_like(table))
        assert np.array_equal(got, g[f"{c}.dtable"]), c


def test_flce_reference_semantics(golden):
    g = golden("flce")
    for c in g.cases():
        X, W, Y = g[f"{c}.X"], g[f"{c}.W"], g[f"{c}.Y"]
        X2, Y1 = X.reshape(-1, X.shape[-1]), Y.reshape(-1)
        loss = O.flce_forward_reference(X2, W, Y1)
        assert abs(float(loss) - float(g[f"{c}.loss"][0])) <= 2e-6 * abs(float(loss))
        dX, dW = O.flce_backward_reference(X2, W, Y1, 1.0, np.zeros_like(X2), np.zeros_like(W))
        assert_close(dX, g[f"{c}.dX"].reshape(dX.shape), 1e-5, f"{c}.dX")
        assert_close(dW, g[f"{c}.dW"], 1e-5, f"{c}.dW")


def test_flce_masked_matches_reference_on_valid_rows(golden):
    """Masked semantics == the reference op run on the valid rows only, rescaled by
    N_valid/N (ignored rows: zero loss, zero dX, no dW contribution)."""
    g = golden("flce")
    for c in g.cases():
        X, W, Y = g[f"{c}.X"], g[f"{c}.W"], g[f"{c}.Y"]
        X2, Y1 = X.reshape(-1, X.shape[-1]), Y.reshape(-1)
        N = X2.shape[0]
        keep = g[f"{c}.valid_rows"]
        r = O.flce_masked(X2, W, Y1)
        f = len(keep) / N
        assert r["n_valid"] == len(keep)
        assert abs(float(r["loss"]) - f * float(g[f"{c}.loss_valid_only"][0])) <= 1e-5 * abs(float(r["loss"]))
        exp_dX = np.zeros_like(X2)
        exp_dX[keep] = f * g[f"{c}.dX_valid_only"].reshape(len(keep), -1)
        assert_close(r["dX"], exp_dX, 1e-5, f"{c}.dX masked")
        assert_close(r["dW"], f * g[f"{c}.dW_valid_only"], 1e-5, f"{c}.dW masked")
        rv = O.flce_masked(X2, W, Y1, reduction="mean_valid")
        assert abs(float(rv["loss"]) - float(g[f"{c}.loss_valid_only"][0])) <= 1e-5 * abs(float(rv["loss"]))


def test_rmsnorm_swiglu(golden):
    g = golden("rmsnorm_swiglu")
    for c in g.cases():
        x, eps = g[f"{c}.x"], float(g[f"{c}.eps"])
        gamma = g[f"{c}.gamma"] if f"{c}.gamma" in g else None
        z, inv = O.rmsnorm_forward(x, gamma, eps)
        assert_close(inv, g[f"{c}.inv_rms"], TIGHT, f"{c}.inv_rms")
        assert_close(z, g[f"{c}.x_norm"], TIGHT, f"{c}.x_norm")
        gu = g[f"{c}.gu"]
        assert_close(O.swiglu_forward(gu), g[f"{c}.hidden"], TIGHT, f"{c}.hidden")
        dgu = O.swiglu_backward(gu, g[f"{c}.dhidden"])
        assert_close(dgu, g[f"{c}.dgu"], TIGHT, f"{c}.dgu")
        dg0 = None if gamma is None else np.zeros_like(gamma)
        dx, dgamma = O.rmsnorm_backward(x, gamma, g[f"{c}.dz"], eps, g[f"{c}.resid"], dg0)
        assert_close(dx, g[f"{c}.dx_with_resid"], 1e-5, f"{c}.dx")
        if gamma is not None:
            assert_close(dgamma, g[f"{c}.dgamma"], 1e-5, f"{c}.dgamma")


def test_rope(golden):
    g = golden("rope")
    for c in g.cases():
        q, k, cos, sin = g[f"{c}.q"], g[f"{c}.k"], g[f"{c}.cos"], g[f"{c}.sin"]
        T, D = q.shape[1], q.shape[3]
        c2, s2 = O.rope_tables(T, D, float(g[f"{c}.theta"]))
        assert np.array_equal(c2, cos) and np.array_equal(s2, sin)
        for sign, tag in ((+1, "pos"), (-1, "neg")):
            assert np.array_equal(O.rope_apply(q, cos, sin, sign), g[f"{c}.q_{tag}"])
            assert np.array_equal(O.rope_apply(k, cos, sin, sign), g[f"{c}.k_{tag}"])
        # forward then backward is the identity up to rounding (rotation)
        back = O.rope_apply(O.rope_apply(q, cos, sin, +1), cos, sin, -1)
        assert_close(back, q, 1e-6, f"{c}.roundtrip")


def test_rmsnorm_flce(golden):
    g = golden("rmsnorm_flce")
    for c in g.cases():
        X, W, G, Y = g[f"{c}.X"][0], g[f"{c}.W"], g[f"{c}.G"], g[f"{c}.Y"][0]
        rs = g[f"{c}.row_scale"][0] if f"{c}.row_scale" in g else None
        r = O.rmsnorm_flce(X, W, G, Y, float(g[f"{c}.eps"]), row_scale=rs)
        assert abs(float(r["loss"]) - float(g[f"{c}.loss"][0])) <= 1e-5 * abs(float(r["loss"]))
        assert_close(r["dX"], g[f"{c}.dX"][0], 1e-5, f"{c}.dX")
        assert_close(r["dW"], g[f"{c}.dW"], 1e-5, f"{c}.dW")
        assert_close(r["dG"], g[f"{c}.dG"], 1e-5, f"{c}.dG")


def test_linear_add(golden):
    g = golden("linear_add")
    for c in g.cases():
        x, act, w, b, dout = (g[f"{c}.{k}"] for k in ("x", "act", "w", "b", "dout"))
        n, k = act.shape[1], act.shape[2]
        out = O.linear_add_forward(x[0], act[0], w, b)
        assert_close(out, g[f"{c}.out"][0], 1e-5, f"{c}.out")
        dx, dact, dw, db = O.linear_add_backward(dout[0], act[0], w, g[f"{c}.pre_x"][0], g[f"{c}.pre_act"][0],
                                                 g[f"{c}.pre_w"], g[f"{c}.pre_b"])
        assert_close(dx, g[f"{c}.dx"][0], TIGHT, f"{c}.dx")
        assert_close(dact, g[f"{c}.dact"][0], 1e-5, f"{c}.dact")
        assert_close(dw, g[f"{c}.dw"], 1e-5, f"{c}.dw")
        assert_close(db, g[f"{c}.db"], 1e-5, f"{c}.db")


def test_adamw_and_bf16(golden):
    g = golden("adamw_bf16")
    lr, lr_t, b1, b2, eps, wd = (float(v) for v in g["hp"])
    p, m, v = O.adamw_step(g["p"], g["g"], g["m"], g["v"], lr, lr_t, b1, b2, eps, wd)
    assert_close(p, g["p_out"], TIGHT, "p")
    assert_close(m, g["m_out"], TIGHT, "m")
    assert_close(v, g["v_out"], TIGHT, "v")
    assert np.array_equal(O.f32_to_bf16_bits(g["bf16_in"]), g["bf16_bits"])


def test_grad_bf16_storage(golden):
    """Gradients kept as bf16 bit patterns: conversion with and without accumulate, the gather
    backward that rounds once per table row, AdamW on bf16 gradients."""
    g = golden("grad_bf16")
    assert np.array_equal(O.f32_to_bf16_store(g["src"], g["dst0"], False), g["conv_plain"])
    assert np.array_equal(O.f32_to_bf16_store(g["src"], g["dst0"], True), g["conv_acc"])
    assert np.array_equal(O.gather_backward_bf16(g["ids"], g["dout"], g["table0"]), g["table1"])
    lr, lr_t, b1, b2, eps, wd = (float(v) for v in g["hp"])
    p, m, v = O.adamw_step_bf16grad(g["p"], g["g_bits"], g["m"], g["v"], lr, lr_t, b1, b2, eps, wd,
                                    grad_scale=float(g["grad_scale"]))
    assert_close(p, g["p_out"], TIGHT, "p")
    assert_close(m, g["m_out"], TIGHT, "m")
    assert_close(v, g["v_out"], TIGHT, "v")
