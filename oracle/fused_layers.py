"""CPU oracle for the fused layer kernels of tuzbing/autograd.

TEST INFRASTRUCTURE ONLY.  This module restates, in plain numpy, the arithmetic of the
reference's CPU backend for the fused-layer path.  It exists to check the CUDA kernels and
to time a CPU baseline; nothing in the shipped package imports it.

Parity status: PINNED.  Every function here is compared with the reference's own
`cpu_*` kernels (run through the reference's `Runtime(device="cpu")` or called directly on
namespace tensors) by `tests/golden/make_golden.py`; the resulting vectors are committed
under `tests/golden/` and `tests/test_oracle_golden.py` re-checks this module against them.

All functions are functional (return new arrays) except where an `*_inplace` name says
otherwise; gradients follow the reference's accumulate-into-grad contract by taking the
incoming gradient buffer and returning the updated one.

Reference citations are `file:line` inside the reference project.
"""
from __future__ import annotations

import numpy as np

# backend.py:18-20
GELU_C = 0.7978845608028654
GELU_A = 0.044715
GELU_A3 = 0.134145

F32 = np.float32


# --------------------------------------------------------------------------------------
# bf16 storage helpers (utils.py:20-27 `bf16_bits`, backend.py:5090-5111): bf16 values are
# kept as uint16 with round-to-nearest-even, NaN kept quiet.
# --------------------------------------------------------------------------------------
def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    bits = np.ascontiguousarray(a, dtype=F32).view(np.uint32)
    is_special = (bits & np.uint32(0x7F800000)) == np.uint32(0x7F800000)
    has_mant = (bits & np.uint32(0x007FFFFF)) != 0
    bias = np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))
    rounded = ((bits.astype(np.uint64) + bias.astype(np.uint64)) >> np.uint64(16)).astype(np.uint32)
    special = bits >> np.uint32(16)
    special = np.where(has_mant, special | np.uint32(0x0040), special)
    out = np.where(is_special, special, rounded) & np.uint32(0xFFFF)
    return out.astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(F32)


def round_to_bf16(a: np.ndarray) -> np.ndarray:
    """fp32 array whose values are exactly representable in bf16 (RNE)."""
    return bf16_bits_to_f32(f32_to_bf16_bits(a))


# --------------------------------------------------------------------------------------
# a1  residual add            backend.py:74-105 (cpu_add_forward / cpu_add_backward)
# --------------------------------------------------------------------------------------
def add_forward(x, r):
    return np.add(x, r)


def add_backward(g, x_grad, r_grad):
    """Same-shape case of cpu_add_backward: both input grads accumulate the upstream g."""
    return np.add(x_grad, g), np.add(r_grad, g)


# --------------------------------------------------------------------------------------
# a2  LayerNorm forward        backend.py:416-433
# --------------------------------------------------------------------------------------
def layernorm_stats(x, eps):
    """mean and rstd exactly as backend.py:423-429 computes them (two-pass variance)."""
    mean = np.mean(x, axis=-1, keepdims=True)
    cen = np.subtract(x, mean)
    var = np.mean(np.multiply(cen, cen), axis=-1, keepdims=True)
    rstd = np.reciprocal(np.sqrt(np.add(var, F32(eps))))
    return mean.astype(F32), rstd.astype(F32)


def layernorm_forward(x, gamma, beta, eps):
    mean, rstd = layernorm_stats(x, eps)
    xhat = np.multiply(np.subtract(x, mean), rstd)
    y = np.add(np.multiply(xhat, gamma), beta)
    return y, mean[..., 0], rstd[..., 0]


def add_layernorm_forward(x, r, gamma, beta, eps):
    """AddOp followed by LayerNormOp, the two graph nodes the fused CUDA kernel replaces."""
    h = add_forward(x, r)
    y, mean, rstd = layernorm_forward(h, gamma, beta, eps)
    return h, y, mean, rstd


# --------------------------------------------------------------------------------------
# a3  LayerNorm backward       backend.py:435-487
# --------------------------------------------------------------------------------------
def layernorm_backward(x, gamma, dy, eps, x_grad, gamma_grad, beta_grad):
    """Returns updated (x_grad, gamma_grad, beta_grad); all three accumulate."""
    mean, rstd = layernorm_stats(x, eps)
    xhat = np.multiply(np.subtract(x, mean), rstd)
    lead = tuple(range(x.ndim - 1))
    # backend.py:458-467: column sums over all leading axes (sequential fp32 np.sum)
    gamma_grad = np.add(gamma_grad, np.sum(np.multiply(dy, xhat), axis=lead))
    beta_grad = np.add(beta_grad, np.sum(dy, axis=lead))
    # backend.py:469-487
    dyg = np.multiply(dy, gamma)
    xg = np.add(x_grad, np.multiply(dyg, rstd))
    m1 = np.multiply(np.mean(dyg, axis=-1, keepdims=True), rstd)
    xg = np.subtract(xg, m1)
    m2 = np.multiply(np.mean(np.multiply(dyg, xhat), axis=-1, keepdims=True), rstd)
    xg = np.subtract(xg, np.multiply(xhat, m2))
    return xg, gamma_grad, beta_grad


# --------------------------------------------------------------------------------------
# a4  RMSNorm (stage inside the fused ops)
#     forward  backend.py:1097-1108 ; backward backend.py:1228-1251
#     same math: backend.py:741-749, :862-886 and debug/check_qwen_kernel.py:195-211
# --------------------------------------------------------------------------------------
def rmsnorm_inv(x, eps):
    ms = np.mean(np.multiply(x, x), axis=-1, keepdims=True)
    return np.reciprocal(np.sqrt(np.add(ms, F32(eps)))).astype(F32)


def rmsnorm_forward(x, gamma, eps):
    inv = rmsnorm_inv(x, eps)
    z = np.multiply(x, inv)
    if gamma is not None:
        z = np.multiply(z, gamma.reshape(1, -1))
    return z, inv[..., 0]


def rmsnorm_backward(x, gamma, dz, eps, x_grad, gamma_grad):
    """dz is the gradient w.r.t. the normalised (and gamma-scaled) output."""
    inv = rmsnorm_inv(x, eps)
    xhat = np.multiply(x, inv)
    if gamma is not None:
        if gamma_grad is not None:
            gamma_grad = np.add(gamma_grad, np.sum(np.multiply(dz, xhat), axis=0))
        dxh = np.multiply(dz, gamma.reshape(1, -1))
    else:
        dxh = dz
    m = np.mean(np.multiply(dxh, xhat), axis=-1, keepdims=True)
    dx = np.multiply(np.subtract(dxh, np.multiply(xhat, m)), inv)
    return np.add(x_grad, dx), gamma_grad


# --------------------------------------------------------------------------------------
# a5  GELU (tanh form)         backend.py:376-414
# --------------------------------------------------------------------------------------
def gelu_forward(x):
    buf = np.multiply(x, x)
    buf = np.multiply(buf, x)
    buf = np.multiply(buf, GELU_A)
    buf = np.add(x, buf)
    buf = np.multiply(buf, GELU_C)
    buf = np.tanh(buf)
    buf = np.add(buf, 1.0)
    buf = np.multiply(x, buf)
    return np.multiply(buf, 0.5).astype(F32)


def gelu_backward(x, dy, x_grad):
    buf = np.multiply(x, x)
    buf = np.multiply(buf, x)
    buf = np.multiply(buf, GELU_A)
    buf = np.add(x, buf)
    buf = np.multiply(buf, GELU_C)
    t = np.tanh(buf)
    acc = np.subtract(1.0, np.multiply(t, t))
    d_inner = GELU_C * (1.0 + GELU_A3 * x * x)
    acc = np.multiply(acc, 0.5 * x * d_inner)
    left = np.multiply(np.add(t, 1.0), 0.5)
    local = np.add(left, acc)
    return np.add(x_grad, np.multiply(dy, local)).astype(F32)


# --------------------------------------------------------------------------------------
# a6  SwiGLU on packed [gate|up] rows
#     forward backend.py:1113-1126 ; backward backend.py:1178-1217
# --------------------------------------------------------------------------------------
def swiglu_forward(gu):
    H = gu.shape[-1] // 2
    g, u = gu[:, :H], gu[:, H:]
    sig = np.reciprocal(np.add(np.exp(np.negative(g)), 1.0))
    return np.multiply(np.multiply(g, sig), u).astype(F32)


def swiglu_backward(gu, dhidden):
    """Returns the packed [dgate|dup] array the reference leaves in `gu`."""
    H = gu.shape[-1] // 2
    g, u = gu[:, :H], gu[:, H:]
    sig = np.reciprocal(np.add(np.exp(np.negative(g)), 1.0))
    dg = np.subtract(1.0, sig)
    dg = np.multiply(dg, g)
    dg = np.add(dg, 1.0)
    dg = np.multiply(dg, sig)
    dg = np.multiply(dg, u)
    dg = np.multiply(dg, dhidden)
    du = np.multiply(np.multiply(g, sig), dhidden)
    return np.concatenate([dg, du], axis=1).astype(F32)


# --------------------------------------------------------------------------------------
# a7  RoPE, rotate-half layout   backend.py:1382-1417; tables module.py:247-255
# --------------------------------------------------------------------------------------
def rope_tables(T, D, theta):
    positions = np.arange(T, dtype=F32)[:, None]
    channels = np.arange(0, D, 2, dtype=F32)[None, :]
    inv_freq = F32(theta) ** (-channels / F32(D))
    freqs = positions * inv_freq
    return np.cos(freqs).astype(F32), np.sin(freqs).astype(F32)


def rope_apply(t, cos, sin, sin_sign):
    """t: (B, T, H, D).  sin_sign=+1: lo' = lo*c - hi*s, hi' = lo*s + hi*c (the reference's
    `apply_rope_backward_np`, which is the Qwen forward).  sin_sign=-1: lo' = lo*c + hi*s,
    hi' = -lo*s + hi*c (`apply_rope_np`, the nanochat forward = transpose of the former)."""
    d2 = t.shape[-1] // 2
    lo, hi = t[..., :d2], t[..., d2:]
    c = cos[None, :, None, :]
    s = sin[None, :, None, :]
    out = np.empty_like(t)
    if sin_sign > 0:
        out[..., :d2] = lo * c - hi * s
        out[..., d2:] = lo * s + hi * c
    else:
        out[..., :d2] = lo * c + hi * s
        out[..., d2:] = -lo * s + hi * c
    return out


# --------------------------------------------------------------------------------------
# a8/a9  embedding gather and its scatter-add backward   backend.py:525-538
# --------------------------------------------------------------------------------------
def gather_forward(ids, table):
    return table[ids.astype(np.int64)]


def gather_backward(ids, dout, table_grad):
    """np.add.at: unbuffered, sequential in ascending flat token order."""
    out = table_grad.copy()
    np.add.at(out, ids.astype(np.int64).ravel(), dout.reshape(-1, table_grad.shape[-1]))
    return out


# --------------------------------------------------------------------------------------
# a10/a11  fused linear + cross-entropy   backend.py:628-714
# --------------------------------------------------------------------------------------
def _softmax_rows(L):
    m = np.max(L, axis=-1, keepdims=True)
    e = np.exp(np.subtract(L, m))
    s = np.sum(e, axis=-1, keepdims=True)
    return np.divide(e, s), m, s


def flce_forward_reference(X, W, Y, chunk=1024):
    """Verbatim semantics of cpu_fused_linear_ce_forward: `-log(p[target] + 1e-10)` for
    targets != -1, python-float accumulation, divided by ALL rows (backend.py:659-664)."""
    N = X.shape[0]
    loss_sum = 0.0
    for i in range(0, N, chunk):
        P, _, _ = _softmax_rows(np.matmul(X[i:i + chunk], W.T))
        Ys = Y[i:i + chunk]
        for j in range(P.shape[0]):
            if Ys[j] != -1:
                loss_sum -= np.log(P[j, Ys[j]] + 1e-10)
    return F32(loss_sum / N)


def flce_backward_reference(X, W, Y, dloss, dX, dW, chunk=1024):
    """Verbatim semantics of cpu_fused_linear_ce_backward: rows whose target is -1 are NOT
    masked, they contribute softmax*scale (backend.py:693-697)."""
    N = X.shape[0]
    scale = F32(dloss) / N
    dX = dX.copy()
    dW = dW.copy()
    for i in range(0, N, chunk):
        Xs = X[i:i + chunk]
        P, _, _ = _softmax_rows(np.matmul(Xs, W.T))
        Ys = Y[i:i + chunk]
        for j in range(P.shape[0]):
            if Ys[j] != -1:
                P[j, Ys[j]] -= 1.0
        P = np.multiply(P, scale)
        dX[i:i + chunk] += np.matmul(P, W)
        dW += np.matmul(P.T, Xs)
    return dX, dW


def flce_valid_mask(Y, V):
    """Rows that take part in the loss: 0 <= target < V (metal_ops.metal:8920;
    backend.py:768 for the newer CPU RMSNorm head)."""
    return (Y >= 0) & (Y < V)


def flce_masked(X, W, Y, dloss=1.0, reduction="mean_all_rows", chunk=1024,
                dX=None, dW=None, row_scale=None):
    """Masked fused linear + CE: ignored / out-of-range targets give zero loss AND zero
    gradient (metal_ops.metal:8920-8926, :8968-8979;
    debug/check_fused_linear_ce_kernel_trace.py:142-177; backend.py:838-840).
    loss uses lse - logit[target] (backend.py:775-776 formulation).
    reduction: "mean_all_rows" divides by N (backend.py:664), "mean_valid" by the number
    of valid rows.  Returns dict(loss, lse, row_loss, dX, dW, n_valid)."""
    N, C = X.shape
    V = W.shape[0]
    valid = flce_valid_mask(Y, V)
    n_valid = int(valid.sum())
    denom = N if reduction == "mean_all_rows" else max(n_valid, 1)
    dX = np.zeros((N, C), F32) if dX is None else dX.copy()
    dW = np.zeros((V, C), F32) if dW is None else dW.copy()
    lse = np.empty(N, F32)
    row_loss = np.zeros(N, F32)
    for i in range(0, N, chunk):
        Xs = X[i:i + chunk]
        L = np.matmul(Xs, W.T)
        P, m, s = _softmax_rows(L)
        n = L.shape[0]
        lse[i:i + n] = (m[:, 0] + np.log(s[:, 0])).astype(F32)
        v = valid[i:i + n]
        rows = np.flatnonzero(v)
        tl = np.zeros(n, F32)
        tl[rows] = L[rows, Y[i:i + n][rows]]
        rl = lse[i:i + n] - tl
        rl[~v] = 0.0
        row_loss[i:i + n] = rl
        P[rows, Y[i:i + n][rows]] -= 1.0
        P[~v] = 0.0
        if row_scale is None:
            P = np.multiply(P, F32(dloss) / F32(denom))
        else:
            P = np.multiply(P, (F32(dloss) * row_scale[i:i + n])[:, None])
        dX[i:i + n] += np.matmul(P, W)
        dW += np.matmul(P.T, Xs)
    if row_scale is None:
        loss = F32(np.sum(row_loss, dtype=F32) / F32(denom))
    else:
        loss = F32(np.sum(row_loss * row_scale, dtype=F32))
    return dict(loss=loss, lse=lse, row_loss=row_loss, dX=dX, dW=dW, n_valid=n_valid)


# --------------------------------------------------------------------------------------
# f1  RMSNorm + linear + CE head   backend.py:716-886
# --------------------------------------------------------------------------------------
def rmsnorm_flce(X, W, G, Y, eps, dloss=1.0, row_scale=None, chunk=1024):
    """Returns dict(loss, dX, dW, dG) for zero incoming gradients."""
    Z, inv = rmsnorm_forward(X, G, eps)
    r = flce_masked(Z, W, Y, dloss=dloss, chunk=chunk, row_scale=row_scale)
    dZ = r["dX"]
    dX, dG = rmsnorm_backward(X, G, dZ, eps, np.zeros_like(X), np.zeros_like(G))
    return dict(loss=r["loss"], dX=dX, dW=r["dW"], dG=dG)


# --------------------------------------------------------------------------------------
# f2  linear projection + bias + residual   backend.py:2040-2058, :2249-2259
# --------------------------------------------------------------------------------------
def linear_add_forward(x, act, w, b):
    out = np.matmul(act, w)
    out = np.add(out, b)
    return np.add(out, x).astype(F32)


def linear_add_backward(dout, act, w, x_grad, act_grad, w_grad, b_grad):
    """Returns updated (x_grad, act_grad, w_grad, b_grad); all accumulate."""
    return (np.add(x_grad, dout), np.add(act_grad, (dout @ w.T).astype(F32)),
            np.add(w_grad, (act.T @ dout).astype(F32)), np.add(b_grad, np.sum(dout, axis=0).astype(F32)))


# --------------------------------------------------------------------------------------
# f3  AdamW fp32 step            backend.py:2013-2038
# --------------------------------------------------------------------------------------
def adamw_step(p, g, m, v, lr, lr_t, b1, b2, eps, wd):
    """Returns updated (p, m, v); python-float scalars multiply fp32 arrays as in the
    reference (numpy keeps the arrays' fp32)."""
    if wd > 0.0:
        p = np.subtract(p, np.multiply(p, lr * wd))
    m = np.add(np.multiply(m, b1), np.multiply(g, 1.0 - b1))
    v = np.add(np.multiply(v, b2), np.multiply(np.multiply(g, g), 1.0 - b2))
    step = np.multiply(np.divide(m, np.add(np.sqrt(v), eps)), lr_t)
    p = np.subtract(p, step)
    return p.astype(F32), m.astype(F32), v.astype(F32)


# --------------------------------------------------------------------------------------
# f4  parameter gradients stored as bf16 bit patterns (grad_dtype="bf16", runtime.py:185-202).
# The reference implements these three only as Metal kernels; each is restated here from the
# kernel text, out of pieces that are pinned on their own (the rounding rule, np.add.at,
# cpu_adamw_step).
# --------------------------------------------------------------------------------------
def f32_to_bf16_store(src, dst_bits, accumulate):
    """`fp32_to_bf16` (metal_ops.metal:12010-12041): dst = bf16(src [+ float(dst)])."""
    value = np.ascontiguousarray(src, dtype=F32)
    if accumulate:
        value = np.add(value, bf16_bits_to_f32(dst_bits).reshape(value.shape))
    return f32_to_bf16_bits(value).reshape(value.shape)


def gather_backward_bf16(ids, dout, table_bits):
    """`gather_backward_bf16_kernel` (metal_ops.metal:12395-12446): per token row that occurs in ids,
    the fp32 sum of its dout rows in ascending position order starting from zero, then
    row = bf16(float(row) + sum); rows that do not occur are left as they are."""
    C = table_bits.shape[-1]
    flat = ids.astype(np.int64).ravel()
    sums = np.zeros(table_bits.shape, F32)
    np.add.at(sums, flat, dout.reshape(-1, C))
    out = np.array(table_bits, dtype=np.uint16, copy=True)
    touched = np.unique(flat)
    out[touched] = f32_to_bf16_bits(np.add(bf16_bits_to_f32(table_bits[touched]), sums[touched])).reshape(-1, C)
    return out


def adamw_step_bf16grad(p, g_bits, m, v, lr, lr_t, b1, b2, eps, wd, grad_scale=1.0):
    """`adamw_step` with its bf16-gradient flag (backend.py:5125-5140): g is widened to fp32 and
    scaled, then the fp32 step."""
    g = np.multiply(bf16_bits_to_f32(g_bits).reshape(p.shape), F32(grad_scale))
    return adamw_step(p, g, m, v, lr, lr_t, b1, b2, eps, wd)
