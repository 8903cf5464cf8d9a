"""Timing of the reference's OWN CPU backend for the fused-layer path (the CPU arm of bench.py).

TEST / MEASUREMENT INFRASTRUCTURE ONLY.  Every number produced here comes from the unmodified
reference modules under `oracle/_ref` (see make_ref.py): one-op graphs compiled by the
reference's `Runtime(device="cpu")` and timed the way the reference times its own ops
(timing_ops.py:76-100: zero_grad, fill the upstream gradient, `perf_counter` around
`rt.forward()` and around `rt.backward_graph()`), plus the reference's standalone numpy RoPE
functions (backend.py:1382-1417), which have no op of their own.

numpy's elementwise passes are single-threaded; only the BLAS calls (`np.matmul`) use several
threads.  The BLAS thread count is set explicitly through threadpoolctl, so that a launcher which
exports OMP_NUM_THREADS=1 (torchrun does) cannot silently turn the baseline into a one-thread run.
"""
from __future__ import annotations

import contextlib
import io
import os
import time

import numpy as np

from . import ref_loader

F32 = np.float32


def use_all_cores():
    """Give BLAS every host core; returns (threads in use, description)."""
    cores = os.cpu_count() or 1
    try:
        from threadpoolctl import threadpool_info, threadpool_limits
        threadpool_limits(limits=cores, user_api="blas")
        blas = [p for p in threadpool_info() if p.get("user_api") == "blas"]
        used = max((int(p.get("num_threads", 1)) for p in blas), default=1)
        lib = ", ".join(f"{p.get('internal_api')} {p.get('version')}" for p in blas) or "unknown BLAS"
        return used, f"{lib}, {used} BLAS threads of {cores} host cores (numpy elementwise passes are single-threaded)"
    except Exception as e:  # threadpoolctl missing: report what the environment gives
        return cores, f"threadpoolctl unavailable ({e}); BLAS threads left to the environment"


class OpGraph:
    """One graph of reference ops compiled by the reference's CPU runtime."""

    def __init__(self, ref, build):
        self.ref = ref
        ref.runtime.Runtime._default_runtime = None
        self.rt = ref.runtime.Runtime(device="cpu")
        self.out, self.leaves = build(ref)
        with contextlib.redirect_stdout(io.StringIO()):       # the runtime prints its arena sizes
            self.rt.loss = self.out
            self.rt.build_topo(self.out)
            self.rt.bind_memory()
        self.rt.is_compiled = True

    def prepare(self):
        """What the reference's timing loop does before each timed pair (timing_ops.py:89-90)."""
        self.rt.zero_grad()
        self.rt.backend.fill(self.out.grad, 1.0)

    def forward(self):
        self.rt.forward()

    def backward(self):
        self.rt.backward_graph()

    def time_pair(self, warmup=1, iters=1):
        """(forward seconds, backward seconds), means over `iters` after `warmup` untimed pairs."""
        for _ in range(warmup):
            self.prepare(); self.forward(); self.backward()
        tf = tb = 0.0
        for _ in range(iters):
            self.prepare()
            t0 = time.perf_counter(); self.forward()
            t1 = time.perf_counter(); self.backward()
            t2 = time.perf_counter()
            tf += t1 - t0; tb += t2 - t1
        return tf / iters, tb / iters


def _leaf(ref, value, requires_grad=True):
    value = np.ascontiguousarray(value)
    return ref.tensor.Tensor(shape=tuple(value.shape), dtype=value.dtype.type, requires_grad=requires_grad,
                             init_val=value, device="cpu")


# ---- builders: each returns build(ref) -> (output tensor, dict of leaves) -------------------------------
def add_layernorm(B, T, C, eps=1e-5, seed=1234):
    rng = np.random.default_rng(seed)
    x, r = rng.standard_normal((B, T, C), dtype=F32), rng.standard_normal((B, T, C), dtype=F32)
    g = (1 + 0.02 * rng.standard_normal(C)).astype(F32)
    b = (0.02 * rng.standard_normal(C)).astype(F32)

    def build(ref):
        tx, tr, tg, tb = _leaf(ref, x), _leaf(ref, r), _leaf(ref, g), _leaf(ref, b)
        h = ref.op.AddOp()(tx, tr)
        return ref.op.LayerNormOp(eps=eps)(h, tg, tb), {"x": tx, "r": tr, "gamma": tg, "beta": tb}
    return build


def gelu(rows, cols, seed=1239):
    x = np.random.default_rng(seed).standard_normal((1, rows, cols), dtype=F32)

    def build(ref):
        tx = _leaf(ref, x)
        return ref.op.GELUOp()(tx), {"x": tx}
    return build


def gather(B, T, V, C, ids=None, seed=1237):
    rng = np.random.default_rng(seed)
    if ids is None:
        ids = rng.integers(0, V, size=(B, T))
    ids = np.asarray(ids).reshape(B, T).astype(np.int32)
    table = (0.02 * rng.standard_normal((V, C), dtype=F32)).astype(F32)

    def build(ref):
        ti, tt = _leaf(ref, ids, requires_grad=False), _leaf(ref, table)
        return ref.op.GatherOp()(ti, tt), {"table": tt}
    return build


def fused_linear_ce(B, T, C, V, ignore_frac=0.05, seed=1235):
    rng = np.random.default_rng(seed)
    X = (rng.standard_normal((B, T, C), dtype=F32) / np.sqrt(C)).astype(F32)
    W = (0.02 * rng.standard_normal((V, C), dtype=F32)).astype(F32)
    Y = rng.integers(0, V, size=(B, T)).astype(np.int32)
    Y[rng.random((B, T)) < ignore_frac] = -1

    def build(ref):
        tx, tw, ty = _leaf(ref, X), _leaf(ref, W), _leaf(ref, Y, requires_grad=False)
        return tx.fused_linear_cross_entropy(tw, ty), {"x": tx, "w": tw}
    return build


def rmsnorm_fused_linear_ce(B, T, C, V, ignore_frac=0.05, eps=1e-6, seed=1241):
    """FusedRMSNormLinearCrossEntropyOp with per-row weights (op.py:306-327, backend.py:716-886)."""
    rng = np.random.default_rng(seed)
    X = rng.standard_normal((B, T, C), dtype=F32)
    W = (0.02 * rng.standard_normal((V, C), dtype=F32)).astype(F32)
    g = (1 + 0.02 * rng.standard_normal(C)).astype(F32)
    Y = rng.integers(0, V, size=(B, T)).astype(np.int32)
    Y[rng.random((B, T)) < ignore_frac] = -1
    rs = np.full((B, T), 1.0 / (B * T), dtype=F32)

    def build(ref):
        tx, tw, tg = _leaf(ref, X), _leaf(ref, W), _leaf(ref, g)
        ty, trs = _leaf(ref, Y, requires_grad=False), _leaf(ref, rs, requires_grad=False)
        return tx.fused_rmsnorm_linear_cross_entropy(tw, tg, ty, row_scale=trs, eps=eps), {"x": tx, "w": tw, "gamma": tg}
    return build


def rmsnorm_mlp(B, T, C, I, eps=1e-6, seed=1236):
    """FusedRMSNormMLPOp: the carrier of the RMSNorm and SwiGLU stages (backend.py:1074-1251)."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((B, T, C), dtype=F32)
    g = (1 + 0.02 * rng.standard_normal(C)).astype(F32)
    wgu = (rng.standard_normal((C, 2 * I), dtype=F32) / np.sqrt(C)).astype(F32)
    wdown = (rng.standard_normal((I, C), dtype=F32) / np.sqrt(I)).astype(F32)

    def build(ref):
        tx, tg, t1, t2 = _leaf(ref, x), _leaf(ref, g), _leaf(ref, wgu), _leaf(ref, wdown)
        return ref.op.FusedRMSNormMLPOp(eps=eps)(tx, tg, t1, t2), {"x": tx, "gamma": tg}
    return build


class RopeBuffers:
    """q (H heads), k (HKV heads) and the cos/sin tables for the reference's numpy RoPE functions."""

    def __init__(self, ref, B, T, H, HKV, D, theta, seed=1240):
        rng = np.random.default_rng(seed)
        self.ref = ref
        self.q = rng.standard_normal((B, T, H, D), dtype=F32)
        self.k = rng.standard_normal((B, T, HKV, D), dtype=F32)
        pos = np.arange(T, dtype=F32)[:, None]
        ch = np.arange(0, D, 2, dtype=F32)[None, :]
        freqs = pos * (F32(theta) ** (-ch / F32(D)))         # module.py:247-250
        self.cos, self.sin = np.cos(freqs).astype(F32), np.sin(freqs).astype(F32)

    def forward(self):
        self.ref.backend.apply_rope_np(self.q, self.k, self.cos, self.sin)

    def backward(self):
        self.ref.backend.apply_rope_backward_np(self.q, self.k, self.cos, self.sin)

    def time_pair(self, iters=1):
        tf = tb = 0.0
        for _ in range(iters):
            t0 = time.perf_counter(); self.forward()
            t1 = time.perf_counter(); self.backward()
            t2 = time.perf_counter()
            tf += t1 - t0; tb += t2 - t1
        return tf / iters, tb / iters


class FusedLayerStepSample:
    """The fused-layer step of the GPT-shaped benchmark model on a sample of `tokens` token rows,
    executed with the reference's CPU kernels: every kernel launch of the step has its counterpart
    executed here - 1 gather, 2L+1 Add+LayerNorm, L RoPE(q,k), L GELU (4x width), 1 fused linear+CE, all
    forward and backward (the gather's backward is the reference's np.add.at scatter-add) - nothing is
    extrapolated over layers.  The one-op graphs are compiled once; a step re-runs them."""

    def __init__(self, n_layer, n_embd, n_head, head_dim, seq_len, vocab, tokens, mlp_ratio=4, rope_theta=1e5):
        self.ref = ref_loader.load()
        self.threads, self.blas = use_all_cores()
        self.L, C = n_layer, n_embd
        T = min(seq_len, tokens)
        B = max(tokens // T, 1)
        self.tokens = B * T
        self.rope = RopeBuffers(self.ref, B, T, n_head, n_head, head_dim, rope_theta)
        self.g_gather = OpGraph(self.ref, gather(B, T, vocab, C))
        self.g_ln = OpGraph(self.ref, add_layernorm(B, T, C))
        self.g_gelu = OpGraph(self.ref, gelu(B * T, mlp_ratio * C))
        self.g_ce = OpGraph(self.ref, fused_linear_ce(B, T, C, vocab))
        self.description = (f"{self.tokens} token rows ({B} x {T}) at full depth {n_layer} and full vocabulary {vocab}: "
                            f"1 gather, {2 * n_layer + 1} Add+LayerNorm, {n_layer} RoPE(q,k), {n_layer} GELU, 1 fused "
                            f"linear+CE, forward and backward, through the reference's Runtime(device='cpu') "
                            f"({ref_loader.blas_info()}; {self.blas})")

    def step(self):
        """One step; returns seconds."""
        t0 = time.perf_counter()
        for g in (self.g_gather, self.g_ln, self.g_gelu, self.g_ce):
            g.prepare()
        self.g_gather.forward()
        for _ in range(2 * self.L + 1):
            self.g_ln.forward()
        for _ in range(self.L):
            self.g_gelu.forward()
        for _ in range(self.L):
            self.rope.forward()
        self.g_ce.forward()
        self.g_ce.backward()
        for _ in range(2 * self.L + 1):
            self.g_ln.backward()
        for _ in range(self.L):
            self.g_gelu.backward()
        for _ in range(self.L):
            self.rope.backward()
        self.g_gather.backward()
        return time.perf_counter() - t0
