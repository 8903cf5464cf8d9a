"""Generate the committed golden vectors by running the reference's own CPU backend.

Run where the reference checkout is available:

    python tests/golden/make_golden.py [--reference /path/to/autograd]

The reference imports `metal_ext` (Apple-only) at module import time; a stub module that
raises on use is injected so that the CPU backend loads on Linux.  Every case is seeded;
inputs and the reference outputs are stored together in one `.npz` per kernel family next
to this script.  `tests/test_oracle_golden.py` checks the numpy oracle against these
files, the GPU parity tests check the CUDA kernels against them.

Two routes into the reference are used, both taken from its own test scripts:
  * whole ops through `Runtime(device="cpu")`: build -> bind_memory -> forward -> inject the
    upstream gradient -> backward_graph (check_tiny_gpt2_kernel.py:473-490);
  * stage-level values harvested from the scratch of the fused ops by calling the `cpu_*`
    kernels on namespace tensors (debug/backend.py:25-36).
"""
from __future__ import annotations

import argparse
import os
import sys
import types
from types import SimpleNamespace as NS

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SEED = 1234  # verify_model.py:22 uses one fixed seed; each case adds an offset


def load_reference(path):
    stub = types.ModuleType("metal_ext")

    class MetalContext:  # noqa: D401 - stub
        def __init__(self, *a, **k):
            raise RuntimeError("metal_ext is not available on this host")

    stub.MetalContext = MetalContext
    sys.modules["metal_ext"] = stub
    sys.path.insert(0, path)
    import backend  # noqa: F401
    import op  # noqa: F401
    import runtime  # noqa: F401
    import tensor  # noqa: F401
    return SimpleNamespaceModules(backend=backend, op=op, runtime=runtime, tensor=tensor)


class SimpleNamespaceModules(NS):
    pass


def make_tensor(ref, shape, dtype, requires_grad, value):
    return ref.tensor.Tensor(shape=tuple(shape), dtype=dtype, requires_grad=requires_grad,
                             init_val=np.asarray(value, dtype=dtype), device="cpu")


def run_single_op(ref, build_fn, upstream, preload=None):
    """check_tiny_gpt2_kernel.py:473-490, plus optional pre-loading of grads (the
    reference's own residual-grad test does that: debug/check_qwen_kernel.py:471-487)."""
    ref.runtime.Runtime._default_runtime = None
    rt = ref.runtime.Runtime(device="cpu")
    out, tracked = build_fn()
    rt.loss = out
    rt.build_topo(out)
    rt.bind_memory()
    rt.forward()
    rt.zero_grad()
    if preload:
        for name, arr in preload.items():
            rt.backend.copy_from_host(tracked[name].grad, arr)
    rt.backend.copy_from_host(out.grad, np.asarray(upstream, dtype=np.float32))
    rt.backward_graph()
    res = {"out": np.array(rt.backend.copy_to_host(out), copy=True)}
    for name, t in tracked.items():
        if t.grad is not None and t.grad.storage is not None:
            res["d" + name] = np.array(rt.backend.copy_to_host(t.grad), copy=True)
    return res


def ns_tensor(data, requires_grad=True, op=None, grad=None):
    t = NS()
    t.shape = data.shape
    t.dtype = data.dtype
    t.requires_grad = requires_grad
    t.op = op
    t.storage = NS(data=data)
    t.grad = None if grad is None else NS(storage=NS(data=grad), shape=grad.shape)
    return t


def scratch_dict(**arrays):
    return {k: NS(data=v) for k, v in arrays.items()}


# ----------------------------------------------------------------------------------
def gen_add_layernorm(ref, out):
    cases = {
        # the reference's own LayerNorm probe shape (check_tiny_gpt2_kernel.py:758-782)
        "probe": (2, 16, 64, 1e-5, SEED + 4),
        # config-1 hidden size at a reduced row count
        "c384": (2, 12, 384, 1e-5, SEED + 10),
        # ragged: C not a multiple of 4, single row
        "ragged": (1, 1, 7, 1e-5, SEED + 11),
        "c100": (3, 5, 100, 1e-6, SEED + 12),
        "c1280": (1, 5, 1280, 1e-5, SEED + 13),
    }
    blob = {}
    for name, (B, T, C, eps, seed) in cases.items():
        rng = np.random.default_rng(seed)
        x = rng.standard_normal((B, T, C), dtype=np.float32)
        r = rng.standard_normal((B, T, C), dtype=np.float32)
        g = (1 + 0.02 * rng.standard_normal(C)).astype(np.float32)
        b = (0.02 * rng.standard_normal(C)).astype(np.float32)
        dy = rng.standard_normal((B, T, C), dtype=np.float32)

        def build():
            xt = make_tensor(ref, x.shape, np.float32, True, x)
            rt_ = make_tensor(ref, r.shape, np.float32, True, r)
            gt = make_tensor(ref, g.shape, np.float32, True, g)
            bt = make_tensor(ref, b.shape, np.float32, True, b)
            h = ref.op.AddOp()(xt, rt_)
            y = ref.op.LayerNormOp(eps=eps)(h, gt, bt)
            return y, {"x": xt, "r": rt_, "gamma": gt, "beta": bt, "h": h}

        res = run_single_op(ref, build, dy)
        # LayerNorm alone with a pre-loaded x.grad (fused residual-grad add)
        h_np = (x + r).astype(np.float32)
        resid = rng.standard_normal((B, T, C), dtype=np.float32)

        def build_ln():
            ht = make_tensor(ref, h_np.shape, np.float32, True, h_np)
            gt = make_tensor(ref, g.shape, np.float32, True, g)
            bt = make_tensor(ref, b.shape, np.float32, True, b)
            y = ref.op.LayerNormOp(eps=eps)(ht, gt, bt)
            return y, {"h": ht, "gamma": gt, "beta": bt}

        res2 = run_single_op(ref, build_ln, dy, preload={"h": resid})
        for k, v in dict(x=x, r=r, gamma=g, beta=b, dy=dy, eps=np.float32(eps), y=res["out"],
                         dx=res["dx"], dr=res["dr"], dgamma=res["dgamma"], dbeta=res["dbeta"],
                         resid=resid, dh_with_resid=res2["dh"]).items():
            blob[f"{name}.{k}"] = v
    np.savez_compressed(os.path.join(out, "add_layernorm.npz"), **blob)


def gen_gelu(ref, out):
    blob = {}
    for name, shape, seed in (("probe", (2, 16, 64), SEED + 5), ("ragged", (3, 37), SEED + 20),
                              ("wide", (5, 1536), SEED + 21)):
        rng = np.random.default_rng(seed)
        x = (rng.standard_normal(shape, dtype=np.float32) * 3).astype(np.float32)
        dy = rng.standard_normal(shape, dtype=np.float32)
        pre = rng.standard_normal(shape, dtype=np.float32)

        def build():
            # x must be an intermediate for the runtime to bind an activation grad; use the
            # leaf directly as the reference probe does (check_tiny_gpt2_kernel.py:783-794)
            xt = make_tensor(ref, shape, np.float32, True, x)
            return ref.op.GELUOp()(xt), {"x": xt}

        res = run_single_op(ref, build, dy, preload={"x": pre})
        blob.update({f"{name}.x": x, f"{name}.dy": dy, f"{name}.pre": pre,
                     f"{name}.y": res["out"], f"{name}.dx": res["dx"]})
    np.savez_compressed(os.path.join(out, "gelu.npz"), **blob)


def gen_gather(ref, out):
    blob = {}
    for name, (B, T, V, C, seed) in {"small": (2, 16, 50, 32, SEED + 30),
                                     "collide": (4, 64, 37, 100, SEED + 31),
                                     "wide": (2, 20, 60, 1536, SEED + 32)}.items():
        rng = np.random.default_rng(seed)
        p = 1.0 / np.arange(1, V + 1) ** 1.1
        p /= p.sum()
        ids = rng.choice(V, size=(B, T), p=p).astype(np.int32)
        table = (0.02 * rng.standard_normal((V, C))).astype(np.float32)
        dout = rng.standard_normal((B, T, C), dtype=np.float32)

        def build():
            it = make_tensor(ref, ids.shape, np.int32, False, ids)
            wt = make_tensor(ref, table.shape, np.float32, True, table)
            return ref.op.GatherOp()(it, wt), {"w": wt}

        res = run_single_op(ref, build, dout)
        blob.update({f"{name}.ids": ids, f"{name}.table": table, f"{name}.dout": dout,
                     f"{name}.out": res["out"], f"{name}.dtable": res["dw"]})
    np.savez_compressed(os.path.join(out, "gather.npz"), **blob)


def gen_flce(ref, out):
    blob = {}
    for name, (B, T, C, V, seed) in {"small": (2, 24, 32, 200, SEED + 40),
                                     "ragged": (1, 37, 20, 131, SEED + 41),
                                     "multi_chunk": (3, 350, 48, 300, SEED + 42)}.items():
        rng = np.random.default_rng(seed)
        X = (rng.standard_normal((B, T, C)) / np.sqrt(C)).astype(np.float32)
        W = (0.02 * rng.standard_normal((V, C))).astype(np.float32)
        if name == "small":
            W *= 20  # spread the softmax so that the target term matters
        Y = rng.integers(0, V, size=(B, T)).astype(np.int32)
        Y[rng.random((B, T)) < 0.05] = -1
        Y[0, 0] = -1

        def build():
            xt = make_tensor(ref, X.shape, np.float32, True, X)
            wt = make_tensor(ref, W.shape, np.float32, True, W)
            yt = make_tensor(ref, Y.shape, np.int32, False, Y)
            return ref.op.FusedLinearCrossEntropyOp()(xt, wt, yt), {"x": xt, "w": wt}

        res = run_single_op(ref, build, np.array([1.0], np.float32))
        blob.update({f"{name}.X": X, f"{name}.W": W, f"{name}.Y": Y, f"{name}.loss": res["out"],
                     f"{name}.dX": res["dx"], f"{name}.dW": res["dw"]})
        # the same op on the valid rows only: the masked semantics (loss, dX, dW scale by
        # N_valid/N; ignored rows get zero dX)
        flatY = Y.reshape(-1)
        keep = np.flatnonzero(flatY != -1)
        Xv = X.reshape(-1, C)[keep][None]
        Yv = flatY[keep][None]

        def build_v():
            xt = make_tensor(ref, Xv.shape, np.float32, True, Xv)
            wt = make_tensor(ref, W.shape, np.float32, True, W)
            yt = make_tensor(ref, Yv.shape, np.int32, False, Yv)
            return ref.op.FusedLinearCrossEntropyOp()(xt, wt, yt), {"x": xt, "w": wt}

        resv = run_single_op(ref, build_v, np.array([1.0], np.float32))
        blob.update({f"{name}.valid_rows": keep, f"{name}.loss_valid_only": resv["out"],
                     f"{name}.dX_valid_only": resv["dx"], f"{name}.dW_valid_only": resv["dw"]})
    np.savez_compressed(os.path.join(out, "flce.npz"), **blob)


def gen_rmsnorm_swiglu(ref, out):
    """Harvest the RMSNorm and SwiGLU stages from cpu_fused_rmsnorm_mlp_* scratch
    (backend.py:1092-1126, :1202-1251)."""
    blob = {}
    for name, (N, C, H, eps, with_gamma, seed) in {
            "qwenish": (12, 96, 40, 1e-6, True, SEED + 50),
            "nogamma": (5, 64, 24, 1e-6, False, SEED + 51),
            "ragged": (3, 50, 7, 1e-5, True, SEED + 52)}.items():
        rng = np.random.default_rng(seed)
        x = rng.standard_normal((N, C), dtype=np.float32)
        gamma = (1 + 0.02 * rng.standard_normal(C)).astype(np.float32)
        wgu = (rng.standard_normal((C, 2 * H)) / np.sqrt(C)).astype(np.float32)
        wdown = (rng.standard_normal((H, C)) / np.sqrt(H)).astype(np.float32)
        dout = rng.standard_normal((N, C), dtype=np.float32)
        resid = rng.standard_normal((N, C), dtype=np.float32)
        opnode = NS(op=NS(eps=eps))
        xt = ns_tensor(x, grad=resid.copy())
        wgu_t = ns_tensor(wgu, grad=np.zeros_like(wgu))
        wd_t = ns_tensor(wdown, grad=np.zeros_like(wdown))
        outt = ns_tensor(np.zeros((N, C), np.float32), op=opnode, grad=dout)
        if with_gamma:
            gt = ns_tensor(gamma, grad=np.zeros_like(gamma))
            inputs = (xt, gt, wgu_t, wd_t)
        else:
            inputs = (xt, wgu_t, wd_t)
        f = np.float32
        sc = scratch_dict(inv_rms=np.zeros((N, 1), f), x_norm=np.zeros((N, C), f),
                          gu=np.zeros((N, 2 * H), f), hidden=np.zeros((N, H), f))
        ref.backend.cpu_fused_rmsnorm_mlp_forward(inputs, (outt,), scratch=sc)
        blob.update({f"{name}.x": x, f"{name}.eps": f(eps), f"{name}.inv_rms": sc["inv_rms"].data[:, 0].copy(),
                     f"{name}.x_norm": sc["x_norm"].data.copy(), f"{name}.gu": sc["gu"].data.copy(),
                     f"{name}.hidden": sc["hidden"].data.copy()})
        if with_gamma:
            blob[f"{name}.gamma"] = gamma
        sb = scratch_dict(inv_rms=np.zeros((N, 1), f), x_norm=np.zeros((N, C), f),
                          dx_norm=np.zeros((N, C), f), gu=np.zeros((N, 2 * H), f),
                          dhidden=np.zeros((N, H), f), gate=np.zeros((N, H), f),
                          sigmoid=np.zeros((N, H), f), tmp_dwdown=np.zeros((H, C), f),
                          tmp_dwgu=np.zeros((C, 2 * H), f))
        ref.backend.cpu_fused_rmsnorm_mlp_backward(inputs, (outt,), scratch=sb)
        dgu = sb["gu"].data.copy()
        # dhidden as the op computed it (DOUT @ Wdown.T) is the SwiGLU-backward stage input.
        dhidden = np.matmul(dout, wdown.T)
        # The op stores mean(dz*xhat) over the first N floats of the flattened GU
        # (backend.py:1240), i.e. it clobbers part of [dgate|dup] AFTER using it.  Rebuild
        # the unclobbered array with the op's own statements (backend.py:1202-1217) and
        # insist that it is bit-identical wherever the op's copy survived.
        gate, up = sc["gu"].data[:, :H], sc["gu"].data[:, H:]
        sig = sb["sigmoid"].data
        dg = np.subtract(1.0, sig)
        dg = np.multiply(dg, gate)
        dg = np.add(dg, 1.0)
        dg = np.multiply(dg, sig)
        dg = np.multiply(dg, up)
        dg = np.multiply(dg, dhidden)
        du = np.multiply(np.multiply(gate, sig), dhidden)
        dgu_full = np.concatenate([dg, du], axis=1).astype(f)
        assert np.array_equal(dgu_full.reshape(-1)[N:], dgu.reshape(-1)[N:]), name
        # dz = dGU @ Wgu.T is the RMSNorm-backward stage input (backend.py:1220)
        dz = np.matmul(dgu_full, wgu.T)
        blob.update({f"{name}.dhidden": dhidden, f"{name}.dz": dz, f"{name}.resid": resid,
                     f"{name}.dx_with_resid": xt.grad.storage.data.copy()})
        if with_gamma:
            blob[f"{name}.dgamma"] = gt.grad.storage.data.copy()
        blob[f"{name}.dgu"] = dgu_full
    np.savez_compressed(os.path.join(out, "rmsnorm_swiglu.npz"), **blob)


def gen_rope(ref, out):
    blob = {}
    for name, (B, T, H, HKV, D, theta, seed) in {"qwen": (2, 9, 4, 2, 128, 1e6, SEED + 60),
                                                 "gpt": (1, 17, 3, 3, 64, 1e5, SEED + 61),
                                                 "tiny": (2, 3, 2, 1, 8, 1e4, SEED + 62)}.items():
        rng = np.random.default_rng(seed)
        q = rng.standard_normal((B, T, H, D), dtype=np.float32)
        k = rng.standard_normal((B, T, HKV, D), dtype=np.float32)
        # module.py:247-250
        positions = np.arange(T, dtype=np.float32)[:, None]
        channels = np.arange(0, D, 2, dtype=np.float32)[None, :]
        inv_freq = np.float32(theta) ** (-channels / np.float32(D))
        freqs = positions * inv_freq
        cos = np.cos(freqs).astype(np.float32)
        sin = np.sin(freqs).astype(np.float32)
        q_neg, k_neg = q.copy(), k.copy()
        ref.backend.apply_rope_np(q_neg, k_neg, cos, sin)
        q_pos, k_pos = q.copy(), k.copy()
        ref.backend.apply_rope_backward_np(q_pos, k_pos, cos, sin)
        blob.update({f"{name}.q": q, f"{name}.k": k, f"{name}.cos": cos, f"{name}.sin": sin,
                     f"{name}.theta": np.float32(theta),
                     f"{name}.q_neg": q_neg, f"{name}.k_neg": k_neg,
                     f"{name}.q_pos": q_pos, f"{name}.k_pos": k_pos})
    np.savez_compressed(os.path.join(out, "rope.npz"), **blob)


def gen_rmsnorm_flce(ref, out):
    blob = {}
    for name, (N, C, V, eps, scaled, seed) in {"plain": (40, 32, 150, 1e-6, False, SEED + 70),
                                               "row_scaled": (33, 24, 97, 1e-6, True, SEED + 71)}.items():
        rng = np.random.default_rng(seed)
        X = rng.standard_normal((1, N, C), dtype=np.float32)
        W = (0.2 * rng.standard_normal((V, C))).astype(np.float32)
        G = (1 + 0.02 * rng.standard_normal(C)).astype(np.float32)
        Y = rng.integers(0, V, size=(1, N)).astype(np.int32)
        Y[0, 1] = -1
        Y[0, 2] = V  # out of range is ignored too (debug/check_qwen_kernel.py:872-874)
        f = np.float32
        xt = ns_tensor(X, grad=np.zeros_like(X))
        wt = ns_tensor(W, grad=np.zeros_like(W))
        gt = ns_tensor(G, grad=np.zeros_like(G))
        yt = ns_tensor(Y, requires_grad=False)
        inputs = [xt, wt, gt, yt]
        if scaled:
            rs = (rng.random(N).astype(f) / N).reshape(1, N)
            inputs.append(ns_tensor(rs, requires_grad=False))
            blob[f"{name}.row_scale"] = rs
        outt = ns_tensor(np.zeros(1, f), op=NS(op=NS(eps=eps)), grad=np.array([1.0], f))
        sc = scratch_dict(logits=np.zeros((N, V), f), x_norm=np.zeros((N, C), f), dx_norm=np.zeros((N, C), f),
                          inv_rms=np.zeros((N, 1), f), max=np.zeros((N, 1), f), sum=np.zeros((N, 1), f),
                          target_logits=np.zeros((N, 1), f), tmp_x=np.zeros((N, C), f),
                          tmp_dw=np.zeros((V, C), f), tmp_dgamma=np.zeros(C, f))
        ref.backend.cpu_fused_rmsnorm_linear_ce_forward(tuple(inputs), (outt,), scratch=sc)
        loss = outt.storage.data.copy()
        ref.backend.cpu_fused_rmsnorm_linear_ce_backward(tuple(inputs), (outt,), scratch=sc)
        blob.update({f"{name}.X": X, f"{name}.W": W, f"{name}.G": G, f"{name}.Y": Y, f"{name}.eps": f(eps),
                     f"{name}.loss": loss, f"{name}.dX": xt.grad.storage.data.copy(),
                     f"{name}.dW": wt.grad.storage.data.copy(), f"{name}.dG": gt.grad.storage.data.copy()})
    np.savez_compressed(os.path.join(out, "rmsnorm_flce.npz"), **blob)


def gen_linear_add(ref, out):
    """cpu_fused_linear_add_forward / _backward (backend.py:2040-2058, :2147-2259) on namespace tensors,
    the branch whose `act` is a materialised tensor."""
    blob = {}
    for name, (N, K, C, seed) in {"square": (48, 64, 64, 1234 + 90), "wide": (130, 32, 96, 1234 + 91),
                                  "mlp_down": (70, 256, 64, 1234 + 92)}.items():
        rng = np.random.default_rng(seed)
        f = np.float32
        x = rng.standard_normal((1, N, C), dtype=f)
        act = rng.standard_normal((1, N, K), dtype=f)
        w = (rng.standard_normal((K, C)) / np.sqrt(K)).astype(f)
        b = (0.1 * rng.standard_normal(C)).astype(f)
        dout = rng.standard_normal((1, N, C), dtype=f)
        pre = {k: rng.standard_normal(v.shape).astype(f) for k, v in dict(x=x, act=act, w=w, b=b).items()}
        xt = ns_tensor(x, grad=pre["x"].copy())
        at = ns_tensor(act, grad=pre["act"].copy())
        at.op = None
        wt = ns_tensor(w, grad=pre["w"].copy())
        bt = ns_tensor(b, grad=pre["b"].copy())
        outt = ns_tensor(np.zeros((1, N, C), f), grad=dout)
        ref.backend.cpu_fused_linear_add_forward((xt, at, wt, bt), (outt,))
        y = outt.storage.data.copy()
        ref.backend.cpu_fused_linear_add_backward((xt, at, wt, bt), (outt,))
        blob.update({f"{name}.x": x, f"{name}.act": act, f"{name}.w": w, f"{name}.b": b, f"{name}.dout": dout,
                     f"{name}.out": y, f"{name}.pre_x": pre["x"], f"{name}.pre_act": pre["act"],
                     f"{name}.pre_w": pre["w"], f"{name}.pre_b": pre["b"],
                     f"{name}.dx": xt.grad.storage.data.copy(), f"{name}.dact": at.grad.storage.data.copy(),
                     f"{name}.dw": wt.grad.storage.data.copy(), f"{name}.db": bt.grad.storage.data.copy()})
    np.savez_compressed(os.path.join(out, "linear_add.npz"), **blob)


def gen_adamw_bf16(ref, out):
    import utils as ref_utils
    rng = np.random.default_rng(SEED + 80)
    n = 1000
    p = rng.standard_normal(n, dtype=np.float32)
    g = rng.standard_normal(n, dtype=np.float32)
    m = (0.1 * rng.standard_normal(n)).astype(np.float32)
    v = (0.01 * rng.random(n)).astype(np.float32)
    hp = dict(lr=3e-4, lr_t=2.9e-4, b1=0.9, b2=0.95, eps=1e-8, wd=0.1)
    p2, m2, v2 = p.copy(), m.copy(), v.copy()
    ref.backend.cpu_adamw_step(NS(data=p2), NS(data=g), NS(data=m2), NS(data=v2), np.zeros(n, np.float32),
                               hp["lr"], hp["lr_t"], hp["b1"], hp["b2"], hp["eps"], hp["wd"])
    vals = np.concatenate([rng.standard_normal(200).astype(np.float32) * 10,
                           np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 1.0039062, 1.0117188,
                                     3.3895314e38, 1e-40], np.float32)])
    bits = np.array([ref_utils.bf16_bits(x) for x in vals], dtype=np.uint16)
    np.savez_compressed(os.path.join(out, "adamw_bf16.npz"), p=p, g=g, m=m, v=v, p_out=p2, m_out=m2,
                        v_out=v2, hp=np.array([hp[k] for k in ("lr", "lr_t", "b1", "b2", "eps", "wd")], np.float64),
                        bf16_in=vals, bf16_bits=bits)


def gen_grad_bf16(ref, out):
    """Gradients stored as bf16 bit patterns.  The reference has these three steps as Metal kernels only;
    the vectors are put together from reference functions that do run here, following the kernel text:
    utils.bf16_bits for every rounding, cpu_gather_backward for the position-ordered sums,
    cpu_adamw_step for the optimizer step."""
    import utils as ref_utils
    rng = np.random.default_rng(SEED + 90)
    bits_of = lambda a: np.array([ref_utils.bf16_bits(x) for x in np.asarray(a, np.float32).ravel()],
                                 dtype=np.uint16).reshape(np.shape(a))
    widen = lambda b: (np.asarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)
    # fp32_to_bf16 with and without accumulate (metal_ops.metal:12010-12041)
    n = 1003
    src = (rng.standard_normal(n) * 3).astype(np.float32)
    src[:6] = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 1.00390625], np.float32)
    dst0 = bits_of((rng.standard_normal(n) * 3).astype(np.float32))
    conv_plain = bits_of(src)
    conv_acc = bits_of(src + widen(dst0))
    # gather_backward_bf16_kernel (metal_ops.metal:12395-12446): sums from zero in position order, one rounding
    V, C, B, T = 50, 24, 3, 40
    ids = rng.integers(0, V // 2, size=(B, T)).astype(np.int32)   # repeats; rows >= V/2 stay untouched
    ids[0, :9] = 7                                                 # a hot row
    dout = rng.standard_normal((B, T, C)).astype(np.float32)
    table0 = bits_of((0.5 * rng.standard_normal((V, C))).astype(np.float32))
    sums = np.zeros((V, C), np.float32)
    w = NS(requires_grad=True, shape=(V, C), grad=NS(storage=NS(data=sums)))
    ref.backend.cpu_gather_backward((NS(storage=NS(data=ids)), w), (NS(grad=NS(storage=NS(data=dout))),))
    table1 = table0.copy()
    touched = np.unique(ids)
    table1[touched] = bits_of(widen(table0[touched]) + sums[touched])
    # adamw_step with bf16 gradients (backend.py:5125-5140)
    m_ = 1000
    p = rng.standard_normal(m_, dtype=np.float32)
    g_bits = bits_of(rng.standard_normal(m_, dtype=np.float32))
    m = (0.1 * rng.standard_normal(m_)).astype(np.float32)
    v = (0.01 * rng.random(m_)).astype(np.float32)
    hp = dict(lr=3e-4, lr_t=2.9e-4, b1=0.9, b2=0.95, eps=1e-8, wd=0.1)
    grad_scale = 0.5
    p2, m2, v2 = p.copy(), m.copy(), v.copy()
    g = widen(g_bits) * np.float32(grad_scale)
    ref.backend.cpu_adamw_step(NS(data=p2), NS(data=g), NS(data=m2), NS(data=v2), np.zeros(m_, np.float32),
                               hp["lr"], hp["lr_t"], hp["b1"], hp["b2"], hp["eps"], hp["wd"])
    np.savez_compressed(os.path.join(out, "grad_bf16.npz"), src=src, dst0=dst0, conv_plain=conv_plain,
                        conv_acc=conv_acc, ids=ids, dout=dout, table0=table0, table1=table1, p=p, g_bits=g_bits,
                        m=m, v=v, p_out=p2, m_out=m2, v_out=v2, grad_scale=np.float64(grad_scale),
                        hp=np.array([hp[k] for k in ("lr", "lr_t", "b1", "b2", "eps", "wd")], np.float64))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("AUTOGRAD_REFERENCE"),
                    help="path of the reference checkout (or set AUTOGRAD_REFERENCE)")
    ap.add_argument("--out", default=HERE)
    args = ap.parse_args()
    if not args.reference:
        ap.error("give --reference or set AUTOGRAD_REFERENCE")
    ref = load_reference(args.reference)
    for fn in (gen_add_layernorm, gen_gelu, gen_gather, gen_flce, gen_rmsnorm_swiglu, gen_rope,
               gen_rmsnorm_flce, gen_linear_add, gen_adamw_bf16, gen_grad_bf16):
        fn(ref, args.out)
        print("wrote", fn.__name__)


if __name__ == "__main__":
    main()
