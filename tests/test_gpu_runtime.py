"""The reference's own graph runtime in front of this backend, on the GPU.

`Runtime(device="cuda")` (runtime.py:69-100) compiles a graph of the reference's own `Tensor` /
`Op` objects - build_topo (runtime.py:123-255) binds every node to this backend's callables,
bind_memory (:272-513) plans ONE arena with this backend's scratch slots inside it - and
`execute` (:802-854) runs zero_grad, forward, the loss-gradient fill and backward_graph.  The same
graph on the same seeded inputs runs through `Runtime(device="cpu")`, the reference's numpy
kernels, in the same process; loss and every leaf gradient must agree (pattern of
check_tiny_gpt2_kernel.py:473-490).

The reference's modules come from `oracle/_ref` (unmodified copies, made by oracle/make_ref.py).
"""
from types import SimpleNamespace

import numpy as np
import pytest

from conftest import TOL_BWD, TOL_FWD, assert_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    from oracle import ref_loader
    if not ref_loader.available():
        pytest.skip("oracle/_ref has not been made (python oracle/make_ref.py --reference <checkout>)")
    mods = ref_loader.load()
    import autograd_b200 as ag
    import gpu_util as G
    ag.register(existing=G.env(), reference=SimpleNamespace(device=mods.device, runtime=mods.runtime, scratch=mods.scratch))
    return mods


def _leaf(ref, device, value, requires_grad=True, name=""):
    value = np.ascontiguousarray(value)
    return ref.tensor.Tensor(shape=tuple(value.shape), dtype=value.dtype.type, requires_grad=requires_grad,
                             init_val=value, device=device, name=name)


def _run(ref, device, build, fuse=False, grad_scale=1.0, repeat=1):
    """Compile and execute `build(device)` -> (loss, leaves); returns loss and leaf gradients on the host."""
    from autograd_b200 import device as agdev
    ref.runtime.Runtime._default_runtime = None
    rt = ref.runtime.Runtime(device=device)
    loss, leaves = build(device)
    rt.loss = loss
    rt.grad_scale = float(grad_scale)
    rt.backend.grad_scale = rt.grad_scale
    rt.build_topo(loss)
    rt.bind_memory()
    rt.is_compiled = True
    fused = agdev.fuse_add_layernorm(rt) if fuse else 0
    for _ in range(repeat):
        rt.execute()
    rt.backend.synchronize()
    out = {"loss": float(np.asarray(rt.backend.copy_to_host(loss)).reshape(-1)[0]), "fused": fused, "rt": rt}
    for name, t in leaves.items():
        if t.grad is not None and t.grad.storage is not None:
            out["d" + name] = np.array(rt.backend.copy_to_host(t.grad), copy=True)
    return out


def _release(res):
    """Give the arena and the leaves of a finished cuda runtime back."""
    import gpu_util as G
    ctx, alloc, be = G.env()
    rt = res["rt"]
    ctx.synchronize()
    be.release_side_buffers()
    seen = set()
    for node in rt.topo:
        for t in node.inputs + node.outputs:
            for s in (t.storage, t.grad.storage if t.grad is not None else None):
                if s is not None and s.ptr.buffer_id not in seen:
                    seen.add(s.ptr.buffer_id)
                    alloc.free(s)
    if rt.unified_arena is not None and rt.unified_arena.ptr.buffer_id not in seen:
        alloc.free(rt.unified_arena)


def _gpt_graph(ref, B, T, C, V, seed, ignore_frac):
    """Gather -> Add -> LayerNorm -> GELU -> Add -> LayerNorm -> fused linear + CE on the tied table."""
    rng = np.random.default_rng(seed)
    f = np.float32
    ids = rng.integers(0, V, size=(B, T)).astype(np.int32)
    ids[0, : T // 3] = 3                                   # a hot table row for the scatter-add
    tg = rng.integers(0, V, size=(B, T)).astype(np.int32)
    if ignore_frac:
        tg[rng.random((B, T)) < ignore_frac] = -1
    table = (0.1 * rng.standard_normal((V, C))).astype(f)
    r = rng.standard_normal((B, T, C)).astype(f)
    g1, g2 = ((1 + 0.02 * rng.standard_normal(C)).astype(f) for _ in range(2))
    b1, b2 = ((0.02 * rng.standard_normal(C)).astype(f) for _ in range(2))

    def build(device):
        op = ref.op
        t_ids = _leaf(ref, device, ids, requires_grad=False, name="ids")
        t_tg = _leaf(ref, device, tg, requires_grad=False, name="targets")
        t_table, t_r = _leaf(ref, device, table, name="table"), _leaf(ref, device, r, name="r")
        t_g1, t_b1 = _leaf(ref, device, g1, name="g1"), _leaf(ref, device, b1, name="b1")
        t_g2, t_b2 = _leaf(ref, device, g2, name="g2"), _leaf(ref, device, b2, name="b2")
        x = op.GatherOp()(t_ids, t_table)
        h1 = op.AddOp()(x, t_r)
        y1 = op.LayerNormOp(eps=1e-5)(h1, t_g1, t_b1)
        a = op.GELUOp()(y1)
        h2 = op.AddOp()(h1, a)
        y2 = op.LayerNormOp(eps=1e-5)(h2, t_g2, t_b2)
        loss = y2.fused_linear_cross_entropy(t_table, t_tg)
        return loss, {"table": t_table, "r": t_r, "g1": t_g1, "b1": t_b1, "g2": t_g2, "b2": t_b2}

    return build


def _compare(cpu, gpu, names, what):
    assert abs(gpu["loss"] - cpu["loss"]) <= TOL_FWD * abs(cpu["loss"]), (what, gpu["loss"], cpu["loss"])
    for n in names:
        assert_close(gpu["d" + n], cpu["d" + n], TOL_BWD, f"{what}: d{n}")


@pytest.mark.parametrize("fuse", [False, True])
def test_reference_runtime_drives_cuda_backend_gpt_graph(ref, fuse):
    """No ignored targets: the reference CPU head and this backend's default (masked) head agree.
    With `fuse`, the Add + LayerNorm pairs run as the fused kernel (h and y in one pass)."""
    import gpu_util as G
    ctx, alloc, be = G.env()
    be.ce_vocab_chunk, be.ce_precision = 512, 1          # two vocabulary panels on the tensor-core path
    build = _gpt_graph(ref, B=4, T=96, C=256, V=1000, seed=31, ignore_frac=0.0)
    cpu = _run(ref, "cpu", build)
    gpu = _run(ref, "cuda", build, fuse=fuse, repeat=2)    # a second execute(): zero_grad must reset every gradient
    assert gpu["fused"] == (2 if fuse else 0)
    assert gpu["rt"].need_scratch is False and gpu["rt"].backend is be
    ln = [n for n in gpu["rt"].topo if type(n.op).__name__ == "LayerNormOp"][0]
    assert "scratch" in ln.backward.keywords               # the partial rows live in the arena, not in the workspace
    _compare(cpu, gpu, ("table", "r", "g1", "b1", "g2", "b2"), f"gpt graph fuse={fuse}")
    G.check_clean_status()
    _release(gpu)
    be.ce_vocab_chunk = 4096


def test_reference_runtime_ignored_targets_and_grad_scale(ref):
    """Targets of -1 with the compat switch: `cpu_fused_linear_ce_backward` does not mask ignored rows
    (backend.py:693-697), and AG_CE_IGNORE_COMPAT_UNMASKED reproduces it verbatim through the runtime;
    the default masked mode must differ from it on the same graph.  grad_scale goes through the
    runtime's own hook (runtime.py:89-95, :814)."""
    import autograd_b200 as ag
    import gpu_util as G
    ctx, alloc, be = G.env()
    build = _gpt_graph(ref, B=2, T=80, C=128, V=700, seed=32, ignore_frac=0.1)
    cpu = _run(ref, "cpu", build, grad_scale=0.5)
    be.ce_ignore_mode = ag.AG_CE_IGNORE_COMPAT_UNMASKED
    try:
        gpu = _run(ref, "cuda", build, grad_scale=0.5)
    finally:
        be.ce_ignore_mode = ag.AG_CE_IGNORE_MASKED
    _compare(cpu, gpu, ("table", "r", "g1", "b1", "g2", "b2"), "compat-unmasked")
    _release(gpu)
    masked = _run(ref, "cuda", build, grad_scale=0.5)
    assert abs(masked["loss"] - cpu["loss"]) <= TOL_FWD * abs(cpu["loss"])     # the loss never counted ignored rows
    d = np.abs(masked["dr"] - cpu["dr"]).max() / np.sqrt(np.mean(cpu["dr"] ** 2))
    assert d > 1e-3, d                                                          # the gradients do differ by design
    G.check_clean_status()
    _release(masked)


def test_reference_runtime_qwen_head_and_projection(ref):
    """Add -> FusedLinearAdd (output aliases its residual input in the arena, runtime.py:397-417) ->
    FusedRMSNormLinearCrossEntropy with row_scale and out-of-range targets (backend.py:716-886),
    the head of the reference's Qwen / RL graphs, on the tensor-core path."""
    import gpu_util as G
    ctx, alloc, be = G.env()
    rng = np.random.default_rng(33)
    f = np.float32
    B, T, C, K, V = 2, 72, 128, 192, 900
    p = rng.standard_normal((B, T, C)).astype(f)
    q = rng.standard_normal((B, T, C)).astype(f)
    act = rng.standard_normal((B, T, K)).astype(f)
    w = (rng.standard_normal((K, C)) / np.sqrt(K)).astype(f)
    b = (0.1 * rng.standard_normal(C)).astype(f)
    gam = (1 + 0.02 * rng.standard_normal(C)).astype(f)
    wv = (0.3 * rng.standard_normal((V, C))).astype(f)
    tg = rng.integers(0, V, size=(B, T)).astype(np.int32)
    tg[0, :5] = -1
    tg[1, :3] = V                                       # out of range: ignored like -1 (backend.py:768)
    rs = (rng.random((B, T)).astype(f) / (B * T)).astype(f)

    def build(device):
        op = ref.op
        t_p, t_q, t_act = _leaf(ref, device, p, name="p"), _leaf(ref, device, q, name="q"), _leaf(ref, device, act, name="act")
        t_w, t_b, t_gam, t_wv = (_leaf(ref, device, v, name=n) for v, n in ((w, "w"), (b, "b"), (gam, "gam"), (wv, "wv")))
        t_tg = _leaf(ref, device, tg, requires_grad=False, name="targets")
        t_rs = _leaf(ref, device, rs, requires_grad=False, name="row_scale")
        h0 = op.AddOp()(t_p, t_q)
        h1 = op.FusedLinearAddOp()(h0, t_act, t_w, t_b)
        loss = h1.fused_rmsnorm_linear_cross_entropy(t_wv, t_gam, t_tg, row_scale=t_rs, eps=1e-6)
        return loss, {"p": t_p, "q": t_q, "act": t_act, "w": t_w, "b": t_b, "gam": t_gam, "wv": t_wv}

    be.ce_vocab_chunk, be.ce_precision = 512, 1
    cpu = _run(ref, "cpu", build)
    gpu = _run(ref, "cuda", build)
    rt = gpu["rt"]
    fla = [n for n in rt.topo if type(n.op).__name__ == "FusedLinearAddOp"][0]
    from autograd_b200.storage import address_of
    assert address_of(fla.outputs[0].storage) == address_of(fla.inputs[0].storage)   # in place in the arena
    _compare(cpu, gpu, ("p", "q", "act", "w", "b", "gam", "wv"), "qwen head")
    G.check_clean_status()
    _release(gpu)
    be.ce_vocab_chunk = 4096
