"""CPU-only checks: the C-ABI library loads and exports every symbol the header declares, the
host-side backend logic (kernel lookup, pointer arithmetic, argument marshalling, scratch
planning, registration into the reference when it is present), the add+LayerNorm peephole, and
the data-parallel reducer on two gloo ranks.  No compute call reaches a GPU here."""
import ctypes
import os
import re
import sys
import types

import numpy as np
import pytest

from conftest import ROOT

import autograd_b200 as ag
from autograd_b200 import _native, hostgraph as hg
from autograd_b200.backend import CudaBackend, bf16_bits_to_f32, f32_to_bf16_bits
from autograd_b200.storage import CudaAllocator, CudaMemPointer, Storage, address_of
from oracle import fused_layers as O


def _header_symbols():
    text = open(os.path.join(ROOT, "include", "autograd_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ag_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_native.LIB_PATH)
    names = _header_symbols()
    assert len(names) >= 35
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    # and the ctypes table covers the header one to one
    assert sorted(_native.SIGNATURES) == names


def test_pybind11_module_covers_the_header_and_agrees_with_ctypes():
    """The pybind11 form of the binding (csrc/cuda_ext.cpp, the shape of the reference's metal_ext
    module) exposes every declared entry point; its adapter takes the same ctypes-typed arguments as
    the ctypes library object.  Host-only entry points are called through both."""
    from autograd_b200 import build as agbuild
    if agbuild.build_pybind() is None:
        pytest.skip("pybind11 or the Python headers are not installed")
    from autograd_b200 import cuda_ext
    names = _header_symbols()
    for n in names:
        assert hasattr(cuda_ext, n), f"{n} declared in the header but not bound by cuda_ext"
    pyb = _native._PybindLibrary(cuda_ext)
    cdll = _native.load_library()
    desc = _native.FlceDesc(16384, 1280, 32768, 4096, _native.AG_CE_3XTF32, 0, 0)
    assert pyb.ag_flce_scratch_bytes(ctypes.byref(desc)) == cdll.ag_flce_scratch_bytes(ctypes.byref(desc)) > 0
    assert pyb.ag_scatter_add_scratch_bytes(65536, 1536, 151936) == cdll.ag_scatter_add_scratch_bytes(65536, 1536, 151936)
    assert pyb.ag_linear_add_scratch_bytes(16384, 1280, 1280, 1) == cdll.ag_linear_add_scratch_bytes(16384, 1280, 1280, 1)
    # a failing call reports through the same channel: no device here, or an invalid one
    h = ctypes.c_void_p()
    rc = pyb.ag_ctx_create(4096, None, ctypes.byref(h))
    assert rc != 0 and h.value is None
    assert isinstance(pyb.ag_last_error(None), bytes) and pyb.ag_last_error(None)
    with pytest.raises(TypeError):
        pyb.ag_synchronize()


def test_context_creation_fails_loudly_without_gpu():
    """No CPU fallback: without a CUDA device the product path raises."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(ag.AgError):
        ag.create(0)


class FakeContext:
    """Records the C-ABI calls the backend would make; hands out fake addresses."""

    def __init__(self):
        self.calls = []
        self.kwargs = []          # keyword arguments of the recorded calls, same order
        self._next = 0x10000000
        self.sm_count = 148

    def alloc(self, nbytes):
        a = self._next
        self._next += (int(nbytes) + 255) // 256 * 256
        return a

    def free(self, addr):
        self.calls.append(("free", addr))
        self.kwargs.append({})

    def norm_partials_bytes(self, c):
        return 148 * 8 * 2 * c * 4

    @staticmethod
    def scatter_add_scratch_bytes(n, c, v):
        return 4096 + n * 16

    @staticmethod
    def flce_desc(n, c, v, **kw):
        return types.SimpleNamespace(N=n, C=c, V=v, **kw)

    @staticmethod
    def flce_scratch_bytes(desc):
        return 1 << 20

    def __getattr__(self, name):
        def rec(*args, **kw):
            self.calls.append((name,) + args)
            self.kwargs.append(kw)
        return rec


def _fake_env():
    ctx = FakeContext()
    alloc = CudaAllocator(ctx)
    be = CudaBackend(ctx, alloc)
    alloc.backend = be
    return ctx, alloc, be


def _t(alloc, shape, dtype=np.float32, requires_grad=True, grad=False):
    t = hg.HostTensor(shape, dtype, requires_grad=requires_grad)
    t.storage = alloc.alloc(shape, dtype)
    if grad:
        t.grad = hg.HostTensor(shape, dtype, requires_grad=False)
        t.grad.storage = alloc.alloc(shape, dtype)
    return t


def test_allocator_views_are_pointer_arithmetic():
    ctx, alloc, be = _fake_env()
    arena = alloc.empty((4096,), np.uint8)
    v = alloc.view(arena, 256, (8, 4), np.float32)
    assert isinstance(v, Storage) and isinstance(v.ptr, CudaMemPointer)
    assert v.ptr.buffer_id == arena.ptr.buffer_id and v.ptr.offset == 256 and v.nbytes == 128
    assert address_of(v) == address_of(arena) + 256
    v2 = alloc.view(v, 64, (4,), np.float32)          # view of a view keeps the base id
    assert v2.ptr.buffer_id == arena.ptr.buffer_id and v2.ptr.offset == 320
    with pytest.raises(RuntimeError, match="View overflow"):
        alloc.view(arena, 4000, (64,), np.float32)
    assert getattr(arena.ptr, "buffer_id", None) is not None   # runtime.py:461 reads this
    assert not hasattr(alloc, "ctx") and not hasattr(be, "ctx") and not hasattr(be, "numpy_view")


def test_kernel_lookup_is_by_op_class_name():
    ctx, alloc, be = _fake_env()
    for name in ("LayerNormOp", "GELUOp", "GatherOp", "FusedLinearCrossEntropyOp", "FusedRMSNormLinearCrossEntropyOp"):
        assert callable(be.get_forward_kernel(hg.make_op(name)))
        assert callable(be.get_backward_kernel(hg.make_op(name)))
    assert be.get_forward_kernel(hg.make_op("SoftmaxOp")) is None     # as backend.py:2562-2574
    assert be.get_backward_kernel(hg.make_op("MatMulOp")) is None
    with pytest.raises(NotImplementedError):
        be.bind_matmul_forward(None)


def test_layernorm_backward_marshalling_accumulates_in_place():
    ctx, alloc, be = _fake_env()
    x, g, b = _t(alloc, (2, 3, 8), grad=True), _t(alloc, (8,), grad=True), _t(alloc, (8,), grad=True)
    y = _t(alloc, (2, 3, 8), grad=True)
    n = hg.make_node(hg.make_op("LayerNormOp", eps=1e-5, normalized_dim=-1), (x, g, b), (y,))
    be.get_backward_kernel(n.op)(n.inputs, n.outputs)
    call = [c for c in ctx.calls if c[0] == "layernorm_backward"][0]
    _, dy, xa, ga, dres, dx, dgam, dbet, part, part_bytes, N, C, eps = call
    assert (N, C) == (6, 8) and eps == 1e-5
    assert dy == address_of(y.grad.storage) and xa == address_of(x.storage)
    assert dres == dx == address_of(x.grad.storage)              # fused residual-gradient add
    assert dgam == address_of(g.grad.storage) and dbet == address_of(b.grad.storage)
    assert part_bytes >= ctx.norm_partials_bytes(8)
    # no upstream gradient: nothing is launched (backend.py:438-439)
    ctx.calls.clear()
    y.grad = None
    be.get_backward_kernel(n.op)(n.inputs, n.outputs)
    assert not ctx.calls
    # a frozen gamma gets no gradient pointer
    y.grad = _t(alloc, (2, 3, 8))
    g.requires_grad = False
    be.get_backward_kernel(n.op)(n.inputs, n.outputs)
    assert [c for c in ctx.calls if c[0] == "layernorm_backward"][0][6] == 0


def test_add_binding_rejects_broadcast_like_the_metal_backend():
    ctx, alloc, be = _fake_env()
    a, b = _t(alloc, (4, 8)), _t(alloc, (8,))
    with pytest.raises(RuntimeError, match="Unsupported Add shape"):
        be.bind_add_forward(hg.make_node(hg.make_op("AddOp"), (a, b), (_t(alloc, (4, 8)),)))


def test_scratch_slots_are_preferred_over_the_workspace():
    ctx, alloc, be = _fake_env()
    ids, tab = _t(alloc, (2, 16), np.int32, requires_grad=False), _t(alloc, (50, 32), grad=True)
    out = _t(alloc, (2, 16, 32), grad=True)
    n = hg.make_node(hg.make_op("GatherOp"), (ids, tab), (out,))
    slot = alloc.alloc((8192,), np.uint8)
    be.get_backward_kernel(n.op)(n.inputs, n.outputs, scratch={"scatter": slot})
    call = [c for c in ctx.calls if c[0] == "gather_backward"][0]
    assert call[4] == address_of(slot) and call[5] == 8192 and call[6:] == (32, 32, 50)
    ctx.calls.clear()
    be.get_backward_kernel(n.op)(n.inputs, n.outputs)            # no scratch: backend workspace
    call = [c for c in ctx.calls if c[0] == "gather_backward"][0]
    assert call[4] != address_of(slot) and call[5] >= ctx.scatter_add_scratch_bytes(32, 32, 50)


def test_bf16_gradient_storage_goes_through_fp32_staging():
    """A parameter whose gradient storage is uint16 (bf16 words, the reference's grad_dtype="bf16"): the
    kernel accumulates into a zeroed fp32 staging area, then one f32_to_bf16(accumulate) adds it into the
    stored gradient; the gather backward and AdamW switch to their bf16-gradient entry points."""
    ctx, alloc, be = _fake_env()
    x, g, b = _t(alloc, (2, 3, 8), grad=True), _t(alloc, (8,)), _t(alloc, (8,), grad=True)
    g.grad = hg.HostTensor((8,), np.uint16, requires_grad=False)
    g.grad.storage = alloc.alloc((8,), np.uint16)
    y = _t(alloc, (2, 3, 8), grad=True)
    n = hg.make_node(hg.make_op("LayerNormOp", eps=1e-5, normalized_dim=-1), (x, g, b), (y,))
    be.get_backward_kernel(n.op)(n.inputs, n.outputs)
    names = [c[0] for c in ctx.calls]
    assert names.index("fill_f32") < names.index("layernorm_backward") < names.index("f32_to_bf16")
    ln = [c for c in ctx.calls if c[0] == "layernorm_backward"][0]
    conv = [c for c in ctx.calls if c[0] == "f32_to_bf16"]
    assert len(conv) == 1                                         # beta keeps its fp32 storage
    stage = ln[6]
    assert stage not in (0, address_of(g.grad.storage)) and ln[7] == address_of(b.grad.storage)
    assert conv[0][1:4] == (stage, address_of(g.grad.storage), 8)
    assert ctx.kwargs[[c[0] for c in ctx.calls].index("f32_to_bf16")] == {"accumulate": True}
    fill = [c for c in ctx.calls if c[0] == "fill_f32"][0]
    assert fill[1] == stage and fill[2] == 0.0

    ctx.calls.clear()
    ctx.kwargs.clear()
    ids, tab = _t(alloc, (2, 16), np.int32, requires_grad=False), _t(alloc, (50, 32))
    tab.grad = hg.HostTensor((50, 32), np.uint16, requires_grad=False)
    tab.grad.storage = alloc.alloc((50, 32), np.uint16)
    out = _t(alloc, (2, 16, 32), grad=True)
    gn = hg.make_node(hg.make_op("GatherOp"), (ids, tab), (out,))
    be.get_backward_kernel(gn.op)(gn.inputs, gn.outputs)
    assert [c[0] for c in ctx.calls if c[0].startswith("gather")] == ["gather_backward_bf16"]

    ctx.calls.clear()
    ctx.kwargs.clear()
    p, m, v = _t(alloc, (64,)), _t(alloc, (64,)), _t(alloc, (64,))
    be.adamw_step(p.storage, tab.grad.storage, m.storage, v.storage, None, 1e-3, 1e-3, 0.9, 0.95, 1e-8, 0.1)
    assert ctx.calls[-1][0] == "adamw_step" and ctx.kwargs[-1] == {"grad_bf16": True}


def test_bf16_host_conversion_matches_the_oracle(golden):
    g = golden("adamw_bf16")
    assert np.array_equal(f32_to_bf16_bits(g["bf16_in"]), g["bf16_bits"])
    a = np.random.default_rng(0).standard_normal(1000).astype(np.float32)
    assert np.array_equal(bf16_bits_to_f32(f32_to_bf16_bits(a)), O.round_to_bf16(a))


# ---------------------------------------------------------------------------------------
# registration into the real reference: its modules as copied to oracle/_ref by oracle/make_ref.py,
# or a checkout named by AUTOGRAD_REFERENCE
# ---------------------------------------------------------------------------------------
REFERENCE = os.environ.get("AUTOGRAD_REFERENCE") or os.path.join(ROOT, "oracle", "_ref")


@pytest.mark.skipif(not os.path.exists(os.path.join(REFERENCE, "runtime.py")), reason="no reference modules")
def test_registers_behind_the_reference_runtime_and_plans_scratch():
    import subprocess
    code = r'''
import sys, types
import numpy as np
sys.path.insert(0, %(root)r)
stub = types.ModuleType("metal_ext")
class MetalContext:
    def __init__(self, *a, **k): raise RuntimeError("no metal")
stub.MetalContext = MetalContext
sys.modules["metal_ext"] = stub
sys.path.insert(0, %(ref)r)
import device as ref_device, runtime as ref_runtime, scratch as ref_scratch
from tensor import Tensor
from op import LayerNormOp, AddOp, GELUOp
sys.path.insert(0, %(root)r + "/tests")
from test_host_cpu import FakeContext
from autograd_b200.backend import CudaBackend
from autograd_b200.storage import CudaAllocator
from autograd_b200 import device as agdev
from types import SimpleNamespace
ctx = FakeContext(); alloc = CudaAllocator(ctx); be = CudaBackend(ctx, alloc); alloc.backend = be
mods = SimpleNamespace(device=ref_device, runtime=ref_runtime, scratch=ref_scratch)
ref_device.Device._allocators["cuda"] = alloc
ref_device.Device._backends["cuda"] = be
agdev._hook_scratch(mods, be)
rt = ref_runtime.Runtime(device="cuda")
assert rt.backend is be and rt.allocator is alloc and rt.need_scratch is False
f = np.float32
x = Tensor((4, 6, 16), f, init_val=np.zeros((4, 6, 16), f), device="cuda")
r = Tensor((4, 6, 16), f, init_val=np.zeros((4, 6, 16), f), device="cuda")
g = Tensor((16,), f, init_val=np.ones(16, f), device="cuda")
b = Tensor((16,), f, init_val=np.zeros(16, f), device="cuda")
h = AddOp()(x, r)
y = GELUOp()(LayerNormOp(eps=1e-5)(h, g, b))
rt.loss = y
rt.build_topo(y)
rt.bind_memory()
ln = [n for n in rt.topo if type(n.op).__name__ == "LayerNormOp"][0]
assert set(ln.scratch_fwd_layout.slots) == {"mean", "rstd"} and "partials" in ln.scratch_bwd_layout.slots
assert "scratch" in ln.forward.keywords and "scratch" in ln.backward.keywords      # arena-resident scratch bound
assert agdev.fuse_add_layernorm(rt) == 1
ctx.calls.clear()
rt.forward()
names = [c[0] for c in ctx.calls]
assert names == ["add_layernorm_forward", "gelu_forward"], names               # the add ran inside the LN kernel
call = ctx.calls[0]
assert call[2] != 0 and call[5] != 0 and call[7] != 0 and call[8] != 0          # r, h, mean, rstd all passed
rt.zero_grad(); rt.backend.fill(y.grad, 1.0); ctx.calls.clear()
rt.backward_graph()
names = [c[0] for c in ctx.calls if c[0] not in ("fill_f32",)]
assert names == ["gelu_backward", "layernorm_backward", "add_backward"], names
print("REGISTRATION-OK")
''' % {"root": ROOT, "ref": REFERENCE}
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120)
    assert "REGISTRATION-OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


# ---------------------------------------------------------------------------------------
# data-parallel reducer, two gloo ranks on CPU
# ---------------------------------------------------------------------------------------
def _dp_worker(rank, world, port, out_q):
    import torch
    import torch.distributed as dist
    from autograd_b200 import dp
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(100)           # same full batch on every rank, each takes its row shard
        full_x = rng.standard_normal((10, 8)).astype(np.float32)
        full_dy = rng.standard_normal((10, 8)).astype(np.float32)
        gamma = np.ones(8, np.float32)
        lo, hi = dp.shard_rows(10, rank, world)
        z = np.zeros(8, np.float32)
        _, dg, db = O.layernorm_backward(full_x[lo:hi], gamma, full_dy[lo:hi], 1e-5, np.zeros((hi - lo, 8), np.float32), z, z)
        small = torch.from_numpy(np.concatenate([dg, db]).copy())
        big = torch.from_numpy(np.full(1000, float(rank + 1), np.float32))
        red = dp.GradAllReducer([small, big])
        assert red.world_size == world and abs(red.grad_scale - 1.0 / world) < 1e-12
        red.reduce()
        loss = red.mean_loss(torch.tensor([float(rank)]))
        # the large bucket once more in its bf16 transport form: half the bytes, values rounded to bf16
        big2 = torch.from_numpy(np.full(1000, 1.0 + 2.0 ** -10 + rank, np.float32))
        red2 = dp.GradAllReducer([big2], wires=[dp.Bf16Wire.for_tensors(big2)])
        assert red2.bytes_per_step == 2000
        red2.reduce()
        want = float(sum(float(torch.tensor(1.0 + 2.0 ** -10 + r).to(torch.bfloat16)) for r in range(world)))
        assert np.all(big2.numpy() == np.float32(want)), (big2[:4], want)
        _, dg_full, db_full = O.layernorm_backward(full_x, gamma, full_dy, 1e-5, np.zeros((10, 8), np.float32), z, z)
        ok = (np.allclose(small.numpy(), np.concatenate([dg_full, db_full]), rtol=1e-5, atol=1e-5)
              and np.all(big.numpy() == sum(range(1, world + 1))) and abs(float(loss) - (world - 1) / 2) < 1e-6)
        out_q.put((rank, bool(ok), lo, hi))
    finally:
        dist.destroy_process_group()


def test_grad_allreduce_two_gloo_ranks():
    import torch.multiprocessing as mp
    from autograd_b200 import dp
    assert [dp.shard_rows(10, r, 3) for r in range(3)] == [(0, 4), (4, 7), (7, 10)]
    ctxm = mp.get_context("spawn")
    q = ctxm.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctxm.Process(target=_dp_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert res == [(0, True, 0, 5), (1, True, 5, 10)], res


def test_rmsnorm_ce_scratch_slot_too_small_for_the_current_precision_is_an_error():
    """The arena slot of FusedRMSNormLinearCrossEntropyOp is sized at planning time from ce_precision /
    ce_vocab_chunk; a setting changed afterwards must not overrun it: the backend compares the real slot
    size with its current need, and hands the C side the bytes that are really left for the head."""
    class Ctx(FakeContext):
        @staticmethod
        def flce_scratch_bytes(desc):
            return (1 << 20) if desc.precision == _native.AG_CE_FP32 else (4 << 20)

    ctx = Ctx()
    alloc = CudaAllocator(ctx)
    be = CudaBackend(ctx, alloc)
    alloc.backend = be
    x, w, g = _t(alloc, (2, 8, 64), grad=True), _t(alloc, (100, 64), grad=True), _t(alloc, (64,), grad=True)
    y = _t(alloc, (2, 8), np.int32, requires_grad=False)
    loss = _t(alloc, (1,), grad=True)
    n = hg.make_node(hg.make_op("FusedRMSNormLinearCrossEntropyOp", eps=1e-6), (x, w, g, y), (loss,))
    be.ce_precision = _native.AG_CE_FP32
    _, z_bytes, part_bytes, flce_bytes = be._rms_flce_layout(16, 64, 100)
    planned = 2 * z_bytes + part_bytes + flce_bytes
    slot = alloc.alloc((planned,), np.uint8)
    be.get_forward_kernel(n.op)(n.inputs, n.outputs, scratch={"rms_flce": slot})          # as planned: fine
    call = [c for c in ctx.calls if c[0] == "flce_forward"][-1]
    assert call[-1] == flce_bytes and call[-2] == address_of(slot) + 2 * z_bytes + part_bytes
    be.ce_precision = _native.AG_CE_3XTF32                                                  # needs 4 MiB now
    with pytest.raises(RuntimeError, match="changed after the graph was planned"):
        be.get_forward_kernel(n.op)(n.inputs, n.outputs, scratch={"rms_flce": slot})
    with pytest.raises(RuntimeError, match="changed after the graph was planned"):
        be.get_backward_kernel(n.op)(n.inputs, n.outputs, scratch={"rms_flce": slot})
    # a larger slot than needed: the head is told what is really left, not the computed minimum
    be.ce_precision = _native.AG_CE_FP32
    big = alloc.alloc((planned + 4096,), np.uint8)
    be.get_forward_kernel(n.op)(n.inputs, n.outputs, scratch={"rms_flce": big})
    assert [c for c in ctx.calls if c[0] == "flce_forward"][-1][-1] == flce_bytes + 4096


def test_adamw_rejects_the_packed_buffer_arguments():
    ctx, alloc, be = _fake_env()
    p, g, m, v = (_t(alloc, (64,)) for _ in range(4))
    with pytest.raises(TypeError, match="packed-buffer"):
        be.adamw_step(p.storage, g.storage, m.storage, v.storage, None, 1e-3, 1e-3, 0.9, 0.95, 1e-8, 0.1,
                      numel=64, decay_numel=32, lr_bc1=1e-3, inv_sqrt_bc2=1.0)
    be.adamw_step(p.storage, g.storage, m.storage, v.storage, None, 1e-3, 1e-3, 0.9, 0.95, 1e-8, 0.1, grad_scale=0.5)
    assert ctx.calls[-1][0] == "adamw_step"


def test_lse_side_buffers_are_bounded_and_released():
    ctx, alloc, be = _fake_env()
    x, w = _t(alloc, (1, 8, 32), grad=True), _t(alloc, (50, 32), grad=True)
    y = _t(alloc, (1, 8), np.int32, requires_grad=False)
    losses = []
    for _ in range(be.MAX_SIDE_BUFFERS + 3):
        loss = _t(alloc, (1,), grad=True)
        n = hg.make_node(hg.make_op("FusedLinearCrossEntropyOp", ignore_index=-1), (x, w, y), (loss,))
        be.get_forward_kernel(n.op)(n.inputs, n.outputs)
        losses.append((loss, n))
    assert len(be._side) == be.MAX_SIDE_BUFFERS
    loss, n = losses[-1]
    be.get_backward_kernel(n.op)(n.inputs, n.outputs)                     # the newest graph still finds its lse
    with pytest.raises(RuntimeError, match="before forward"):            # the oldest was evicted
        be.get_backward_kernel(losses[0][1].op)(losses[0][1].inputs, losses[0][1].outputs)
    be.release_side_buffers()
    assert not be._side


def test_host_cost_of_the_backend_layer_per_step():
    """The benchmark's end-to-end arm drives the C ABI directly; a graph runtime goes through the backend's
    callables, which add Python work per call (shape arithmetic, gradient targets, scratch slots, the CE
    descriptor).  This replays the callable sequence of one fused-layer step of the depth-20 model on a
    recording context - 1 gather, 41 LayerNorm, 20 GELU, 1 fused linear + CE, forward and backward, plus the
    runtime's zero-fills - and bounds the host time: it has to stay far below the 67-69 ms the GPU needs for
    the step, so that launches stay ahead of the device."""
    import time
    ctx, alloc, be = _fake_env()
    B, T, C, V, L, I = 16, 2048, 1280, 32768, 20, 5120
    ids, tg = _t(alloc, (B, T), np.int32, requires_grad=False), _t(alloc, (B, T), np.int32, requires_grad=False)
    table = _t(alloc, (V, C), grad=True)
    x0 = _t(alloc, (B, T, C), grad=True)
    nodes = [hg.make_node(hg.make_op("GatherOp"), (ids, table), (x0,))]
    h = x0
    for _ in range(2 * L + 1):
        g, b, y = _t(alloc, (C,), grad=True), _t(alloc, (C,), grad=True), _t(alloc, (B, T, C), grad=True)
        nodes.append(hg.make_node(hg.make_op("LayerNormOp", eps=1e-5, normalized_dim=-1), (h, g, b), (y,)))
        h = y
    for _ in range(L):
        u, a = _t(alloc, (B, T, I), grad=True), _t(alloc, (B, T, I), grad=True)
        nodes.append(hg.make_node(hg.make_op("GELUOp"), (u,), (a,)))
    loss = _t(alloc, (1,), grad=True)
    nodes.append(hg.make_node(hg.make_op("FusedLinearCrossEntropyOp", ignore_index=-1), (h, table, tg), (loss,)))
    fwd = [be.get_forward_kernel(n.op) for n in nodes]
    bwd = [be.get_backward_kernel(n.op) for n in nodes]
    grads = [t.grad for n in nodes for t in n.inputs + n.outputs if t.grad is not None]

    def step():
        for g_ in grads:                       # the runtime's zero_grad / clear lists (runtime.py:828-854)
            be.fill(g_, 0.0)
        for n, f in zip(nodes, fwd):
            f(n.inputs, n.outputs)
        for n, f in zip(reversed(nodes), reversed(bwd)):
            f(n.inputs, n.outputs)

    step()
    ctx.calls.clear(); ctx.kwargs.clear()
    t0 = time.perf_counter()
    for _ in range(5):
        step()
    per_step_ms = 1e3 * (time.perf_counter() - t0) / 5
    launches = sum(1 for c in ctx.calls if c[0] not in ("free",)) / 5
    print(f"host time of the backend layer: {per_step_ms:.2f} ms per step for {launches:.0f} C-ABI calls")
    assert launches >= 2 * (1 + 41 + 20 + 1)
    assert per_step_ms < 20.0, per_step_ms


def test_bench_clock_summary_uses_the_samples_under_load():
    """bench.py's clock record: the median SM clock is taken over the nvidia-smi samples at which the GPU was
    busy (at least half utilisation), not over idle readings before and after the timed region; throttle reasons
    are collected over all samples."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("_bench_for_test", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)

    class Done:
        def terminate(self): pass
        def wait(self, timeout=None): return 0
        def kill(self): pass

    na = "Not Active"
    rows = [f"0, 1965, 1965, 180.0, 0x0, {na}, {na}, {na}, {na}, 0"] * 6            # idle before the step
    rows += [f"0, {mhz}, 1965, 990.0, 0x4, {na}, {na}, {na}, Active, 100" for mhz in (1545, 1560, 1590, 1605, 1620)]
    rows += [f"0, 1965, 1965, 200.0, 0x0, {na}, {na}, {na}, {na}, 3"] * 4            # idle during the CPU baseline
    s = bench.ClockSampler(0)
    with open(s.path, "w") as f:
        f.write("\n".join(rows) + "\n")
    s.out = open(s.path)          # stop() closes it
    s.proc = Done()
    got = s.stop()
    assert got["sm_mhz"] == 1590 and got["sm_max_mhz"] == 1965
    assert got["samples"] == 15 and got["samples_under_load"] == 5
    assert got["reasons"] == ["sw_power_cap"]
    assert not os.path.exists(s.path)
