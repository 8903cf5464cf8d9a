"""Registration of the `cuda` device.

Stand-alone:   ctx, allocator, backend = autograd_b200.create(device=0)
With autograd: autograd_b200.register(device=0) seeds the reference's class-level registries
`Device._allocators["cuda"]` / `Device._backends["cuda"]`, which `Device.get_allocator` /
`Device.get_backend` consult before their built-in "cpu"/"mps" branches (device.py:11, :22),
so `Runtime(device="cuda")` (runtime.py:77-78) picks this backend up without any edit to the
reference.  It also gives the hot-path ops arena-resident scratch: the runtime only plans
scratch for ops listed in `runtime.METAL_SCRATCH_OPS` on non-CPU devices (runtime.py:16-17,
:309, :342) through the module-level `plan_node_scratch` (runtime.py:12, :244), so both are
extended in place.
"""
from __future__ import annotations

import sys

import numpy as np

from .backend import CudaBackend
from .context import CudaContext
from .storage import CudaAllocator, DEVICE_NAME

_CUDA_SCRATCH_OPS = ("LayerNormOp", "GatherOp", "FusedLinearCrossEntropyOp", "FusedRMSNormLinearCrossEntropyOp",
                     "FusedLinearAddOp")


def create(device: int = 0, stream: int | None = None):
    """A context, an allocator and a backend wired together."""
    ctx = CudaContext(device, stream)
    allocator = CudaAllocator(ctx)
    backend = CudaBackend(ctx, allocator)
    allocator.backend = backend
    return ctx, allocator, backend


def cuda_scratch_layouts(node, backend, pack_slots):
    """Scratch slots of one graph node on the cuda device as (forward, backward) layouts built
    with the runtime's own `pack_slots` (scratch.py:65-72); (None, None) for other ops."""
    from math import prod
    name = type(node.op).__name__
    ctx = backend.context
    u8 = np.uint8
    if name == "LayerNormOp":
        x = node.inputs[0]
        n, c = int(prod(x.shape[:-1])), int(x.shape[-1])
        fwd = pack_slots([("mean", (n,), np.float32), ("rstd", (n,), np.float32)], align=256)
        bwd = pack_slots([("partials", (ctx.norm_partials_bytes(c),), u8)], align=256)
        return fwd, bwd
    if name == "GatherOp":
        ids, table = node.inputs[0], node.inputs[1]
        nbytes = ctx.scatter_add_scratch_bytes(int(prod(ids.shape)), int(table.shape[1]), int(table.shape[0]))
        return None, pack_slots([("scatter", (nbytes,), u8)], align=256)
    if name == "FusedLinearCrossEntropyOp":
        x, w = node.inputs[0], node.inputs[1]
        n, c, v = int(prod(x.shape[:-1])), int(x.shape[-1]), int(w.shape[0])
        nbytes = ctx.flce_scratch_bytes(backend._flce_desc(n, c, v))
        return (pack_slots([("flce", (nbytes,), u8)], align=256), pack_slots([("flce", (nbytes,), u8)], align=256))
    if name == "FusedRMSNormLinearCrossEntropyOp":
        x, w = node.inputs[0], node.inputs[1]
        n, c, v = int(prod(x.shape[:-1])), int(x.shape[-1]), int(w.shape[0])
        _, z_bytes, part_bytes, flce_bytes = backend._rms_flce_layout(n, c, v)
        nbytes = 2 * z_bytes + part_bytes + flce_bytes
        return (pack_slots([("rms_flce", (nbytes,), u8)], align=256),
                pack_slots([("rms_flce", (nbytes,), u8)], align=256))
    if name == "FusedLinearAddOp":
        act, w = node.inputs[1], node.inputs[2]
        n, k, c = int(prod(act.shape[:-1])), int(act.shape[-1]), int(w.shape[1])
        nbytes = ctx.linear_add_scratch_bytes(n, k, c, backend._linear_precision())
        return (pack_slots([("linear_add", (nbytes,), u8)], align=256),
                pack_slots([("linear_add", (nbytes,), u8)], align=256))
    return None, None


def register(device: int = 0, stream: int | None = None, reference=None, existing=None):
    """Create the cuda device (or take `existing`, a (context, allocator, backend) triple from
    `create`) and, when the reference's modules are importable (or passed as `reference`, an object
    with attributes `device`, `runtime`, `scratch`), hook it into them.
    Returns (context, allocator, backend)."""
    ctx, allocator, backend = existing if existing is not None else create(device, stream)
    mods = reference
    if mods is None:
        mods = _find_reference_modules()
    if mods is not None:
        mods.device.Device._allocators[DEVICE_NAME] = allocator
        mods.device.Device._backends[DEVICE_NAME] = backend
        _hook_scratch(mods, backend)
    return ctx, allocator, backend


def _find_reference_modules():
    from types import SimpleNamespace
    try:
        import device as ref_device  # the reference is a flat set of top-level modules
        import runtime as ref_runtime
        import scratch as ref_scratch
    except Exception:
        return None
    if not hasattr(ref_device, "Device") or not hasattr(ref_runtime, "plan_node_scratch"):
        return None
    return SimpleNamespace(device=ref_device, runtime=ref_runtime, scratch=ref_scratch)


def _hook_scratch(mods, backend):
    rt = mods.runtime
    for op_name in _CUDA_SCRATCH_OPS:
        if op_name not in rt.METAL_SCRATCH_OPS:
            rt.METAL_SCRATCH_OPS.append(op_name)
    original = rt.plan_node_scratch
    if getattr(original, "_autograd_b200", False):
        original = original._original
    pack_slots = mods.scratch.pack_slots

    def plan_node_scratch(node, use_f16_gemm=False):
        dev = getattr(node.outputs[0], "device", None)
        if dev == DEVICE_NAME:
            fwd, bwd = cuda_scratch_layouts(node, backend, pack_slots)
            if fwd is not None or bwd is not None:
                return fwd, bwd
        return original(node, use_f16_gemm)

    plan_node_scratch._autograd_b200 = True
    plan_node_scratch._original = original
    rt.plan_node_scratch = plan_node_scratch


def fuse_add_layernorm(runtime):
    """Optional peephole over a compiled `Runtime`: an `Add` whose output feeds a `LayerNorm`
    that comes after it in topological order, with no other consumer in between, is executed
    by the fused kernel (h = x + r and y = LayerNorm(h) in one pass).  Returns the number of
    fused pairs.  Backward is unchanged: LayerNorm backward accumulates into h.grad and the
    Add backward distributes it."""
    backend = runtime.backend
    topo = list(runtime.topo)
    fused = 0
    for i, node in enumerate(topo):
        if type(node.op).__name__ != "AddOp" or len(node.outputs) != 1:
            continue
        h = node.outputs[0]
        x, r = node.inputs[0], node.inputs[1]
        if tuple(x.shape) != tuple(r.shape):
            continue
        first = next((m for m in topo[i + 1:] if h in m.inputs), None)
        if first is None or type(first.op).__name__ != "LayerNormOp" or first.inputs[0] is not h:
            continue
        ln = first
        eps = ln.op.eps
        if ln.op.normalized_dim not in (-1, len(h.shape) - 1):
            continue

        def fused_forward(inputs, outputs, scratch=None, _x=x, _r=r, _h=h, _eps=eps):
            mean = rstd = None
            if scratch is not None:
                mean, rstd = _View(scratch["mean"]), _View(scratch["rstd"])
            backend.fused_add_layernorm_forward(_x, _r, inputs[1], inputs[2], _h, outputs[0], _eps, mean, rstd)

        kw = getattr(ln.forward, "keywords", None) or {}
        if "scratch" in kw:
            import functools
            ln.forward = functools.partial(fused_forward, scratch=kw["scratch"])
        else:
            ln.forward = fused_forward
        node.forward = lambda inputs, outputs, scratch=None: None
        fused += 1
    return fused


class _View:
    """Adapter: a scratch Storage seen as a tensor-like object with `.storage`."""
    __slots__ = ("storage",)

    def __init__(self, storage):
        self.storage = storage
