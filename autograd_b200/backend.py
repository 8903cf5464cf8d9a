"""`CudaBackend`: the kernel table of the `cuda` device.

It has the interface of the reference's `Backend` (backend.py:22-69) as the reference's
runtime uses it: `get_forward_kernel(op)` / `get_backward_kernel(op)` return callables
`fn(inputs, outputs, scratch=None)` (bound at runtime.py:241-243, called at :806-853) or
`None` for ops this backend has no kernel for (backend.py:2562-2574 behaves the same);
`bind_add_forward/backward` and `bind_matmul_forward/backward` exist because every non-CPU
device is routed through them (runtime.py:248-255).  Kernels are looked up by the op's
class NAME, so the reference's op classes and stand-ins with the same names both work.

Backward kernels ACCUMULATE into `.grad` buffers: a non-"mps" device takes the runtime
branch that zero-fills gradients itself (runtime.py:812-816, :844-854).

Two things are deliberately absent: `numpy_view` (device memory is not host addressable;
callers fall back to `copy_to_host`, runtime.py:118-121) and an attribute named `ctx`
(the reference's optimizer and runtime treat it as "this is Metal", optimizer.py:78).
"""
from __future__ import annotations

from math import prod

import numpy as np

from . import _native as N
from .storage import Storage, CudaMemPointer, address_of


def _addr(t):
    return 0 if t is None or t.storage is None else address_of(t.storage)


def _ag_dtype(dtype):
    dt = np.dtype(dtype)
    if dt == np.dtype(np.float32):
        return N.AG_F32
    if dt == np.dtype(np.uint16):
        return N.AG_BF16  # bf16 bit patterns, the reference's convention (utils.py:20-27)
    raise TypeError(f"unsupported activation dtype {dt}")


def f32_to_bf16_bits(a):
    """Round-to-nearest-even fp32 -> bf16 bit patterns, NaN kept quiet (utils.py:20-27)."""
    u = np.uint64
    bits = np.atleast_1d(np.ascontiguousarray(a, dtype=np.float32)).view(np.uint32).astype(u)
    rounded = (bits + u(0x7FFF) + ((bits >> u(16)) & u(1))) >> u(16)
    special = (bits & u(0x7F800000)) == u(0x7F800000)
    nan = special & ((bits & u(0x007FFFFF)) != u(0))
    special_bits = (bits >> u(16)) | np.where(nan, u(0x0040), u(0))
    return np.where(special, special_bits, rounded).astype(np.uint16).reshape(np.shape(a))


def bf16_bits_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


class CudaBackend:
    mixed_precision = False

    def __init__(self, context, allocator):
        self._context = context
        self._allocator = allocator
        # attributes the runtime writes (runtime.py:84, :93-95)
        self.use_fp16_gemm = False
        self.accumulate_parameter_grads = False
        self.grad_scale = 1.0
        # knobs of the fused linear + CE head
        self.ce_precision = N.AG_CE_3XTF32
        self.ce_vocab_chunk = 4096
        self.ce_reduction = N.AG_CE_MEAN_ALL_ROWS
        self.ce_ignore_mode = N.AG_CE_IGNORE_MASKED
        self._workspace = None       # grow-only scratch for calls that arrive without arena scratch
        self._grad_stage = None      # grow-only fp32 staging of gradients whose storage is bf16
        self._side = {}              # id(loss tensor) -> (loss tensor, Storage holding lse), forward -> backward
        self._forward = {
            "LayerNormOp": self._layernorm_forward,
            "GELUOp": self._gelu_forward,
            "GatherOp": self._gather_forward,
            "FusedLinearCrossEntropyOp": self._flce_forward,
            "FusedRMSNormLinearCrossEntropyOp": self._rms_flce_forward,
            "FusedLinearAddOp": self._linear_add_forward,
        }
        self._backward = {
            "LayerNormOp": self._layernorm_backward,
            "GELUOp": self._gelu_backward,
            "GatherOp": self._gather_backward,
            "FusedLinearCrossEntropyOp": self._flce_backward,
            "FusedRMSNormLinearCrossEntropyOp": self._rms_flce_backward,
            "FusedLinearAddOp": self._linear_add_backward,
        }

    # ------------------------------------------------------------------ Backend interface
    @property
    def context(self):
        return self._context

    def get_forward_kernel(self, op):
        return self._forward.get(type(op).__name__)

    def get_backward_kernel(self, op):
        return self._backward.get(type(op).__name__)

    def fill_storage(self, storage, value):
        self.fill_storage2(storage, value)

    def fill_storage2(self, storage, value):
        dt = np.dtype(storage.dtype)
        n = int(prod(storage.shape))
        addr = address_of(storage)
        if dt == np.dtype(np.float32):
            self._context.fill_f32(addr, float(value), n)
        elif dt == np.dtype(np.uint16):
            self._context.fill_pattern(addr, int(f32_to_bf16_bits(np.float32(value)).reshape(-1)[0]), 2, n)
        elif dt.kind in "iu" and dt.itemsize in (1, 2, 4):
            self._context.fill_pattern(addr, int(value) & 0xFFFFFFFF, dt.itemsize, n)
        else:
            raise TypeError(f"fill: unsupported dtype {dt}")

    def fill_scalar(self, tensor, value):
        self.fill_storage(tensor.storage, float(value))

    def fill(self, tensor, value):
        self.fill_scalar(tensor, float(value))

    def init(self, tensor):
        """backend.py:43-60"""
        v = tensor.init_val
        if v is None:
            return
        try:
            if isinstance(v, (int, float)):
                self.fill_scalar(tensor, float(v))
            elif isinstance(v, np.ndarray):
                self.copy_from_host(tensor, np.asarray(v, dtype=tensor.dtype))
            elif v == "xavier":
                # utils.py:68-71: despite the name, a normal with std sqrt(2/(fan_in+fan_out))
                fan_in, fan_out = tensor.shape[-2], tensor.shape[-1]
                std = np.sqrt(2.0 / (fan_in + fan_out))
                self.copy_from_host(tensor, np.random.normal(0, std, tensor.shape).astype(tensor.dtype))
            elif v == "zeros":
                self.fill_scalar(tensor, 0.0)
            else:
                raise ValueError(f"unknown init_val: {v!r}")
        finally:
            tensor.init_val = None

    def copy_from_host(self, tensor, host_np):
        st = tensor.storage
        if np.dtype(st.dtype) == np.dtype(np.uint16) and np.asarray(host_np).dtype != np.uint16:
            host = f32_to_bf16_bits(np.asarray(host_np, dtype=np.float32))
        else:
            host = np.ascontiguousarray(np.asarray(host_np, dtype=st.dtype))
        if host.size != int(prod(tensor.shape)):
            raise ValueError(f"copy_from_host: host has {host.size} elements, tensor {tensor.shape}")
        self._context.copy_from_host(address_of(st), host)

    def copy_to_host(self, tensor):
        st = tensor.storage
        out = self._context.copy_to_host(address_of(st), tuple(tensor.shape), st.dtype)
        if np.dtype(st.dtype) == np.dtype(np.uint16):
            return bf16_bits_to_f32(out).reshape(tuple(tensor.shape))
        return out

    def begin_pass(self):
        pass

    def end_pass(self):
        pass

    def synchronize(self):
        self._context.synchronize()

    def adamw_step(self, p_storage, g_storage, m_storage, v_storage, tmp_storage, lr, lr_t, b1, b2, eps,
                   weight_decay, grad_scale=1.0, **extra):
        # The packed-buffer form of the reference's Metal dispatch (optimizer.py:471-486) passes
        # numel, decay_numel, lr_bc1 and inv_sqrt_bc2, which change both the extent and the maths of
        # the step; that form is not implemented here, and dropping them would be a silently wrong step.
        unsupported = sorted(k for k in extra if k in ("numel", "decay_numel", "lr_bc1", "inv_sqrt_bc2"))
        if unsupported:
            raise TypeError(f"adamw_step: the packed-buffer arguments {unsupported} are not supported by the cuda backend")
        n = int(prod(p_storage.shape))
        grad_bf16 = np.dtype(g_storage.dtype) == np.dtype(np.uint16)  # backend.py:5128, :5139
        self._context.adamw_step(address_of(p_storage), address_of(g_storage), address_of(m_storage),
                                 address_of(v_storage), n, lr, lr_t, b1, b2, eps, weight_decay, grad_scale,
                                 grad_bf16=grad_bf16)

    # ------------------------------------------------------------------ Add / MatMul binding
    def bind_add_forward(self, node):
        x, y = node.inputs[0], node.inputs[1]
        if tuple(x.shape) != tuple(y.shape):
            # backend.py:5030-5033 rejects the same way on Metal
            raise RuntimeError(f"Unsupported Add shape: x.shape={x.shape}, y.shape={y.shape}")
        n = int(prod(x.shape))
        ctx = self._context

        def _fwd(inputs, outputs, scratch=None):
            ctx.add_forward(_addr(inputs[0]), _addr(inputs[1]), _addr(outputs[0]), n)
        return _fwd

    def bind_add_backward(self, node):
        x, y = node.inputs[0], node.inputs[1]
        if tuple(x.shape) != tuple(y.shape):
            raise RuntimeError(f"Unsupported Add shape: x.shape={x.shape}, y.shape={y.shape}")
        n = int(prod(x.shape))
        ctx = self._context

        def _bwd(inputs, outputs, scratch=None):
            out = outputs[0]
            if out.grad is None:
                return
            xg = _addr(inputs[0].grad) if inputs[0].requires_grad else 0
            yg = _addr(inputs[1].grad) if inputs[1].requires_grad else 0
            ctx.add_backward(_addr(out.grad), xg, yg, n)
        return _bwd

    def bind_matmul_forward(self, node):
        raise NotImplementedError("the cuda backend covers the fused layer kernels only; MatMulOp has no kernel")

    def bind_matmul_backward(self, node, scratch_views):
        raise NotImplementedError("the cuda backend covers the fused layer kernels only; MatMulOp has no kernel")

    # ------------------------------------------------------------------ workspace
    def workspace(self, nbytes):
        """Backend-owned scratch for calls that come without arena scratch.  Grow-only; a
        regrow waits for the stream before the old buffer is released."""
        nbytes = (int(nbytes) + 255) // 256 * 256
        if self._workspace is None or self._workspace.nbytes < nbytes:
            if self._workspace is not None:
                self._allocator.free(self._workspace)
            self._workspace = self._allocator.alloc((nbytes,), np.uint8)
        return self._workspace

    def _grad_targets(self, *params):
        """Where the kernels accumulate the gradients of `params`, and a function to call after them.

        fp32 gradient storage: the storage itself.  Gradient stored as bf16 bit patterns (uint16 storage,
        the reference's grad_dtype="bf16", runtime.py:185-202): a zeroed fp32 staging area; the returned
        function then adds it into the stored values with one rounding, the reference's
        fp32_to_bf16(accumulate) step after a gradient GEMM (backend.py:3298, :4743)."""
        addrs, staged, off = [], [], 0
        for t in params:
            if t is None or not t.requires_grad or t.grad is None:
                addrs.append(0)
            elif np.dtype(t.grad.storage.dtype) != np.dtype(np.uint16):
                addrs.append(_addr(t.grad))
            else:
                n = int(prod(t.shape))
                staged.append((len(addrs), off, n))
                addrs.append(None)
                off += (n * 4 + 255) // 256 * 256
        if not staged:
            return addrs, lambda: None
        stage = self._grad_stage
        if stage is None or stage.nbytes < off:
            if stage is not None:
                self._allocator.free(stage)
            stage = self._grad_stage = self._allocator.alloc((off,), np.uint8)
        base = address_of(stage)
        self._context.fill_f32(base, 0.0, off // 4)
        for i, o, _n in staged:
            addrs[i] = base + o

        def flush():
            for i, o, n in staged:
                self._context.f32_to_bf16(base + o, _addr(params[i].grad), n, accumulate=True)

        return addrs, flush

    def _slot(self, scratch, name, nbytes):
        """Address and size of scratch[name] if the runtime planned it, else of the workspace."""
        if scratch is not None:
            try:
                st = scratch[name]
                return address_of(st), st.nbytes
            except (KeyError, TypeError):
                pass
        ws = self.workspace(nbytes)
        return address_of(ws), ws.nbytes

    # ------------------------------------------------------------------ LayerNorm
    @staticmethod
    def _rows_cols(t):
        return int(prod(t.shape[:-1])), int(t.shape[-1])

    def _layernorm_forward(self, inputs, outputs, scratch=None):
        x, gamma, beta = inputs[0], inputs[1], inputs[2]
        out = outputs[0]
        op = out.op.op
        if op.normalized_dim not in (-1, len(x.shape) - 1):
            raise NotImplementedError("LayerNorm over a non-last axis")
        n, c = self._rows_cols(x)
        mean = rstd = 0
        if scratch is not None:
            try:
                mean, rstd = address_of(scratch["mean"]), address_of(scratch["rstd"])
            except (KeyError, TypeError):
                pass
        self._context.add_layernorm_forward(_addr(x), 0, _addr(gamma), _addr(beta), 0, _addr(out), mean, rstd, n, c,
                                            op.eps)

    def fused_add_layernorm_forward(self, x, r, gamma, beta, h, y, eps, mean=None, rstd=None):
        """h = x + r ; y = LayerNorm(h): the AddOp + LayerNormOp pair in one pass over HBM."""
        n, c = self._rows_cols(x)
        self._context.add_layernorm_forward(_addr(x), _addr(r), _addr(gamma), _addr(beta), _addr(h), _addr(y),
                                            _addr(mean), _addr(rstd), n, c, eps)

    def _layernorm_backward(self, inputs, outputs, scratch=None):
        x, gamma, beta = inputs[0], inputs[1], inputs[2]
        out = outputs[0]
        if out.grad is None:
            return
        op = out.op.op
        n, c = self._rows_cols(x)
        need = self._context.norm_partials_bytes(c)
        part, part_bytes = self._slot(scratch, "partials", need)
        dx = _addr(x.grad) if x.requires_grad else 0
        (dgamma, dbeta), flush = self._grad_targets(gamma, beta)
        self._context.layernorm_backward(_addr(out.grad), _addr(x), _addr(gamma), dx, dx, dgamma, dbeta, part,
                                         part_bytes, n, c, op.eps)
        flush()

    # ------------------------------------------------------------------ GELU
    def _gelu_forward(self, inputs, outputs, scratch=None):
        x, out = inputs[0], outputs[0]
        self._context.gelu_forward(_addr(x), _addr(out), int(prod(x.shape)))

    def _gelu_backward(self, inputs, outputs, scratch=None):
        x, out = inputs[0], outputs[0]
        if out.grad is None or not x.requires_grad:
            return
        self._context.gelu_backward(_addr(x), _addr(out.grad), _addr(x.grad), _addr(x.grad), int(prod(x.shape)))

    # ------------------------------------------------------------------ Gather
    def _gather_forward(self, inputs, outputs, scratch=None):
        ids, table = inputs[0], inputs[1]
        out = outputs[0]
        if np.dtype(ids.dtype) != np.dtype(np.int32):
            raise TypeError("Gather indices must be int32")
        v, c = table.shape
        self._context.gather_forward(_addr(ids), _addr(table), _addr(out), int(prod(ids.shape)), c, v)

    def _gather_backward(self, inputs, outputs, scratch=None):
        ids, table = inputs[0], inputs[1]
        out = outputs[0]
        if out.grad is None or not table.requires_grad:
            return
        v, c = table.shape
        n = int(prod(ids.shape))
        need = self._context.scatter_add_scratch_bytes(n, c, v)
        sc, sc_bytes = self._slot(scratch, "scatter", need)
        if np.dtype(table.grad.storage.dtype) == np.dtype(np.uint16):  # backend.py:2807-2812
            self._context.gather_backward_bf16(_addr(ids), _addr(out.grad), _addr(table.grad), sc, sc_bytes, n, c, v)
        else:
            self._context.gather_backward(_addr(ids), _addr(out.grad), _addr(table.grad), sc, sc_bytes, n, c, v)

    # ------------------------------------------------------------------ fused linear + CE
    def _flce_desc(self, n, c, v):
        return self._context.flce_desc(n, c, v, vocab_chunk=self.ce_vocab_chunk, precision=self.ce_precision,
                                       reduction=self.ce_reduction, ignore_mode=self.ce_ignore_mode)

    # The lse vector must survive from the head's forward to its backward, which the runtime's
    # scratch (one execution step) cannot give; it lives in a side buffer per loss tensor.  The
    # tensor classes have no weak references, so an entry holds its loss tensor (its id cannot be
    # reused while the entry exists) and the table is bounded: beyond MAX_SIDE_BUFFERS graphs the
    # least recently used entry is released.
    MAX_SIDE_BUFFERS = 8

    def _lse_buffer(self, out, n):
        key = id(out)
        ent = self._side.pop(key, None)
        st = ent[1] if ent is not None else None
        if st is None or st.nbytes < n * 4:
            if st is not None:
                self._context.synchronize()
                self._allocator.free(st)
            st = self._allocator.alloc((n,), np.float32)
        self._side[key] = (out, st)          # most recently used last
        while len(self._side) > self.MAX_SIDE_BUFFERS:
            _, old = self._side.pop(next(iter(self._side)))
            self._context.synchronize()
            self._allocator.free(old)
        return st

    def _lse_lookup(self, out):
        ent = self._side.get(id(out))
        return None if ent is None or ent[0] is not out else ent[1]

    def release_side_buffers(self):
        """Free every forward -> backward side buffer (call when the graphs that own them are dropped)."""
        self._context.synchronize()
        for _, st in self._side.values():
            self._allocator.free(st)
        self._side.clear()

    def _flce_forward(self, inputs, outputs, scratch=None):
        x, w, targets = inputs[0], inputs[1], inputs[2]
        row_scale = inputs[3] if len(inputs) > 3 else None
        out = outputs[0]
        n, c = self._rows_cols(x)
        v = w.shape[0]
        desc = self._flce_desc(n, c, v)
        need = self._context.flce_scratch_bytes(desc)
        sc, sc_bytes = self._slot(scratch, "flce", need)
        lse = self._lse_buffer(out, n)
        self._context.flce_forward(desc, _addr(x), _addr(w), _addr(targets), _addr(row_scale), _addr(out),
                                   address_of(lse), sc, sc_bytes)

    def _flce_backward(self, inputs, outputs, scratch=None):
        x, w, targets = inputs[0], inputs[1], inputs[2]
        row_scale = inputs[3] if len(inputs) > 3 else None
        out = outputs[0]
        if out.grad is None:
            return
        n, c = self._rows_cols(x)
        v = w.shape[0]
        desc = self._flce_desc(n, c, v)
        need = self._context.flce_scratch_bytes(desc)
        sc, sc_bytes = self._slot(scratch, "flce", need)
        lse = self._lse_lookup(out)
        if lse is None:
            raise RuntimeError("FusedLinearCrossEntropy backward called before forward")
        dx = _addr(x.grad) if x.requires_grad else 0
        (dw,), flush = self._grad_targets(w)
        self._context.flce_backward(desc, _addr(x), _addr(w), _addr(targets), _addr(row_scale), _addr(out.grad),
                                    address_of(lse), dx, dw, sc, sc_bytes)
        flush()

    # ------------------------------------------------------------------ linear + bias + residual
    def _linear_precision(self):
        # the projection GEMMs are tensor-core only; the exact-fp32 CE mode maps to 3xTF32 here
        return N.AG_CE_BF16 if self.ce_precision == N.AG_CE_BF16 else N.AG_CE_3XTF32

    def _linear_add_forward(self, inputs, outputs, scratch=None):
        """backend.py:2040-2058: out = act @ w + b + x (out may alias x)."""
        x, act, w, b = inputs
        out = outputs[0]
        n, k = self._rows_cols(act)
        c = w.shape[1]
        prec = self._linear_precision()
        sc, sc_bytes = self._slot(scratch, "linear_add", self._context.linear_add_scratch_bytes(n, k, c, prec))
        self._context.linear_add_forward(_addr(x), _addr(act), _addr(w), _addr(b), _addr(out), n, k, c, prec, sc,
                                         sc_bytes)

    def _linear_add_backward(self, inputs, outputs, scratch=None):
        """backend.py:2249-2259 (the branch whose `act` is still materialised)."""
        x, act, w, b = inputs
        out = outputs[0]
        if out.grad is None:
            return
        if w.requires_grad and act.op is not None and getattr(act.op.op, "op_name", "") == "FusedRMSNormGQA":
            raise NotImplementedError(
                "FusedLinearAdd backward after FusedRMSNormGQA recomputes the attention output on the reference "
                "CPU path (backend.py:2156-2245); attention is outside this backend")
        n, k = self._rows_cols(act)
        c = w.shape[1]
        prec = self._linear_precision()
        sc, sc_bytes = self._slot(scratch, "linear_add", self._context.linear_add_scratch_bytes(n, k, c, prec))
        (dw, db), flush = self._grad_targets(w, b)
        self._context.linear_add_backward(_addr(out.grad), _addr(act), _addr(w),
                                          _addr(x.grad) if x.requires_grad else 0,
                                          _addr(act.grad) if act.requires_grad else 0,
                                          dw, db, n, k, c, prec, sc, sc_bytes)
        flush()

    # ------------------------------------------------------------------ RMSNorm + linear + CE
    def _rms_flce_layout(self, n, c, v):
        desc = self._flce_desc(n, c, v)
        z_bytes = (n * c * 4 + 255) // 256 * 256
        part_bytes = (self._context.norm_partials_bytes(c) + 255) // 256 * 256
        flce_bytes = self._context.flce_scratch_bytes(desc)
        return desc, z_bytes, part_bytes, flce_bytes

    def _rms_flce_slot(self, scratch, n, c, v):
        """(desc, base, z_bytes, part_bytes, bytes left for the CE head) of the "rms_flce" slot.

        The slot was sized when the graph was planned, from ce_precision / ce_vocab_chunk as they
        were then; the head's need depends on both.  The size that is handed on is what really
        remains in the slot after z, dz and the partial rows, so that a setting changed after
        planning is caught here or by the C side's own size check instead of overrunning the arena."""
        desc, z_bytes, part_bytes, flce_bytes = self._rms_flce_layout(n, c, v)
        need = 2 * z_bytes + part_bytes + flce_bytes
        base, slot_bytes = self._slot(scratch, "rms_flce", need)
        if slot_bytes < need:
            raise RuntimeError(
                f"FusedRMSNormLinearCrossEntropy: the scratch slot has {slot_bytes} bytes but the current "
                f"ce_precision / ce_vocab_chunk need {need}; they were changed after the graph was planned")
        return desc, base, z_bytes, part_bytes, slot_bytes - (2 * z_bytes + part_bytes)

    def _rms_flce_forward(self, inputs, outputs, scratch=None):
        """backend.py:716-797: z = RMSNorm(x)*gamma, then the linear + CE head on z."""
        x, w, gamma, targets = inputs[:4]
        row_scale = inputs[4] if len(inputs) == 5 else None
        out = outputs[0]
        n, c = self._rows_cols(x)
        v = w.shape[0]
        desc, base, z_bytes, part_bytes, flce_bytes = self._rms_flce_slot(scratch, n, c, v)
        z = base
        self._context.rmsnorm_forward(_addr(x), _addr(gamma), z, 0, n, c, out.op.op.eps)
        lse = self._lse_buffer(out, n)
        self._context.flce_forward(desc, z, _addr(w), _addr(targets), _addr(row_scale), _addr(out), address_of(lse),
                                   base + 2 * z_bytes + part_bytes, flce_bytes)

    def _rms_flce_backward(self, inputs, outputs, scratch=None):
        """backend.py:799-886."""
        x, w, gamma, targets = inputs[:4]
        row_scale = inputs[4] if len(inputs) == 5 else None
        out = outputs[0]
        if out.grad is None:
            return
        n, c = self._rows_cols(x)
        v = w.shape[0]
        eps = out.op.op.eps
        desc, base, z_bytes, part_bytes, flce_bytes = self._rms_flce_slot(scratch, n, c, v)
        z, dz, part = base, base + z_bytes, base + 2 * z_bytes
        lse = self._lse_lookup(out)
        if lse is None:
            raise RuntimeError("FusedRMSNormLinearCrossEntropy backward called before forward")
        self._context.rmsnorm_forward(_addr(x), _addr(gamma), z, 0, n, c, eps)
        need_dz = x.requires_grad or gamma.requires_grad
        if need_dz:
            self._context.fill_f32(dz, 0.0, n * c)
        (dw, dg), flush = self._grad_targets(w, gamma)
        self._context.flce_backward(desc, z, _addr(w), _addr(targets), _addr(row_scale), _addr(out.grad),
                                    address_of(lse), dz if need_dz else 0, dw,
                                    base + 2 * z_bytes + part_bytes, flce_bytes)
        if need_dz:
            dx = _addr(x.grad) if x.requires_grad else 0
            self._context.rmsnorm_backward(dz, _addr(x), _addr(gamma), dx, dx, dg, part, part_bytes, n, c, eps)
        flush()

    # ------------------------------------------------------------------ stage kernels without a reference op
    # RMSNorm, SwiGLU and RoPE are stages inside the reference's fused ops (backend.py:1097-1126,
    # :1202-1251, :1382-1417); they are exposed here on tensors for callers that run the
    # surrounding GEMMs / attention themselves.
    def rmsnorm_forward(self, x, gamma, y, eps, inv_rms=None):
        n, c = self._rows_cols(x)
        self._context.rmsnorm_forward(_addr(x), _addr(gamma), _addr(y), _addr(inv_rms), n, c, eps,
                                      _ag_dtype(x.storage.dtype))

    def rmsnorm_backward(self, dz, x, gamma, eps, dx, dgamma=None, dres=None, scratch=None):
        """dx = (dres or 0) + local; pass dres=dx to accumulate in place."""
        n, c = self._rows_cols(x)
        part, part_bytes = self._slot(scratch, "partials", self._context.norm_partials_bytes(c))
        self._context.rmsnorm_backward(_addr(dz), _addr(x), _addr(gamma), _addr(dres), _addr(dx), _addr(dgamma), part,
                                       part_bytes, n, c, eps, _ag_dtype(x.storage.dtype))

    def swiglu_forward(self, gu, hidden):
        n, two_i = self._rows_cols(gu)
        self._context.swiglu_forward(_addr(gu), _addr(hidden), n, two_i // 2, _ag_dtype(gu.storage.dtype))

    def swiglu_backward(self, gu, dhidden):
        n, two_i = self._rows_cols(gu)
        self._context.swiglu_backward(_addr(gu), _addr(dhidden), n, two_i // 2, _ag_dtype(gu.storage.dtype))

    def rope_qk(self, q, k, cos, sin, sin_sign=1):
        b, t, h, d = q.shape
        hkv = k.shape[2] if k is not None else 0
        self._context.rope_qk(_addr(q), _addr(k), _addr(cos), _addr(sin), b, t, h, hkv, d, sin_sign=sin_sign,
                              dtype=_ag_dtype(q.storage.dtype))
