"""`CudaContext`: the Python face of one `ag_ctx` (device + stream), the counterpart of the
reference's `metal_ext.MetalContext` (metal_ext.mm:770-796).  Methods take raw device
addresses (ints) and sizes; they map one to one onto the C ABI.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _native as N
from ._native import lib


def _p(addr):
    """int / None -> c_void_p"""
    return C.c_void_p(int(addr)) if addr else C.c_void_p(0)


class CudaContext:
    def __init__(self, device: int = 0, stream: int | None = None):
        h = C.c_void_p()
        rc = lib.ag_ctx_create(int(device), _p(stream), C.byref(h))
        if rc != N.AG_OK:
            raise N.AgError(rc, (lib.ag_last_error(None) or b"").decode())
        self._h = h
        self.device = int(device)
        sm, l2, tot, maj, mnr = C.c_int(), C.c_int64(), C.c_int64(), C.c_int(), C.c_int()
        self._check(lib.ag_device_info(h, C.byref(sm), C.byref(l2), C.byref(tot), C.byref(maj), C.byref(mnr)))
        self.sm_count, self.l2_bytes, self.total_bytes = sm.value, l2.value, tot.value
        self.compute_capability = (maj.value, mnr.value)

    # ------------------------------------------------------------------ plumbing
    def _check(self, rc):
        if rc != N.AG_OK:
            raise N.AgError(rc, (lib.ag_last_error(self._h) or b"").decode())

    def close(self):
        if getattr(self, "_h", None):
            lib.ag_ctx_destroy(self._h)
            self._h = None

    def __del__(self):  # best effort
        try:
            self.close()
        except Exception:
            pass

    def set_stream(self, stream):
        self._check(lib.ag_set_stream(self._h, _p(stream)))

    def alloc(self, nbytes: int) -> int:
        out = C.c_void_p()
        self._check(lib.ag_alloc(self._h, int(nbytes), C.byref(out)))
        return int(out.value or 0)

    def free(self, addr: int):
        self._check(lib.ag_free(self._h, _p(addr)))

    def copy_from_host(self, dst_addr: int, host: np.ndarray):
        host = np.ascontiguousarray(host)
        self._check(lib.ag_copy_h2d(self._h, _p(dst_addr), host.ctypes.data_as(C.c_void_p), host.nbytes))

    def copy_to_host(self, src_addr: int, shape, dtype) -> np.ndarray:
        out = np.empty(shape, dtype=dtype)
        self._check(lib.ag_copy_d2h(self._h, out.ctypes.data_as(C.c_void_p), _p(src_addr), out.nbytes))
        return out

    def copy_h2d_raw(self, dst_addr: int, host_addr: int, nbytes: int):
        self._check(lib.ag_copy_h2d(self._h, _p(dst_addr), _p(host_addr), int(nbytes)))

    def copy_d2h_raw(self, host_addr: int, src_addr: int, nbytes: int):
        self._check(lib.ag_copy_d2h(self._h, _p(host_addr), _p(src_addr), int(nbytes)))

    def synchronize(self):
        self._check(lib.ag_synchronize(self._h))

    def status(self) -> int:
        f = C.c_int()
        self._check(lib.ag_status(self._h, C.byref(f)))
        return f.value

    def check_status(self):
        f = self.status()
        if f:
            names = [n for n, b in (("BAD_INDEX", 1), ("WAIT_EXPIRED", 2), ("STAGE_FALLBACK", 4)) if f & b]
            raise N.AgError(N.AG_ERR_DEVICE, "device status word: " + "|".join(names))

    @property
    def launch_count(self) -> int:
        return int(lib.ag_launch_count(self._h))

    def begin_pass_profiled(self):
        self._check(lib.ag_pass_begin_profiled(self._h))

    def end_pass_profiled(self) -> float:
        ms = C.c_float()
        self._check(lib.ag_pass_end_profiled(self._h, C.byref(ms)))
        return ms.value

    def event_record(self, index: int):
        self._check(lib.ag_event_record(self._h, int(index)))

    def event_elapsed_ms(self, start_index: int, end_index: int) -> float:
        ms = C.c_float()
        self._check(lib.ag_event_elapsed(self._h, int(start_index), int(end_index), C.byref(ms)))
        return ms.value

    def tc_timing(self, enable: bool, first_event_index: int = 0):
        """Bracket every tensor-core GEMM launch of the CE head with pool events (see the header)."""
        self._check(lib.ag_tc_timing(self._h, 1 if enable else 0, int(first_event_index)))

    def tc_timing_count(self) -> int:
        return int(lib.ag_tc_timing_count(self._h))

    def alloc_host(self, nbytes: int) -> int:
        out = C.c_void_p()
        self._check(lib.ag_alloc_host(self._h, int(nbytes), C.byref(out)))
        return int(out.value or 0)

    def free_host(self, addr: int):
        self._check(lib.ag_free_host(self._h, _p(addr)))

    # ------------------------------------------------------------------ kernels
    def fill_f32(self, dst, value, n):
        self._check(lib.ag_fill_f32(self._h, _p(dst), float(value), int(n)))

    def fill_pattern(self, dst, pattern, itemsize, n):
        self._check(lib.ag_fill_pattern(self._h, _p(dst), int(pattern) & 0xFFFFFFFF, int(itemsize), int(n)))

    def add_forward(self, x, y, out, n):
        self._check(lib.ag_add_forward(self._h, _p(x), _p(y), _p(out), int(n)))

    def add_backward(self, g, xgrad, ygrad, n):
        self._check(lib.ag_add_backward(self._h, _p(g), _p(xgrad), _p(ygrad), int(n)))

    def add_layernorm_forward(self, x, r, gamma, beta, h, y, mean, rstd, N_, C_, eps):
        self._check(lib.ag_add_layernorm_forward(self._h, _p(x), _p(r), _p(gamma), _p(beta), _p(h), _p(y), _p(mean),
                                                 _p(rstd), int(N_), int(C_), float(eps)))

    def norm_partials_bytes(self, C_):
        return int(lib.ag_norm_partials_bytes(self._h, int(C_)))

    def layernorm_backward(self, dy, x, gamma, dres, dx, dgamma, dbeta, partials, partials_bytes, N_, C_, eps):
        self._check(lib.ag_layernorm_backward(self._h, _p(dy), _p(x), _p(gamma), _p(dres), _p(dx), _p(dgamma),
                                              _p(dbeta), _p(partials), int(partials_bytes), int(N_), int(C_),
                                              float(eps)))

    def layernorm_backward_noalloc(self, dy, x, gamma, dres, dx, dgamma, dbeta, N_, C_, eps):
        """LayerNorm backward whose partial-sum workspace lives inside the library: for callers
        that cannot hand over (or allocate) scratch memory.  C_ <= 4096."""
        self._check(lib.ag_layernorm_backward_noalloc(self._h, _p(dy), _p(x), _p(gamma), _p(dres), _p(dx),
                                                      _p(dgamma), _p(dbeta), int(N_), int(C_), float(eps)))

    def debug_expire_staging(self):
        """Test hook: the next norm kernel gives up its staging wait at once (see the header)."""
        self._check(lib.ag_debug_expire_staging(self._h))

    def rmsnorm_forward(self, x, gamma, y, inv_rms, N_, C_, eps, dtype=N.AG_F32):
        self._check(lib.ag_rmsnorm_forward(self._h, _p(x), _p(gamma), _p(y), _p(inv_rms), int(N_), int(C_), float(eps),
                                           int(dtype)))

    def rmsnorm_backward(self, dz, x, gamma, dres, dx, dgamma, partials, partials_bytes, N_, C_, eps, dtype=N.AG_F32):
        self._check(lib.ag_rmsnorm_backward(self._h, _p(dz), _p(x), _p(gamma), _p(dres), _p(dx), _p(dgamma),
                                            _p(partials), int(partials_bytes), int(N_), int(C_), float(eps),
                                            int(dtype)))

    def gelu_forward(self, x, y, n):
        self._check(lib.ag_gelu_forward(self._h, _p(x), _p(y), int(n)))

    def gelu_backward(self, x, dy, dres, dx, n):
        self._check(lib.ag_gelu_backward(self._h, _p(x), _p(dy), _p(dres), _p(dx), int(n)))

    def swiglu_forward(self, gu, hidden, N_, I_, dtype=N.AG_F32):
        self._check(lib.ag_swiglu_forward(self._h, _p(gu), _p(hidden), int(N_), int(I_), int(dtype)))

    def swiglu_backward(self, gu, dhidden, N_, I_, dtype=N.AG_F32):
        self._check(lib.ag_swiglu_backward(self._h, _p(gu), _p(dhidden), int(N_), int(I_), int(dtype)))

    def rope_qk(self, q, k, cos, sin, B, T, H, HKV, D, q_token_stride=None, k_token_stride=None, sin_sign=1,
                dtype=N.AG_F32):
        qs = H * D if q_token_stride is None else q_token_stride
        ks = HKV * D if k_token_stride is None else k_token_stride
        self._check(lib.ag_rope_qk(self._h, _p(q), _p(k), _p(cos), _p(sin), int(B), int(T), int(H), int(HKV), int(D),
                                   int(qs), int(ks), int(sin_sign), int(dtype)))

    def gather_forward(self, ids, table, out, n_ids, C_, V_):
        self._check(lib.ag_gather_forward(self._h, _p(ids), _p(table), _p(out), int(n_ids), int(C_), int(V_)))

    @staticmethod
    def scatter_add_scratch_bytes(n_ids, C_, V_):
        return int(lib.ag_scatter_add_scratch_bytes(int(n_ids), int(C_), int(V_)))

    def gather_backward(self, ids, dout, dtable, scratch, scratch_bytes, n_ids, C_, V_):
        self._check(lib.ag_gather_backward(self._h, _p(ids), _p(dout), _p(dtable), _p(scratch), int(scratch_bytes),
                                           int(n_ids), int(C_), int(V_)))

    def gather_backward_bf16(self, ids, dout, dtable_bits, scratch, scratch_bytes, n_ids, C_, V_):
        """Table gradient kept as bf16 bit patterns: row = bf16(float(row) + fp32 sum of its dout rows)."""
        self._check(lib.ag_gather_backward_bf16(self._h, _p(ids), _p(dout), _p(dtable_bits), _p(scratch),
                                                int(scratch_bytes), int(n_ids), int(C_), int(V_)))

    def f32_to_bf16(self, src, dst_bits, n, accumulate=False):
        self._check(lib.ag_f32_to_bf16(self._h, _p(src), _p(dst_bits), int(n), 1 if accumulate else 0))

    def bf16_to_f32(self, src_bits, dst, n):
        self._check(lib.ag_bf16_to_f32(self._h, _p(src_bits), _p(dst), int(n)))

    @staticmethod
    def flce_desc(N_, C_, V_, vocab_chunk=4096, precision=N.AG_CE_3XTF32, reduction=N.AG_CE_MEAN_ALL_ROWS,
                  ignore_mode=N.AG_CE_IGNORE_MASKED):
        return N.FlceDesc(int(N_), int(C_), int(V_), int(vocab_chunk), int(precision), int(reduction),
                          int(ignore_mode))

    @staticmethod
    def flce_scratch_bytes(desc):
        return int(lib.ag_flce_scratch_bytes(C.byref(desc)))

    def flce_forward(self, desc, X, W, targets, row_scale, loss, lse, scratch, scratch_bytes):
        self._check(lib.ag_flce_forward(self._h, C.byref(desc), _p(X), _p(W), _p(targets), _p(row_scale), _p(loss),
                                        _p(lse), _p(scratch), int(scratch_bytes)))

    def flce_backward(self, desc, X, W, targets, row_scale, dloss, lse, dX, dW, scratch, scratch_bytes):
        self._check(lib.ag_flce_backward(self._h, C.byref(desc), _p(X), _p(W), _p(targets), _p(row_scale), _p(dloss),
                                         _p(lse), _p(dX), _p(dW), _p(scratch), int(scratch_bytes)))

    @staticmethod
    def linear_add_scratch_bytes(N_, K_, C_, precision=N.AG_CE_3XTF32):
        return int(lib.ag_linear_add_scratch_bytes(int(N_), int(K_), int(C_), int(precision)))

    def linear_add_forward(self, x, act, w, b, out, N_, K_, C_, precision, scratch, scratch_bytes):
        self._check(lib.ag_linear_add_forward(self._h, _p(x), _p(act), _p(w), _p(b), _p(out), int(N_), int(K_), int(C_),
                                              int(precision), _p(scratch), int(scratch_bytes)))

    def linear_add_backward(self, dout, act, w, dx, dact, dw, db, N_, K_, C_, precision, scratch, scratch_bytes):
        self._check(lib.ag_linear_add_backward(self._h, _p(dout), _p(act), _p(w), _p(dx), _p(dact), _p(dw), _p(db),
                                               int(N_), int(K_), int(C_), int(precision), _p(scratch),
                                               int(scratch_bytes)))

    def adamw_step(self, p, g, m, v, n, lr, lr_t, b1, b2, eps, weight_decay, grad_scale=1.0, grad_bf16=False):
        fn = lib.ag_adamw_step_bf16grad if grad_bf16 else lib.ag_adamw_step
        self._check(fn(self._h, _p(p), _p(g), _p(m), _p(v), int(n), float(lr), float(lr_t), float(b1), float(b2),
                       float(eps), float(weight_decay), float(grad_scale)))
