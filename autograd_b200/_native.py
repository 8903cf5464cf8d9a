"""ctypes binding of the C ABI declared in include/autograd_b200.h.

There is no fallback: if the shared library is missing or does not load, importing this
module raises, and every non-zero status code becomes a `RuntimeError` carrying the
library's own message.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libautograd_b200.so")

AG_OK, AG_ERR_INVALID, AG_ERR_CUDA, AG_ERR_SCRATCH, AG_ERR_DEVICE = range(5)
AG_F32, AG_BF16 = 0, 1
AG_STATUS_BAD_INDEX, AG_STATUS_WAIT_EXPIRED, AG_STATUS_STAGE_FALLBACK = 1, 2, 4
AG_CE_FP32, AG_CE_3XTF32, AG_CE_BF16, AG_CE_BF16X3 = 0, 1, 2, 3
AG_CE_MEAN_ALL_ROWS, AG_CE_MEAN_VALID = 0, 1
AG_CE_IGNORE_MASKED, AG_CE_IGNORE_COMPAT_UNMASKED = 0, 1


class FlceDesc(C.Structure):
    _fields_ = [("N", C.c_int64), ("C", C.c_int32), ("V", C.c_int32), ("vocab_chunk", C.c_int32),
                ("precision", C.c_int32), ("reduction", C.c_int32), ("ignore_mode", C.c_int32)]


_ctx = C.c_void_p
_ptr = C.c_void_p
_i64 = C.c_int64
_int = C.c_int
_f32 = C.c_float
_f64 = C.c_double
_sz = C.c_size_t

# name -> (restype, argtypes); mirrors include/autograd_b200.h one to one
SIGNATURES = {
    "ag_ctx_create": (_int, [_int, _ptr, C.POINTER(_ctx)]),
    "ag_ctx_destroy": (_int, [_ctx]),
    "ag_set_stream": (_int, [_ctx, _ptr]),
    "ag_last_error": (C.c_char_p, [_ctx]),
    "ag_device_info": (_int, [_ctx, C.POINTER(_int), C.POINTER(_i64), C.POINTER(_i64), C.POINTER(_int), C.POINTER(_int)]),
    "ag_alloc": (_int, [_ctx, _sz, C.POINTER(_ptr)]),
    "ag_free": (_int, [_ctx, _ptr]),
    "ag_copy_h2d": (_int, [_ctx, _ptr, _ptr, _sz]),
    "ag_copy_d2h": (_int, [_ctx, _ptr, _ptr, _sz]),
    "ag_synchronize": (_int, [_ctx]),
    "ag_status": (_int, [_ctx, C.POINTER(_int)]),
    "ag_launch_count": (_i64, [_ctx]),
    "ag_pass_begin_profiled": (_int, [_ctx]),
    "ag_pass_end_profiled": (_int, [_ctx, C.POINTER(_f32)]),
    "ag_event_record": (_int, [_ctx, _int]),
    "ag_event_elapsed": (_int, [_ctx, _int, _int, C.POINTER(_f32)]),
    "ag_tc_timing": (_int, [_ctx, _int, _int]),
    "ag_tc_timing_count": (_int, [_ctx]),
    "ag_alloc_host": (_int, [_ctx, _sz, C.POINTER(_ptr)]),
    "ag_free_host": (_int, [_ctx, _ptr]),
    "ag_fill_f32": (_int, [_ctx, _ptr, _f32, _i64]),
    "ag_fill_pattern": (_int, [_ctx, _ptr, C.c_uint32, _int, _i64]),
    "ag_add_forward": (_int, [_ctx, _ptr, _ptr, _ptr, _i64]),
    "ag_add_backward": (_int, [_ctx, _ptr, _ptr, _ptr, _i64]),
    "ag_add_layernorm_forward": (_int, [_ctx, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _int, _f32]),
    "ag_norm_partials_bytes": (_sz, [_ctx, _int]),
    "ag_layernorm_backward": (_int, [_ctx, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _sz, _i64, _int, _f32]),
    "ag_layernorm_backward_noalloc": (_int, [_ctx, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _int, _f32]),
    "ag_debug_expire_staging": (_int, [_ctx]),
    "ag_rmsnorm_forward": (_int, [_ctx, _ptr, _ptr, _ptr, _ptr, _i64, _int, _f32, _int]),
    "ag_rmsnorm_backward": (_int, [_ctx, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _sz, _i64, _int, _f32, _int]),
    "ag_gelu_forward": (_int, [_ctx, _ptr, _ptr, _i64]),
    "ag_gelu_backward": (_int, [_ctx, _ptr, _ptr, _ptr, _ptr, _i64]),
    "ag_swiglu_forward": (_int, [_ctx, _ptr, _ptr, _i64, _int, _int]),
    "ag_swiglu_backward": (_int, [_ctx, _ptr, _ptr, _i64, _int, _int]),
    "ag_rope_qk": (_int, [_ctx, _ptr, _ptr, _ptr, _ptr, _int, _int, _int, _int, _int, _i64, _i64, _int, _int]),
    "ag_gather_forward": (_int, [_ctx, _ptr, _ptr, _ptr, _i64, _int, _int]),
    "ag_scatter_add_scratch_bytes": (_sz, [_i64, _int, _int]),
    "ag_gather_backward": (_int, [_ctx, _ptr, _ptr, _ptr, _ptr, _sz, _i64, _int, _int]),
    "ag_flce_scratch_bytes": (_sz, [C.POINTER(FlceDesc)]),
    "ag_flce_forward": (_int, [_ctx, C.POINTER(FlceDesc), _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _sz]),
    "ag_flce_backward": (_int, [_ctx, C.POINTER(FlceDesc), _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _sz]),
    "ag_linear_add_scratch_bytes": (_sz, [_i64, _int, _int, _int]),
    "ag_linear_add_forward": (_int, [_ctx, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _int, _int, _int, _ptr, _sz]),
    "ag_linear_add_backward": (_int, [_ctx, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _int, _int, _int, _ptr, _sz]),
    "ag_adamw_step": (_int, [_ctx, _ptr, _ptr, _ptr, _ptr, _i64, _f64, _f64, _f64, _f64, _f64, _f64, _f64]),
    "ag_f32_to_bf16": (_int, [_ctx, _ptr, _ptr, _i64, _int]),
    "ag_bf16_to_f32": (_int, [_ctx, _ptr, _ptr, _i64]),
    "ag_gather_backward_bf16": (_int, [_ctx, _ptr, _ptr, _ptr, _ptr, _sz, _i64, _int, _int]),
    "ag_adamw_step_bf16grad": (_int, [_ctx, _ptr, _ptr, _ptr, _ptr, _i64, _f64, _f64, _f64, _f64, _f64, _f64, _f64]),
}


def load_library(path: str = LIB_PATH) -> C.CDLL:
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `python -m autograd_b200.build` (needs nvcc). "
            "autograd_b200 has no CPU or library fallback.")
    lib = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export it
        fn.restype = res
        fn.argtypes = args
    return lib


class _PybindLibrary:
    """The call surface of the ctypes library object over the pybind11 module `cuda_ext`
    (csrc/cuda_ext.cpp): `lib.ag_xxx(*args)` with the same ctypes-typed arguments.  Pointer
    arguments (c_void_p values, `byref(...)` out-parameters, ctypes structures, ints, None) become
    integer addresses, which is what the module takes; everything else is passed as a Python number."""

    def __init__(self, module):
        self._module = module
        for name, (res, argtypes) in SIGNATURES.items():
            setattr(self, name, self._adapt(getattr(module, name), argtypes))  # AttributeError if not exported

    @staticmethod
    def _address(a):
        if a is None:
            return 0
        if isinstance(a, int):
            return a
        if isinstance(a, C.c_void_p):
            return a.value or 0
        inner = getattr(a, "_obj", None)      # byref(x)
        if inner is not None:
            return C.addressof(inner)
        if isinstance(a, C._Pointer):
            return C.cast(a, C.c_void_p).value or 0
        return C.addressof(a)                 # a structure or a simple ctypes object passed by address

    @classmethod
    def _adapt(cls, fn, argtypes):
        is_ptr = [t is _ptr or t is _ctx or (isinstance(t, type) and issubclass(t, C._Pointer)) for t in argtypes]
        is_float = [t in (_f32, _f64) for t in argtypes]

        def call(*args):
            if len(args) != len(argtypes):
                raise TypeError(f"{fn.__name__} takes {len(argtypes)} arguments, got {len(args)}")
            conv = []
            for a, p, f in zip(args, is_ptr, is_float):
                if p:
                    conv.append(cls._address(a))
                else:
                    a = getattr(a, "value", a)
                    conv.append(float(a) if f else int(a))
            return fn(*conv)
        return call


def load_binding():
    """The library object the package calls: ctypes by default; AG_B200_BINDING=pybind11 selects the
    compiled pybind11 module (built by `python setup.py build_ext --inplace` / build.py where pybind11
    and the Python headers are present).  Either way the same libautograd_b200.so does the work."""
    which = os.environ.get("AG_B200_BINDING", "ctypes").lower()
    cdll = load_library()
    if which == "ctypes":
        return cdll, "ctypes"
    if which != "pybind11":
        raise ImportError(f"AG_B200_BINDING={which!r}: choose ctypes or pybind11")
    try:
        from . import cuda_ext
    except ImportError as e:
        raise ImportError(f"AG_B200_BINDING=pybind11 but autograd_b200.cuda_ext does not import ({e}); "
                          "build it with `python setup.py build_ext --inplace`") from e
    return _PybindLibrary(cuda_ext), "pybind11"


lib, BINDING = load_binding()


class AgError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"autograd_b200 error {code}: {message}")
        self.code = code
