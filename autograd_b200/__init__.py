"""autograd_b200: a B200 (sm_100a) `cuda` device for autograd's fused layer kernels.

Importing the package loads `libautograd_b200.so` (the C ABI in include/autograd_b200.h);
there is no CPU or library fallback, a missing library is an ImportError.
"""
from . import _native
from ._native import (AG_BF16, AG_CE_3XTF32, AG_CE_BF16, AG_CE_BF16X3, AG_CE_FP32, AG_CE_IGNORE_COMPAT_UNMASKED,
                      AG_CE_IGNORE_MASKED, AG_CE_MEAN_ALL_ROWS, AG_CE_MEAN_VALID, AG_F32, AG_STATUS_BAD_INDEX,
                      AG_STATUS_STAGE_FALLBACK, AG_STATUS_WAIT_EXPIRED, AgError)
from .backend import CudaBackend
from .context import CudaContext
from .device import create, fuse_add_layernorm, register
from .storage import CudaAllocator, CudaMemPointer, Storage

__all__ = ["CudaBackend", "CudaContext", "CudaAllocator", "CudaMemPointer", "Storage", "create", "register",
           "fuse_add_layernorm", "AgError"]
