"""Device storage and allocator for the `cuda` device, with the interface of the
reference's `Allocator` / `Storage` (storage.py:6-47) and the pointer convention of its
`MetalMemPointer` (storage.py:66-70): `ptr.buffer_id` is the base device address of the
allocation, `ptr.offset` a byte offset into it.  The allocator deliberately has no `ctx`
attribute: the reference runtime keys its Metal-only parameter packing on that name
(runtime.py:154-206).
"""
from __future__ import annotations

from math import prod

import numpy as np

DEVICE_NAME = "cuda"


class CudaMemPointer:
    __slots__ = ("buffer_id", "offset")

    def __init__(self, buffer_id: int, offset: int = 0):
        self.buffer_id = int(buffer_id)
        self.offset = int(offset)

    @property
    def address(self) -> int:
        return self.buffer_id + self.offset

    def __repr__(self):
        return f"CudaMemPointer(0x{self.buffer_id:x}+{self.offset})"


class Storage:
    """Same slots as the reference's Storage (storage.py:6-17)."""
    __slots__ = ("ptr", "shape", "dtype", "device", "nbytes")

    def __init__(self, ptr, shape, dtype, device, nbytes):
        self.ptr = ptr
        self.shape = tuple(shape)
        self.dtype = dtype
        self.device = device
        self.nbytes = nbytes

    @property
    def data(self):
        return self.ptr


def address_of(storage) -> int:
    """Device address of anything carrying a CudaMemPointer in `.ptr`."""
    return storage.ptr.buffer_id + storage.ptr.offset


class CudaAllocator:
    """alloc / view / empty / zeros / ones / free, as storage.py:19-47 and :72-90."""

    def __init__(self, context):
        self.device = DEVICE_NAME
        self._context = context
        self._live = {}  # base address -> nbytes
        self.backend = None  # set by register(); used by zeros/ones

    def alloc(self, shape, dtype=np.float32):
        nbytes = int(prod(shape)) * np.dtype(dtype).itemsize
        base = self._context.alloc(max(nbytes, 1))
        self._live[base] = nbytes
        return Storage(CudaMemPointer(base, 0), shape, dtype, self.device, nbytes)

    def empty(self, shape, dtype=np.float32):
        return self.alloc(shape, dtype)

    def zeros(self, shape, dtype=np.float32):
        s = self.alloc(shape, dtype)
        self.backend.fill_storage2(s, 0)
        return s

    def ones(self, shape, dtype=np.float32):
        s = self.alloc(shape, dtype)
        self.backend.fill_storage2(s, 1)
        return s

    def view(self, storage, offset_bytes, shape, dtype):
        nbytes = int(prod(shape)) * np.dtype(dtype).itemsize
        if offset_bytes + nbytes > storage.nbytes:
            # storage.py:59-60 raises the same way on the CPU
            raise RuntimeError(f"View overflow: {offset_bytes}+{nbytes}>{storage.nbytes}")
        ptr = CudaMemPointer(storage.ptr.buffer_id, storage.ptr.offset + int(offset_bytes))
        return Storage(ptr, shape, dtype, self.device, nbytes)

    def free(self, storage=None):
        """Free one allocation (by its base storage) or, with no argument, all of them."""
        if storage is not None:
            base = storage.ptr.buffer_id
            if self._live.pop(base, None) is not None:
                self._context.free(base)
            return
        for base in list(self._live):
            self._context.free(base)
        self._live.clear()

    @property
    def bytes_in_use(self):
        return sum(self._live.values())
