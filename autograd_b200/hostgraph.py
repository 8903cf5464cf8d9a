"""Minimal tensor / node objects with the attributes the kernel callables read
(`shape`, `dtype`, `requires_grad`, `grad`, `storage`, `op`), for driving the backend
without the reference's graph runtime: benchmarks, tests and stand-alone use.  The
reference does the same with namespace objects in its own checkers (debug/backend.py:25-36).
"""
from __future__ import annotations

from types import SimpleNamespace

import numpy as np


class HostTensor:
    __slots__ = ("shape", "dtype", "grad_dtype", "device", "requires_grad", "grad", "op", "init_val", "storage",
                 "name")

    def __init__(self, shape, dtype=np.float32, requires_grad=True, device="cuda", name=""):
        self.shape = tuple(shape)
        self.dtype = dtype
        self.grad_dtype = dtype
        self.device = device
        self.requires_grad = requires_grad
        self.grad = None
        self.op = None
        self.init_val = None
        self.storage = None
        self.name = name

    @property
    def ndim(self):
        return len(self.shape)


def make_op(class_name: str, **attrs):
    """An object whose class is called `class_name` (kernel lookup is by class name, as the
    reference keys its tables on the op class) carrying the given attributes."""
    cls = type(class_name, (), {"op_name": class_name[:-2] if class_name.endswith("Op") else class_name})
    op = cls()
    for k, v in attrs.items():
        setattr(op, k, v)
    return op


def make_node(op, inputs, outputs):
    node = SimpleNamespace(op=op, inputs=tuple(inputs), outputs=tuple(outputs), forward=None, backward=None,
                           scratch_fwd_layout=None, scratch_bwd_layout=None, name="")
    for o in outputs:
        o.op = node
    return node


def device_tensor(backend, allocator, array=None, shape=None, dtype=np.float32, requires_grad=True, with_grad=False,
                  name=""):
    """Allocate a HostTensor on the device, optionally initialised from `array` and with a
    zero-filled gradient tensor attached."""
    if array is not None:
        array = np.ascontiguousarray(array)
        shape, dtype = array.shape, array.dtype
    t = HostTensor(shape, dtype, requires_grad=requires_grad, name=name)
    t.storage = allocator.alloc(t.shape, t.dtype)
    if array is not None:
        backend.copy_from_host(t, array)
    if with_grad:
        g = HostTensor(t.shape, t.dtype, requires_grad=False, name=name + ".grad")
        g.storage = allocator.alloc(g.shape, g.dtype)
        backend.fill_storage2(g.storage, 0)
        t.grad = g
    return t
