"""Helpers of the GPU parity tests: one device per session, upload/download of numpy arrays as
tensor-like objects, graph-node stand-ins for calling the backend's kernel callables exactly
the way the reference runtime does (fn(inputs, outputs, scratch=None))."""
import numpy as np

import autograd_b200 as ag
from autograd_b200 import hostgraph as hg

_ENV = None


def env():
    """(context, allocator, backend); creation failure is a test failure, never a skip."""
    global _ENV
    if _ENV is None:
        _ENV = ag.create(0)
    return _ENV


def up(array, requires_grad=True, grad=None, name=""):
    """numpy -> device tensor; grad: None (no grad tensor), 0 (zero-filled) or an array."""
    ctx, alloc, be = env()
    t = hg.device_tensor(be, alloc, array=np.ascontiguousarray(array), requires_grad=requires_grad, name=name)
    if grad is not None:
        g = hg.HostTensor(t.shape, t.dtype, requires_grad=False)
        g.storage = alloc.alloc(g.shape, g.dtype)
        if isinstance(grad, np.ndarray):
            be.copy_from_host(g, grad)
        else:
            be.fill_storage2(g.storage, 0)
        t.grad = g
    return t


def empty(shape, dtype=np.float32, requires_grad=True, grad=None):
    ctx, alloc, be = env()
    t = hg.HostTensor(shape, dtype, requires_grad=requires_grad)
    t.storage = alloc.alloc(t.shape, t.dtype)
    if grad is not None:
        g = hg.HostTensor(t.shape, t.dtype, requires_grad=False)
        g.storage = alloc.alloc(g.shape, g.dtype)
        if isinstance(grad, np.ndarray):
            be.copy_from_host(g, grad)
        else:
            be.fill_storage2(g.storage, 0)
        t.grad = g
    return t


def down(t):
    ctx, alloc, be = env()
    return be.copy_to_host(t)


def free(*tensors):
    ctx, alloc, be = env()
    ctx.synchronize()
    for t in tensors:
        if t is None:
            continue
        if t.grad is not None and t.grad.storage is not None:
            alloc.free(t.grad.storage)
        if t.storage is not None:
            alloc.free(t.storage)


def node(op_name, inputs, outputs, **attrs):
    return hg.make_node(hg.make_op(op_name, **attrs), inputs, outputs)


def run_forward(n):
    ctx, alloc, be = env()
    fn = be.get_forward_kernel(n.op)
    assert fn is not None, type(n.op).__name__
    fn(n.inputs, n.outputs)


def run_backward(n):
    ctx, alloc, be = env()
    fn = be.get_backward_kernel(n.op)
    assert fn is not None, type(n.op).__name__
    fn(n.inputs, n.outputs)


def check_clean_status():
    ctx, _, _ = env()
    assert ctx.status() == 0


def bf16_grad(t, bits):
    """Attach to t a gradient stored as bf16 bit patterns (uint16), preloaded with `bits`."""
    ctx, alloc, be = env()
    g = hg.HostTensor(t.shape, np.uint16, requires_grad=False)
    g.storage = alloc.alloc(g.shape, np.uint16)
    be.copy_from_host(g, np.ascontiguousarray(bits, dtype=np.uint16))
    t.grad = g
    return g


def down_bits(t):
    """The raw 16-bit words of a bf16-stored tensor."""
    ctx, alloc, be = env()
    return ctx.copy_to_host(t.storage.ptr.address, tuple(t.shape), np.uint16)
