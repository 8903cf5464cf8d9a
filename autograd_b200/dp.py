"""Token-row-sharded data parallelism: one process per GPU, every rank runs the fused-layer
kernels on its own rows, and the only exchange is an allreduce(sum) of the column
reductions - all dgamma/dbeta (one small contiguous bucket), the tied dW_vocab / embedding
gradient (one large bucket) - plus the scalar loss.  The reference is single-process
(train_autograd.py:341), so there is no reference behaviour to match beyond single-process
numerics; the mean over the global batch is obtained by running each rank's backward with
grad_scale = 1/world_size (the hook at runtime.py:89-95, :814) and summing.

`torch.distributed` is the plumbing: NCCL over NVLink on GPUs, gloo on CPU for tests.  No
kernel of this package reads another GPU's memory.
"""
from __future__ import annotations

import numpy as np


class DeviceArrayView:
    """A device address seen through `__cuda_array_interface__`, so that torch can alias it
    without a copy (torch.as_tensor(view, device="cuda"))."""

    def __init__(self, address: int, n_items: int, typestr: str = "<f4"):
        self.__cuda_array_interface__ = {
            "shape": (int(n_items),), "typestr": typestr, "data": (int(address), False), "version": 3, "strides": None,
        }


def as_torch(address: int, n_floats: int, device_index: int = 0):
    import torch
    return torch.as_tensor(DeviceArrayView(address, n_floats), device=torch.device("cuda", device_index))


class GradAllReducer:
    """Sums gradient buckets over the ranks of a process group.

    `buckets` is a list of 1-D tensors (torch CUDA tensors aliasing the backend's gradient
    buffers, or CPU tensors in tests).  reduce() launches one allreduce per bucket on the
    current stream of the backend (NCCL) and returns after enqueueing; gloo is synchronous.
    """

    def __init__(self, buckets, group=None, wires=None):
        """`wires`: optional list, one entry per bucket, each None or a `Bf16Wire`: that bucket then
        crosses the links as bf16 (half the bytes): packed before the allreduce, summed in bf16,
        widened back into the fp32 bucket afterwards.  The reference's counterpart is keeping the
        parameter gradients themselves as bf16 (grad_dtype="bf16", runtime.py:185-202)."""
        import torch.distributed as dist
        self._dist = dist
        self.group = group
        self.buckets = list(buckets)
        self.wires = list(wires) if wires is not None else [None] * len(self.buckets)
        if len(self.wires) != len(self.buckets):
            raise ValueError("one wire entry (or None) per bucket")
        self.world_size = dist.get_world_size(group) if dist.is_initialized() else 1
        self.bytes_per_step = sum(int(t.numel()) * t.element_size()
                                  for t in (w.tensor if w is not None else b for b, w in zip(self.buckets, self.wires)))

    @property
    def grad_scale(self) -> float:
        """Upstream gradient each rank feeds its local mean loss so that the summed
        gradients are those of the mean over the global batch."""
        return 1.0 / self.world_size

    def reduce(self, timer=None):
        """One allreduce(sum) per bucket.  `timer`: an optional `CommTimer`; each collective (with the
        pack / unpack of its wire form, if any) is then bracketed by a device-side event pair."""
        if self.world_size == 1:
            return
        for i, (b, w) in enumerate(zip(self.buckets, self.wires)):
            if timer is not None:
                timer.begin(f"bucket{i}")
            if w is None:
                self._dist.all_reduce(b, op=self._dist.ReduceOp.SUM, group=self.group)
            else:
                w.pack()
                self._dist.all_reduce(w.tensor, op=self._dist.ReduceOp.SUM, group=self.group)
                w.unpack()
            if timer is not None:
                timer.end()

    def mean_loss(self, loss_tensor):
        """Global mean of the per-rank mean losses (equal token counts per rank) by an allreduce of its
        own.  A caller that keeps the loss scalar inside one of the gradient buckets gets its sum from
        `reduce()` already and only divides by `world_size`."""
        if self.world_size == 1:
            return loss_tensor
        self._dist.all_reduce(loss_tensor, op=self._dist.ReduceOp.SUM, group=self.group)
        loss_tensor /= self.world_size
        return loss_tensor


class CommTimer:
    """Device-side timing of collectives: an event pair on the current CUDA stream around each one
    (the process group's own stream is ordered against it on both sides), summed per name."""

    def __init__(self):
        import torch
        self._torch = torch
        self._open = None
        self._pairs = []

    def begin(self, name):
        e0 = self._torch.cuda.Event(enable_timing=True)
        e0.record()
        self._open = (name, e0)

    def end(self):
        name, e0 = self._open
        e1 = self._torch.cuda.Event(enable_timing=True)
        e1.record()
        self._pairs.append((name, e0, e1))
        self._open = None

    def totals_ms(self):
        """name -> milliseconds summed over every bracketed collective; synchronises the device."""
        self._torch.cuda.synchronize()
        out = {}
        for name, e0, e1 in self._pairs:
            out[name] = out.get(name, 0.0) + float(e0.elapsed_time(e1))
        return out


class Bf16Wire:
    """bf16 transport form of one fp32 gradient bucket.

    `tensor` is what the allreduce sums (dtype torch.bfloat16); `pack()` rounds the fp32 bucket into
    it (to nearest even, utils.py:20-27) and `unpack()` widens the summed values back.  On a GPU
    both are this package's conversion kernels on the backend's stream (`for_device`); `for_tensors`
    is the host form with torch ops, for CPU process groups."""

    def __init__(self, tensor, pack, unpack):
        self.tensor, self.pack, self.unpack = tensor, pack, unpack

    @classmethod
    def for_device(cls, ctx, allocator, address: int, n_floats: int, device_index: int = 0):
        import torch
        bits = allocator.alloc((int(n_floats),), np.uint16)
        bits_addr = bits.ptr.address
        t = torch.as_tensor(DeviceArrayView(bits_addr, n_floats, "<i2"),
                            device=torch.device("cuda", device_index)).view(torch.bfloat16)
        wire = cls(t, lambda: ctx.f32_to_bf16(address, bits_addr, n_floats, accumulate=False),
                   lambda: ctx.bf16_to_f32(bits_addr, address, n_floats))
        wire.storage = bits  # keeps the device buffer alive
        return wire

    @classmethod
    def for_tensors(cls, bucket):
        import torch
        t = torch.empty(bucket.shape, dtype=torch.bfloat16, device=bucket.device)
        return cls(t, lambda: t.copy_(bucket), lambda: bucket.copy_(t))


def shard_rows(n_rows: int, rank: int, world_size: int):
    """Contiguous row range [start, stop) of `rank`; the first n_rows % world_size ranks get
    one extra row."""
    base, extra = divmod(int(n_rows), int(world_size))
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)
