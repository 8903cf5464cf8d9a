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

    def __init__(self, buckets, group=None):
        import torch.distributed as dist
        self._dist = dist
        self.group = group
        self.buckets = list(buckets)
        self.world_size = dist.get_world_size(group) if dist.is_initialized() else 1
        self.bytes_per_step = sum(int(b.numel()) * b.element_size() for b in self.buckets)

    @property
    def grad_scale(self) -> float:
        """Upstream gradient each rank feeds its local mean loss so that the summed
        gradients are those of the mean over the global batch."""
        return 1.0 / self.world_size

    def reduce(self):
        if self.world_size == 1:
            return
        for b in self.buckets:
            self._dist.all_reduce(b, op=self._dist.ReduceOp.SUM, group=self.group)

    def mean_loss(self, loss_tensor):
        """Global mean of the per-rank mean losses (equal token counts per rank)."""
        if self.world_size == 1:
            return loss_tensor
        self._dist.all_reduce(loss_tensor, op=self._dist.ReduceOp.SUM, group=self.group)
        loss_tensor /= self.world_size
        return loss_tensor


def shard_rows(n_rows: int, rank: int, world_size: int):
    """Contiguous row range [start, stop) of `rank`; the first n_rows % world_size ranks get
    one extra row."""
    base, extra = divmod(int(n_rows), int(world_size))
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)
