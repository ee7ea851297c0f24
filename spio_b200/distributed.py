"""Data-parallel plumbing for the gw8 layer: batch sharding and the one exchange the path
needs, the sum of the per-rank weight gradients.

Forward and input gradient touch only a rank's own images; the weight gradient is a sum
over the batch, so each rank computes the partial over its shard and the partials are added
with one all-reduce (NCCL over NVLink on GPUs, gloo on CPU ranks in tests).  The reference
has no multi-device support to mirror; its only device awareness is keying the kernel cache
by device ordinal (spio/kernels/kernel_key.py:13-18).
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist


def shard_range(global_batch: int, world_size: int, rank: int) -> Tuple[int, int]:
    """[begin, end) of the images rank ``rank`` owns; shards differ by at most one image."""
    if not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} outside world of size {world_size}")
    return global_batch * rank // world_size, global_batch * (rank + 1) // world_size


def shard_batch(t: torch.Tensor, world_size: int, rank: int) -> torch.Tensor:
    """The rank's slice along the batch dimension (a view)."""
    b, e = shard_range(t.shape[0], world_size, rank)
    return t[b:e]


class GradWeightReducer:
    """Sums weight gradients over the ranks, on a side stream when on CUDA so the all-reduce
    overlaps whatever the caller launches next (the input-gradient kernel)."""

    def __init__(self, group: Optional[dist.ProcessGroup] = None, device: Optional[torch.device] = None):
        self.group = group
        self.device = torch.device(device) if device is not None else None
        self._side = None
        if self.device is not None and self.device.type == "cuda":
            self._side = torch.cuda.Stream(self.device)

    @property
    def world_size(self) -> int:
        return dist.get_world_size(self.group) if dist.is_initialized() else 1

    def start(self, grad_weight: torch.Tensor) -> None:
        """Begin summing ``grad_weight`` in place; returns at once on CUDA."""
        if self.world_size == 1:
            return
        if self._side is None:
            dist.all_reduce(grad_weight, group=self.group)
            return
        main = torch.cuda.current_stream(self.device)
        self._side.wait_stream(main)
        with torch.cuda.stream(self._side):
            dist.all_reduce(grad_weight, group=self.group)
        grad_weight.record_stream(self._side)

    def finish(self) -> None:
        """Make the current stream wait for the sum started by :meth:`start`."""
        if self._side is not None and self.world_size > 1:
            torch.cuda.current_stream(self.device).wait_stream(self._side)
