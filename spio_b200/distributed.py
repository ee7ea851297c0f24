"""Data-parallel plumbing for the gw8 layer: batch sharding and the one exchange the path
needs, the sum of the per-rank weight gradients.

Forward and input gradient touch only a rank's own images; the weight gradient is a sum
over the batch, so each rank computes the partial over its shard and the partials are added
with one all-reduce (NCCL over NVLink on GPUs, gloo on CPU ranks in tests), or, on the GPUs of
one node, by :class:`PeerExchange`: two small kernels inside the step's chain of dependent
launches that store every rank's gradient into every rank's exchange buffer and add the
copies in rank order.  The reference has no multi-device support to mirror; its only device
awareness is keying the kernel cache by device ordinal (spio/kernels/kernel_key.py:13-18).
"""

from __future__ import annotations

import ctypes
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


def rank_order_sum(parts) -> torch.Tensor:
    """The sum :class:`PeerExchange` computes: ``((0 + parts[0]) + parts[1]) + ...`` in fp32, in
    rank order, identical on every rank.  Used by the CPU tests as the statement of that order."""
    total = torch.zeros_like(parts[0], dtype=torch.float32)
    for p in parts:
        total = total + p.to(torch.float32)
    return total


class PeerExchange:
    """Exchange buffers of the data-parallel weight-gradient sum on the GPUs of one node.

    Every rank allocates one buffer through the library, the ranks swap the CUDA IPC handles
    with ``all_gather_object`` over ``group`` (any backend) and map each other's buffers.  After
    that no host-side communication happens: ``options()`` gives the structure the combined
    backward call takes (``spio_gw8_backward_opts.dp``), and the caller calls ``advance()`` once
    per exchange, on every rank alike.  ``capacity`` is the largest vector (floats of dw plus
    dbias) that will be summed.
    """

    def __init__(self, capacity: int, group: Optional[dist.ProcessGroup] = None,
                 device: Optional[torch.device] = None):
        from . import _clib

        self._lib = _clib.load()
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.capacity = (int(capacity) + 3) // 4 * 4
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.seq = 0
        self._local = ctypes.c_void_p()
        self._peers = []
        nbytes = self._lib.spio_dp_buffer_bytes(self.world, self.capacity)
        if nbytes == 0:
            raise ValueError(f"world size {self.world} is not supported by the peer exchange")
        handle = (ctypes.c_ubyte * 64)()
        with torch.cuda.device(self.device):
            _clib.check(self._lib.spio_dp_buffer_alloc(nbytes, ctypes.byref(self._local), handle), "peer exchange")
            handles = [bytes(handle)]
            if self.world > 1:
                handles = [None] * self.world
                dist.all_gather_object(handles, bytes(handle), group=group)
            self._table = (ctypes.c_void_p * self.world)()
            for r, h in enumerate(handles):
                if r == self.rank:
                    self._table[r] = self._local.value
                    continue
                peer = ctypes.c_void_p()
                _clib.check(self._lib.spio_dp_buffer_open(h, ctypes.byref(peer)), f"peer exchange, rank {r}")
                self._peers.append(peer)
                self._table[r] = peer.value
            if self.world > 1:
                dist.barrier(group=group)  # every buffer is zeroed and mapped before the first push

    def options(self):
        """``spio_dp_exchange`` for the next exchange (keep the returned object alive for the call)."""
        from . import _clib

        return _clib.DpExchange(ctypes.cast(self._table, ctypes.POINTER(ctypes.c_void_p)), self.rank, self.world,
                                self.seq, self.capacity)

    def advance(self) -> None:
        self.seq += 1

    def close(self) -> None:
        for peer in self._peers:
            self._lib.spio_dp_buffer_close(peer)
        self._peers = []
        if self._local:
            self._lib.spio_dp_buffer_free(self._local)
            self._local = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
