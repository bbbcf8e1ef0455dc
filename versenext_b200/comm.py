"""The library's NCCL communicator (`vn_comm_*`): all-gathers of device buffers on the context's stream.

The reference's decode path has no collective (its only one is the training loop's `all_reduce`,
verse_torch/training.py:2260-2266); this serves the vocabulary-sharded LM head + acceptance.  The 128-byte NCCL id
is made by rank 0 and handed to the other ranks by whatever the host already has -- here an object broadcast over
an existing `torch.distributed` group (any backend), used once at set-up and never on the data path.
"""

from __future__ import annotations

import ctypes as C

import numpy as np

from .device import Context, DeviceArray


class Comm:
    def __init__(self, ctx: Context, unique_id: bytes, world: int, rank: int):
        if len(unique_id) != 128:
            raise ValueError("the NCCL unique id has 128 bytes")
        self.ctx, self.world, self.rank = ctx, int(world), int(rank)
        buf = (C.c_uint8 * 128).from_buffer_copy(unique_id)
        h = C.c_void_p()
        ctx._check(ctx.lib.vn_comm_create(ctx.handle, buf, self.world, self.rank, C.byref(h)))
        self.handle = h

    @staticmethod
    def unique_id(ctx: Context) -> bytes:
        buf = (C.c_uint8 * 128)()
        ctx._check(ctx.lib.vn_comm_unique_id(buf))
        return bytes(buf)

    @classmethod
    def from_torch_group(cls, ctx: Context, group=None) -> "Comm":
        """One communicator over the ranks of an initialised torch.distributed group."""
        import torch.distributed as dist
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        box = [cls.unique_id(ctx) if rank == 0 else None]
        dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        return cls(ctx, box[0], world, rank)

    def all_gather(self, send: DeviceArray, recv: DeviceArray):
        """recv [world, ...send.shape] <- every rank's send (asynchronous, on the context's stream)."""
        if recv.nbytes != send.nbytes * self.world:
            raise ValueError("recv must hold world x send bytes")
        self.ctx._check(self.ctx.lib.vn_all_gather(self.handle, C.c_void_p(send.ptr), C.c_void_p(recv.ptr), send.nbytes))
        return recv

    def __del__(self):
        try:
            if getattr(self, "handle", None):
                self.ctx.lib.vn_comm_destroy(self.handle)
                self.handle = None
        except Exception:
            pass
