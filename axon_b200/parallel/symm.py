"""Peer-memory plumbing: buffers that every rank of a process group can address from device code.

``SymmetricBuffer`` wraps ``torch.distributed._symmetric_memory`` (CUDA VMM allocations exchanged
between ranks): each rank allocates the same number of bytes, rendezvous maps every peer's
allocation, and the wrapper exposes the table of peer base pointers that the native kernels take
(plain NVLink loads/stores; never a TMA multicast). ``PeerBarrier`` is the bounded device-side
barrier over per-rank signal pads. On CPU (gloo) the same classes degrade to process-local tensors so
host-side logic stays testable.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist


class SymmetricBuffer:
    def __init__(self, numel: int, dtype: torch.dtype, group=None, device=None):
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.numel, self.dtype = numel, dtype
        if self.device.type == "cuda":
            import torch.distributed._symmetric_memory as symm
            self.tensor = symm.empty(numel, dtype=dtype, device=self.device)
            self.handle = symm.rendezvous(self.tensor, self.group.group_name if hasattr(self.group, "group_name") else self.group)
            self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
            self.signal_pad_ptrs = [int(p) for p in self.handle.signal_pad_ptrs]
        else:
            self.tensor = torch.zeros(numel, dtype=dtype)
            self.handle = None
            self.ptrs = [self.tensor.data_ptr()] * self.world
            self.signal_pad_ptrs = [0] * self.world

    def ptr_array(self):
        return (ctypes.c_ulonglong * self.world)(*self.ptrs)

    def peer_tensor(self, rank: int, numel: int | None = None, offset: int = 0) -> torch.Tensor:
        """A tensor aliasing ``rank``'s buffer (for host-side checks; kernels use the raw pointers)."""
        if self.handle is None:
            return self.tensor
        n = self.numel if numel is None else numel
        return self.handle.get_buffer(rank, (n,), self.dtype, offset)

    def barrier(self) -> None:
        if self.handle is not None:
            self.handle.barrier()
        elif self.world > 1:
            dist.barrier(self.group)


class PeerBarrier:
    """Device-side barrier: each rank writes an increasing epoch into its slot of every peer's pad and
    waits (bounded, ~2 s) until all slots of its own pad reached the epoch. A timeout is reported
    through the per-device status word, never by hanging."""

    def __init__(self, group=None, device=None):
        self.buf = SymmetricBuffer(64, torch.int32, group, device)
        self.buf.tensor.zero_()
        self.buf.barrier()
        self.epoch = 0

    def __call__(self) -> None:
        from ..ops import _common as C
        self.epoch += 1
        if self.buf.handle is None:
            if self.buf.world > 1:
                dist.barrier(self.buf.group)
            return
        rc = C.lib().axb_peer_barrier(self.buf.ptr_array(), self.buf.rank, self.buf.world, ctypes.c_uint(self.epoch),
                                      C.ptr(C.status(self.buf.device)), C.stream())
        C.launched(rc, "peer_barrier")
