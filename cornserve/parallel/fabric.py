"""Peer-memory fabric: buffers that every rank of a group can address directly over NVLink.

Built on ``torch.distributed._symmetric_memory`` (CUDA VMM allocations whose handles are exchanged at a
rendezvous, plus an NVSwitch multicast mapping when the hardware offers it).  The kernels in this package
receive the raw peer pointers; the collectives themselves are written here, not delegated to NCCL.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..logging import get_logger

logger = get_logger(__name__)


@dataclass
class SymmetricBuffer:
    """One symmetric allocation: the local tensor and the same region in every rank's memory."""

    local: torch.Tensor
    ptrs: list[int]            # ptrs[r] = address of rank r's copy, valid on this device
    multicast_ptr: int         # NVSwitch multicast address of the region (0 = not available)
    handle: object

    def ptr_array(self) -> ctypes.Array:
        arr = (ctypes.c_void_p * len(self.ptrs))(*self.ptrs)
        return arr


class Fabric:
    def __init__(self, group) -> None:
        self.group = group
        self.rank, self.world = group.rank, group.size
        self.device = group.device
        self._buffers: list[SymmetricBuffer] = []

    @classmethod
    def create(cls, group) -> "Fabric":
        if group.device.type != "cuda":
            raise RuntimeError("the peer-memory fabric needs CUDA devices")
        return cls(group)

    @classmethod
    def loopback(cls, device: torch.device | str) -> "Fabric":
        """A one-rank fabric whose "peer" buffers are this GPU's own memory.  The fused kernels then run their whole
        communication path (pushes, arrival counters, waits) against themselves on a single GPU, which is how they are
        timed and profiled in isolation (a profiler that replays a kernel cannot be pointed at one rank of a group:
        the replays would break the counters the other ranks wait on)."""
        from .state import ParallelGroup

        f = cls(ParallelGroup(0, 1, None, None, torch.device(device)))
        f._loopback = True
        f.group.fabric = f
        return f

    def alloc(self, numel: int, dtype: torch.dtype, zero: bool = True) -> SymmetricBuffer:
        """Collective: every rank of the group must call with the same arguments, in the same order."""
        if getattr(self, "_loopback", False):
            t = torch.zeros(numel, dtype=dtype, device=self.device) if zero else torch.empty(numel, dtype=dtype, device=self.device)
            buf = SymmetricBuffer(t, [t.data_ptr()], 0, None)
            self._buffers.append(buf)
            return buf
        import torch.distributed._symmetric_memory as symm

        t = symm.empty(numel, dtype=dtype, device=self.device)
        if zero:
            t.zero_()
        torch.cuda.synchronize(self.device)
        h = symm.rendezvous(t, self.group.group if self.group.group is not None else dist.group.WORLD)
        ptrs = [int(p) for p in h.buffer_ptrs]
        mc = 0
        try:
            if h.has_multicast_support(self.device.type, self.device.index):
                mc = int(h.multicast_ptr)
        except Exception:
            mc = 0
        buf = SymmetricBuffer(t, ptrs, mc, h)
        self._buffers.append(buf)
        dist.barrier(group=self.group.group)
        return buf
