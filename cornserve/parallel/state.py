"""Process-group state for tensor / sequence / expert parallelism.

One process drives one GPU.  A :class:`ParallelGroup` wraps a ``torch.distributed`` group (NCCL on
GPUs, gloo on CPU) and, when available, the peer-memory fabric used by the fused kernels.  The
rendezvous address is always passed in by the caller (the resource manager hands out ports), so
several groups can live on one host (the reference hard-codes port 29500:
python/cornserve/task_executors/eric/distributed/parallel.py:130-166).
"""

from __future__ import annotations

import datetime
import os
from dataclasses import dataclass, field
from typing import Any

import torch
import torch.distributed as dist


@dataclass
class ParallelGroup:
    """Rank/size of one parallel dimension plus its communication back-ends."""

    rank: int = 0
    size: int = 1
    group: Any = None  # torch.distributed.ProcessGroup or None when size == 1
    fabric: Any = None  # cornserve.parallel.fabric.Fabric or None
    device: torch.device = field(default_factory=lambda: torch.device("cpu"))

    @property
    def is_first(self) -> bool:
        return self.rank == 0

    # -- baseline collectives (NCCL / gloo); the fused kernels bypass these ------------------
    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.size == 1:
            return x
        dist.all_reduce(x, group=self.group)
        return x

    def all_gather(self, x: torch.Tensor, dim: int = -1) -> torch.Tensor:
        """Concatenate the ranks' tensors along ``dim``."""
        if self.size == 1:
            return x
        x = x.contiguous()
        flat = torch.empty((self.size * x.shape[0], *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(flat, x, group=self.group)  # the concatenated form works on NCCL and gloo alike
        out = flat.view(self.size, *x.shape)
        if dim < 0:
            dim += x.dim()
        out = out.movedim(0, dim)
        shape = list(x.shape)
        shape[dim] *= self.size
        return out.reshape(shape)

    def reduce_scatter(self, x: torch.Tensor) -> torch.Tensor:
        """Sum over ranks and keep this rank's slice of dim 0."""
        if self.size == 1:
            return x
        x = x.contiguous()
        out = torch.empty((x.shape[0] // self.size, *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x, group=self.group)
        return out

    def all_to_all(self, x: torch.Tensor) -> torch.Tensor:
        """Equal-split all-to-all along dim 0."""
        if self.size == 1:
            return x
        x = x.contiguous()
        out = torch.empty_like(x)
        dist.all_to_all_single(out, x, group=self.group)
        return out

    def broadcast_object(self, obj: Any, src: int = 0) -> Any:
        if self.size == 1:
            return obj
        box = [obj]
        dist.broadcast_object_list(box, src=dist.get_global_rank(self.group, src) if self.group else src,
                                   group=self.group)
        return box[0]

    def barrier(self) -> None:
        if self.size > 1:
            dist.barrier(group=self.group)


_SINGLE = ParallelGroup()
_tp_group: ParallelGroup = _SINGLE


def single_group(device: torch.device | str = "cpu") -> ParallelGroup:
    return ParallelGroup(device=torch.device(device))


def get_tp_group() -> ParallelGroup:
    return _tp_group


def set_tp_group(g: ParallelGroup) -> None:
    global _tp_group
    _tp_group = g


def init_distributed(
    rank: int,
    world_size: int,
    *,
    master_addr: str = "127.0.0.1",
    master_port: int | None = None,
    backend: str | None = None,
    local_device: int | None = None,
    timeout_s: float = 600.0,
    with_fabric: bool = True,
) -> ParallelGroup:
    """Join (or create) the default process group and return it as a :class:`ParallelGroup`.

    On GPUs the back-end is NCCL and the device is ``cuda:local_device``; without CUDA it is gloo.
    If ``torch.distributed`` is already initialised (e.g. launched by torchrun) it is reused.
    """
    use_cuda = torch.cuda.is_available() and backend != "gloo"
    backend = backend or ("nccl" if use_cuda else "gloo")
    if use_cuda:
        dev_idx = local_device if local_device is not None else int(os.environ.get("LOCAL_RANK", rank))
        torch.cuda.set_device(dev_idx)
        device = torch.device("cuda", dev_idx)
    else:
        device = torch.device("cpu")
    if world_size == 1:
        g = ParallelGroup(0, 1, None, None, device)
        return g
    if not dist.is_initialized():
        port = master_port or int(os.environ.get("MASTER_PORT", "29511"))
        kwargs: dict[str, Any] = {}
        if use_cuda:
            kwargs["device_id"] = device
        dist.init_process_group(
            backend,
            init_method=f"tcp://{master_addr}:{port}",
            rank=rank,
            world_size=world_size,
            timeout=datetime.timedelta(seconds=timeout_s),
            **kwargs,
        )
    g = ParallelGroup(dist.get_rank(), dist.get_world_size(), dist.group.WORLD, None, device)
    if use_cuda and with_fabric:
        try:
            from .fabric import Fabric

            g.fabric = Fabric.create(g)
        except Exception as e:  # the NCCL path keeps working without peer memory
            import logging

            logging.getLogger(__name__).warning("peer-memory fabric unavailable: %s", e)
    return g
