"""Client-side configuration (reference: python/cornserve/sidecar/schema.py:12-108)."""

from __future__ import annotations

import dataclasses
from math import prod

import torch


@dataclasses.dataclass
class SidecarConfig:
    """``group`` lists the sidecar ranks of this executor's tensor-parallel group (sorted); the smallest
    rank is the group leader.  Shapes are hints for the slot size: a slot holds one row, i.e.
    ``prod(shape[1:])`` elements, so a tensor of ``n`` rows takes ``n`` contiguous slots."""

    sidecar_rank: int
    group: list[int] | None = None
    max_workers: int = 8
    send_tensor_dtype: torch.dtype | None = None
    send_tensor_shape: tuple[int, ...] | int | None = None
    recv_tensor_dtype: torch.dtype | None = None
    recv_tensor_shape: tuple[int, ...] | int | None = None
    concurrent_copy: bool = False
    # This client stands for every rank of ``group``: the other ranks of the executor have no sidecar client of their
    # own (an executor whose leader alone talks to the sidecars), so it also answers for them where the protocol counts
    # the members of a group (``mark_done``).
    whole_group: bool = False

    def __post_init__(self) -> None:
        if self.group is None:
            self.group = [self.sidecar_rank]
        self.group = sorted(self.group)
        if self.sidecar_rank not in self.group:
            raise ValueError("Sidecar rank should be in the group")
        if self.max_workers <= 0:
            raise ValueError("Max workers should be positive")
        if self.send_tensor_shape is None and self.recv_tensor_shape is None:
            raise ValueError("Either send tensor shape or recv tensor shape should be set")
        if (self.send_tensor_shape is None) != (self.send_tensor_dtype is None):
            raise ValueError("Send tensor shape and dtype should be set together")
        if (self.recv_tensor_shape is None) != (self.recv_tensor_dtype is None):
            raise ValueError("Recv tensor shape and dtype should be set together")

    @staticmethod
    def _tuple(shape) -> tuple[int, ...]:
        return shape if isinstance(shape, tuple) else (shape,)

    def get_send_tensor_shape(self) -> tuple[int, ...]:
        return self._tuple(self.send_tensor_shape if self.send_tensor_shape is not None else self.recv_tensor_shape)

    def get_recv_tensor_shape(self) -> tuple[int, ...]:
        return self._tuple(self.recv_tensor_shape if self.recv_tensor_shape is not None else self.send_tensor_shape)

    @staticmethod
    def _slot_numel(shape: tuple[int, ...]) -> int:
        return max(1, prod(abs(d) for d in shape[1:])) if len(shape) > 1 else max(1, abs(shape[0]))

    def get_send_slot_numel(self) -> int:
        return self._slot_numel(self.get_send_tensor_shape())

    def get_recv_slot_numel(self) -> int:
        return self._slot_numel(self.get_recv_tensor_shape())

    def get_send_dtype(self) -> torch.dtype:
        return self.send_tensor_dtype or self.recv_tensor_dtype  # type: ignore[return-value]

    def get_recv_dtype(self) -> torch.dtype:
        return self.recv_tensor_dtype or self.send_tensor_dtype  # type: ignore[return-value]

    @property
    def leader(self) -> int:
        return self.group[0]

    @property
    def shard_rank(self) -> int:
        return self.group.index(self.sidecar_rank)
