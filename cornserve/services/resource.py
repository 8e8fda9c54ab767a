"""GPU inventory and allocation (reference: python/cornserve/services/resource.py:14-276).

One "node" here is the local box; the model still supports several nodes so that placement policies
(``spread`` / ``pack``, co-location) and their errors behave as in the reference."""

from __future__ import annotations

import heapq
from dataclasses import dataclass, field


class CannotColocateError(Exception):
    """No single node has enough free GPUs for a request that must be co-located."""


class NotEnoughGPUsError(Exception):
    """The cluster does not have enough free GPUs."""


@dataclass
class GPU:
    node: str
    global_rank: int
    local_rank: int
    owner: str | None = None

    @property
    def is_free(self) -> bool:
        return self.owner is None

    def allocate_to(self, owner: str) -> "GPU":
        if self.owner is not None:
            raise ValueError(f"GPU {self.global_rank} is already owned by {self.owner}")
        self.owner = owner
        return self

    def free(self) -> "GPU":
        self.owner = None
        return self


@dataclass
class Resource:
    gpus: list[GPU] = field(default_factory=list)

    def __post_init__(self):
        self._by_node: dict[str, list[GPU]] = {}
        for g in self.gpus:
            self._by_node.setdefault(g.node, []).append(g)
        for lst in self._by_node.values():
            lst.sort(key=lambda g: g.local_rank)

    @classmethod
    def single_node(cls, num_gpus: int, node: str = "localhost") -> "Resource":
        return cls([GPU(node, i, i) for i in range(num_gpus)])

    def num_free(self) -> int:
        return sum(g.is_free for g in self.gpus)

    def owned_by(self, owner: str) -> list[GPU]:
        return [g for g in self.gpus if g.owner == owner]

    def allocate(self, num_gpus: int, owner: str, must_colocate: bool = True,
                 node_selection_policy: str = "spread") -> list[GPU]:
        """Allocate ``num_gpus`` GPUs to ``owner``.

        ``spread`` prefers the node with the most free GPUs (and, on ties, the one where the owner has
        the fewest GPUs); ``pack`` prefers the fullest node that still fits.  Without ``must_colocate``
        the request may span nodes, taking whole chunks from the preferred nodes first.
        """
        if num_gpus <= 0:
            raise ValueError("num_gpus must be positive")
        if node_selection_policy not in ("spread", "pack"):
            raise ValueError(f"unknown policy {node_selection_policy}")
        free = {n: [g for g in lst if g.is_free] for n, lst in self._by_node.items()}
        if sum(len(v) for v in free.values()) < num_gpus:
            raise NotEnoughGPUsError(f"{num_gpus} GPUs requested, {sum(len(v) for v in free.values())} free")
        owned = {n: sum(g.owner == owner for g in lst) for n, lst in self._by_node.items()}
        sign = -1 if node_selection_policy == "spread" else 1
        heap = [(sign * len(f), sign * -owned[n] if node_selection_policy == "spread" else -owned[n], n)
                for n, f in free.items() if f]
        heapq.heapify(heap)
        if must_colocate:
            fits = sorted(h for h in heap if len(free[h[2]]) >= num_gpus)
            if not fits:
                raise CannotColocateError(f"no node has {num_gpus} free GPUs")
            chosen = free[fits[0][2]][:num_gpus]
        else:
            chosen = []
            while len(chosen) < num_gpus and heap:
                _, _, n = heapq.heappop(heap)
                chosen.extend(free[n][: num_gpus - len(chosen)])
        for g in chosen:
            g.allocate_to(owner)
        return chosen

    def release(self, gpus: list[GPU]) -> None:
        for g in gpus:
            g.free()

    def render(self) -> str:
        """ASCII view of GPU ownership, one line per node."""
        lines = []
        for node, lst in sorted(self._by_node.items()):
            cells = " | ".join(f"{g.global_rank}:{(g.owner or '-')[:18]}" for g in lst)
            lines.append(f"{node}: [ {cells} ]")
        return "\n".join(lines)
