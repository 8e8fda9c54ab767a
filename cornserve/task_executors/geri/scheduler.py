"""First-come-first-served scheduler of the generator engine (reference:
python/cornserve/task_executors/geri/engine/scheduler.py:24-396).  A batch is the longest *prefix* of the
waiting queue whose requests are compatible with the head (images: same height, width and step count; audio:
same chunk and left-context sizes), capped by ``max_batch_size``; a later compatible request never overtakes an
incompatible one in front of it."""

from __future__ import annotations

from collections import deque

from .schema import Batch, EngineRequest


class Scheduler:
    def __init__(self, max_batch_size: int = 1) -> None:
        self.max_batch_size = max_batch_size
        self.waiting: deque[EngineRequest] = deque()

    def enqueue(self, request: EngineRequest) -> None:
        if any(r.request_id == request.request_id for r in self.waiting):
            raise ValueError(f"duplicate request id {request.request_id}")
        self.waiting.append(request)

    def has_waiting_requests(self) -> bool:
        return bool(self.waiting)

    def __len__(self) -> int:
        return len(self.waiting)

    def abort(self, request_id: str) -> bool:
        for r in list(self.waiting):
            if r.request_id == request_id:
                self.waiting.remove(r)
                return True
        return False

    def schedule(self) -> Batch | None:
        if not self.waiting:
            return None
        head = self.waiting[0]
        key = head.batch_key()
        picked: list[EngineRequest] = []
        while self.waiting and len(picked) < self.max_batch_size and self.waiting[0].batch_key() == key:
            picked.append(self.waiting.popleft())
        return Batch(picked)
