"""First-come-first-served scheduler of the encoder engine (reference:
python/cornserve/task_executors/eric/engine/scheduler.py:22-187).  Requests wait in arrival order; a batch
takes consecutive not-yet-scheduled items from the head of the queue as long as they share modality and
adapter (model id) and the batch stays within ``max_batch_size``.  A request completes when all of its
items have completed."""

from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass, field

from .schema import Batch, EngineRequest, ProcessedItem


@dataclass
class _Tracked:
    request: EngineRequest
    next_item: int = 0
    done: set[str] = field(default_factory=set)


class Scheduler:
    def __init__(self, max_batch_size: int | None = 1) -> None:
        self.max_batch_size = max_batch_size
        self.queue: OrderedDict[str, _Tracked] = OrderedDict()

    def enqueue(self, request: EngineRequest) -> None:
        if request.request_id in self.queue:
            raise ValueError(f"duplicate request id {request.request_id}")
        self.queue[request.request_id] = _Tracked(request)

    def has_waiting_requests(self) -> bool:
        return any(t.next_item < len(t.request.items) for t in self.queue.values())

    def schedule(self) -> Batch | None:
        picked: list[tuple[_Tracked, ProcessedItem]] = []
        key = None
        for t in self.queue.values():
            stop = False
            while t.next_item < len(t.request.items):
                item = t.request.items[t.next_item]
                k = (item.modality, item.model_id)
                if key is None:
                    key = k
                if k != key or (self.max_batch_size is not None and len(picked) >= self.max_batch_size):
                    stop = True
                    break
                picked.append((t, item))
                t.next_item += 1
            if stop or (picked and t.next_item < len(t.request.items)):
                break
        if not picked:
            return None
        data: dict[str, list] = {}
        for _, item in picked:
            for k, v in item.processed.items():
                data.setdefault(k, []).append(v)
        return Batch(
            modality=key[0], adapter_name=key[1],
            request_ids=[t.request.request_id for t, _ in picked], data_ids=[i.id for _, i in picked],
            receiver_ranks=[i.receiver_sidecar_ranks for _, i in picked], data=data,
            trace_carriers=[t.request.trace_carrier for t, _ in picked],
        )

    def process_batch_result(self, request_ids: list[str], data_ids: list[str]) -> list[str]:
        """Mark items done; returns the ids of the requests that are now complete (and forgets them)."""
        finished = []
        for rid, did in zip(request_ids, data_ids, strict=True):
            t = self.queue.get(rid)
            if t is None:
                continue
            t.done.add(did)
            if len(t.done) == len(t.request.items):
                finished.append(rid)
                del self.queue[rid]
        return finished

    def abort(self, request_id: str) -> None:
        self.queue.pop(request_id, None)
