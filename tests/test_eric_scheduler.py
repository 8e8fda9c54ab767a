"""Encoder scheduler: FCFS, batching of consecutive compatible items, request completion."""

import torch

from cornserve.task_executors.eric.scheduler import Scheduler
from cornserve.task_executors.eric.schema import EngineRequest, Modality, ProcessedItem


def _req(rid, specs):
    return EngineRequest(rid, [ProcessedItem(f"{rid}-{i}", m, model, {"x": torch.zeros(1)}) for i, (m, model) in enumerate(specs)])


def test_batches_consecutive_compatible_items():
    s = Scheduler(max_batch_size=3)
    s.enqueue(_req("a", [(Modality.IMAGE, "m")] * 2))
    s.enqueue(_req("b", [(Modality.IMAGE, "m")] * 2))
    s.enqueue(_req("c", [(Modality.VIDEO, "m")]))
    b = s.schedule()
    assert b.data_ids == ["a-0", "a-1", "b-0"] and b.modality == Modality.IMAGE and len(b.data["x"]) == 3
    assert s.process_batch_result(b.request_ids, b.data_ids) == ["a"]
    b = s.schedule()
    assert b.data_ids == ["b-1"]  # the video item is not mixed into an image batch
    assert s.process_batch_result(b.request_ids, b.data_ids) == ["b"]
    b = s.schedule()
    assert b.data_ids == ["c-0"] and b.modality == Modality.VIDEO
    assert s.process_batch_result(b.request_ids, b.data_ids) == ["c"]
    assert s.schedule() is None and not s.has_waiting_requests()


def test_adapter_boundaries_and_unbounded_batches():
    s = Scheduler(max_batch_size=None)
    s.enqueue(_req("a", [(Modality.IMAGE, "m1"), (Modality.IMAGE, "m2"), (Modality.IMAGE, "m2")]))
    assert s.schedule().data_ids == ["a-0"]
    b = s.schedule()
    assert b.data_ids == ["a-1", "a-2"] and b.adapter_name == "m2"
    s2 = Scheduler(max_batch_size=1)
    s2.enqueue(_req("x", [(Modality.IMAGE, "m")] * 2))
    assert [s2.schedule().data_ids, s2.schedule().data_ids] == [["x-0"], ["x-1"]]
    assert s2.process_batch_result(["x"], ["x-0"]) == []
    assert s2.process_batch_result(["x"], ["x-1"]) == ["x"]
