"""Encoder engine: a thread that schedules batches and drives the worker(s) while the router keeps
accepting requests (reference: python/cornserve/task_executors/eric/engine/core.py:84-272, which uses
separate engine and worker processes connected by ZMQ and a shared-memory ring; here rank 0's worker
shares the process and the other TP ranks follow a ``torch.distributed`` broadcast)."""

from __future__ import annotations

import asyncio
import queue
import threading
import time
import traceback

from ... import ops
from ...logging import get_logger
from ...parallel.state import ParallelGroup
from .config import EricConfig
from .scheduler import Scheduler
from .schema import EngineRequest, EngineResponse, Status
from .worker import Worker, broadcast_batch

logger = get_logger(__name__)


class Engine:
    def __init__(self, config: EricConfig, group: ParallelGroup | None = None) -> None:
        self.config = config
        self.group = group
        self.worker = Worker(config, 0, group)
        self.scheduler = Scheduler(config.server.max_batch_size)
        self.inbox: queue.Queue[EngineRequest | None] = queue.Queue()
        self.futures: dict[str, tuple[asyncio.AbstractEventLoop, asyncio.Future]] = {}
        self.alive = True
        self.thread = threading.Thread(target=self._run, name="eric-engine", daemon=True)
        self.thread.start()

    # -- called from the router's event loop --------------------------------------------------------------
    async def embed(self, request: EngineRequest) -> EngineResponse:
        if not self.alive:
            return EngineResponse(request.request_id, Status.ERROR, "engine is not running")
        loop = asyncio.get_running_loop()
        fut: asyncio.Future = loop.create_future()
        self.futures[request.request_id] = (loop, fut)
        self.inbox.put(request)
        return await fut

    def _resolve(self, request_id: str, resp: EngineResponse) -> None:
        entry = self.futures.pop(request_id, None)
        if entry is not None:
            loop, fut = entry
            loop.call_soon_threadsafe(lambda: fut.done() or fut.set_result(resp))

    # -- engine thread ---------------------------------------------------------------------------------------
    def _call_workers(self, method: str, *args) -> None:
        if self.group is not None and self.group.size > 1:
            if method == "execute_model":
                # the followers get the small part of the batch as an object and the inputs by a device broadcast
                # from this rank's staged copy (the reference pickles whole batches through a shared-memory ring)
                t0 = time.perf_counter()
                staged = self.worker.stage(args[0])
                broadcast_batch(self.group, staged, self.worker.device)
                self.worker.stats["broadcast_ms"] += (time.perf_counter() - t0) * 1e3
                self.worker.execute_model(staged)
                return
            self.group.broadcast_object((method, args), src=0)
        getattr(self.worker, method)(*args)

    def _run(self) -> None:
        ops.bind_thread(self.worker.device)  # a new thread starts on CUDA device 0
        try:
            while True:
                if not self.scheduler.has_waiting_requests():
                    item = self.inbox.get()
                    if item is None:
                        break
                    self.scheduler.enqueue(item)
                while True:  # drain whatever arrived meanwhile
                    try:
                        item = self.inbox.get_nowait()
                    except queue.Empty:
                        break
                    if item is None:
                        raise SystemExit
                    self.scheduler.enqueue(item)
                self.step()
        except SystemExit:
            pass
        except Exception:
            logger.exception("Engine loop died")
        finally:
            self.alive = False
            for rid in list(self.futures):
                self._resolve(rid, EngineResponse(rid, Status.ERROR, "engine stopped"))

    def step(self) -> None:
        batch = self.scheduler.schedule()
        if batch is None:
            return
        try:
            self._call_workers("execute_model", batch)
        except Exception as e:
            logger.exception("Batch execution failed")
            msg = f"{e}\n{traceback.format_exc(limit=3)}"
            for rid in dict.fromkeys(batch.request_ids):
                self.scheduler.abort(rid)
                self._resolve(rid, EngineResponse(rid, Status.ERROR, msg))
            return
        for rid in self.scheduler.process_batch_result(batch.request_ids, batch.data_ids):
            self._resolve(rid, EngineResponse(rid, Status.SUCCESS))

    def start_profile(self, out_dir: str) -> None:
        self._call_workers("start_profile", out_dir)

    def stop_profile(self) -> None:
        self._call_workers("stop_profile")

    def shutdown(self) -> None:
        self.inbox.put(None)
        self.thread.join(timeout=10)
        if self.group is not None and self.group.size > 1:
            try:
                self.group.broadcast_object(("shutdown", ()), src=0)
            except Exception:
                pass
        self.worker.shutdown()
