"""Generator engine: a thread that batches compatible requests and runs the model while the router keeps
accepting requests (reference: python/cornserve/task_executors/geri/engine/core.py:71-675, where the engine is a
separate process fed over ZMQ; the batch and streaming behaviour is the same).

Batch mode (images): one response per request when its batch finishes.  Streaming mode (audio): the model is a
generator of waveform chunks; each chunk is packed to little-endian PCM16 on the device and pushed to the
request's queue as soon as it exists, followed by a ``FINISHED`` marker.
"""

from __future__ import annotations

import asyncio
import queue
import threading
import traceback
from typing import Any

import torch

from ... import ops
from ...logging import get_logger
from ...parallel.state import ParallelGroup
from ...tracing import extract, get_tracer
from .config import GeriConfig
from .loader import load_model
from .scheduler import Scheduler
from .schema import Batch, EngineRequest, EngineResponse, GeriMode, Status

logger = get_logger(__name__)
tracer = get_tracer(__name__)


def collect_embed_chunks(chunks: list[torch.Tensor], skip_tokens: int = 0) -> torch.Tensor:
    """Concatenate the forwarded chunks of one tensor and drop the first ``skip_tokens`` rows (the system-prompt
    part of an LLM's hidden states); reference: geri/engine/core.py:164-190."""
    x = chunks[0] if len(chunks) == 1 else torch.cat(chunks, dim=0)
    return x[skip_tokens:] if skip_tokens else x


class Engine:
    def __init__(self, config: GeriConfig, device: torch.device, group: ParallelGroup | None = None) -> None:
        self.config, self.device, self.group = config, device, group
        self.entry, self.model = load_model(config.model.id, device, group, seed=config.model.seed)
        if self.entry.modality != config.model.modality:
            raise ValueError(f"{config.model.id} generates {self.entry.modality.value}, not {config.model.modality.value}")
        self.mode = self.entry.mode
        self.scheduler = Scheduler(config.server.max_batch_size)
        self.inbox: queue.Queue[EngineRequest | None] = queue.Queue()
        self.futures: dict[str, tuple[asyncio.AbstractEventLoop, asyncio.Future]] = {}
        self.streams: dict[str, tuple[asyncio.AbstractEventLoop, asyncio.Queue]] = {}
        self.alive = True
        self.thread = threading.Thread(target=self._run, name="geri-engine", daemon=True)
        self.thread.start()

    # -- called from the router's event loop ------------------------------------------------------------
    async def generate(self, request: EngineRequest) -> EngineResponse:
        if not self.alive:
            return EngineResponse(request.request_id, Status.ERROR, error_message="engine is not running")
        loop = asyncio.get_running_loop()
        fut: asyncio.Future = loop.create_future()
        self.futures[request.request_id] = (loop, fut)
        self.inbox.put(request)
        return await fut

    def generate_stream(self, request: EngineRequest) -> asyncio.Queue:
        """Queue of ``EngineResponse``: chunks (``SUCCESS``), then ``FINISHED`` or ``ERROR``."""
        loop = asyncio.get_running_loop()
        q: asyncio.Queue = asyncio.Queue()
        if not self.alive:
            q.put_nowait(EngineResponse(request.request_id, Status.ERROR, error_message="engine is not running"))
            return q
        self.streams[request.request_id] = (loop, q)
        self.inbox.put(request)
        return q

    def _resolve(self, resp: EngineResponse, final: bool = True) -> None:
        rid = resp.request_id
        if rid in self.futures:
            loop, fut = self.futures.pop(rid)
            loop.call_soon_threadsafe(lambda: fut.done() or fut.set_result(resp))
        elif rid in self.streams:
            loop, q = self.streams[rid]
            if final:
                self.streams.pop(rid, None)
            loop.call_soon_threadsafe(q.put_nowait, resp)

    # -- engine thread -----------------------------------------------------------------------------------
    def _run(self) -> None:
        ops.bind_thread(self.device)  # a new thread starts on CUDA device 0
        try:
            while True:
                if not self.scheduler.has_waiting_requests():
                    item = self.inbox.get()
                    if item is None:
                        break
                    self.scheduler.enqueue(item)
                while True:
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
            for rid in list(self.futures) + list(self.streams):
                self._resolve(EngineResponse(rid, Status.ERROR, error_message="engine stopped"))

    def step(self) -> None:
        batch = self.scheduler.schedule()
        if batch is None:
            return
        ctx = extract(batch.requests[0].trace_carrier) if batch.requests[0].trace_carrier else None
        try:
            with tracer.start_as_current_span("GeriEngine.step", context=ctx) as span:
                span.set_attribute("geri.batch_size", len(batch.requests))
                if self.mode is GeriMode.BATCH:
                    self._execute_batch(batch)
                else:
                    self._execute_stream(batch)
        except Exception as e:
            logger.exception("Batch execution failed")
            msg = f"{e}\n{traceback.format_exc(limit=3)}"
            for rid in batch.request_ids:
                self._resolve(EngineResponse(rid, Status.ERROR, error_message=msg))

    def _call_model(self, method: str, *args, **kw) -> Any:
        if self.group is not None and self.group.size > 1:
            self.group.broadcast_object((method, args, kw), src=0)
        return getattr(self.model, method)(*args, **kw)

    def _execute_batch(self, batch: Batch) -> None:
        p = batch.params
        embeds = [r.embeds for r in batch.requests]
        kw: dict[str, Any] = {}
        if batch.requests[0].negative_embeds is not None:
            kw = {"negative_embeds": [r.negative_embeds for r in batch.requests],
                  "true_cfg_scale": self.config.model.true_cfg_scale}
        images = self._call_model("generate", embeds, p["height"], p["width"], p["num_inference_steps"], **kw)
        for r, img in zip(batch.requests, images, strict=True):
            self._resolve(EngineResponse(r.request_id, Status.SUCCESS, generated=img))

    def _execute_stream(self, batch: Batch) -> None:
        p = batch.params
        codes = [r.embeds for r in batch.requests]
        finished = [False] * len(codes)
        for chunk in self.model.generate(codes, p.get("chunk_size"), p.get("left_context_size")):
            for i, (r, wav) in enumerate(zip(batch.requests, chunk)):
                if wav is None:
                    if not finished[i]:
                        finished[i] = True
                        self._resolve(EngineResponse(r.request_id, Status.FINISHED))
                    continue
                pcm = ops.pcm16(wav.reshape(-1)).cpu().numpy().tobytes()  # little-endian int16
                self._resolve(EngineResponse(r.request_id, Status.SUCCESS, generated=pcm), final=False)
        for i, r in enumerate(batch.requests):
            if not finished[i]:
                self._resolve(EngineResponse(r.request_id, Status.FINISHED))

    def shutdown(self) -> None:
        self.inbox.put(None)
        self.thread.join(timeout=10)
        if self.group is not None and self.group.size > 1:
            try:
                self.group.broadcast_object(("shutdown", (), {}), src=0)
            except Exception:
                pass


def sp_worker_main(config_json: str, rank: int, world: int, master_port: int) -> None:
    """Entry of a sequence-parallel worker process (rank > 0): replay the model calls rank 0 broadcasts."""
    from ...parallel.state import init_distributed
    from ..eric.worker import pick_device

    config = GeriConfig.model_validate_json(config_json)
    device = pick_device(rank)
    group = init_distributed(rank, world, master_port=master_port, local_device=device.index if device.type == "cuda" else None,
                             backend=None if device.type == "cuda" else "gloo")
    _, model = load_model(config.model.id, device, group, seed=config.model.seed)
    while True:
        method, args, kw = group.broadcast_object(None, src=0)
        if method == "shutdown":
            break
        getattr(model, method)(*args, **kw)
