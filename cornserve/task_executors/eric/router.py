"""HTTP API of the encoder executor (reference: python/cornserve/task_executors/eric/router/app.py:22-105)."""

from __future__ import annotations

import uuid

from fastapi import FastAPI, Request, Response

from ...logging import get_logger
from ...tracing import inject
from .api import EmbeddingRequest, EmbeddingResponse, Status
from .config import EricConfig
from .engine import Engine
from .processor import Processor
from .schema import EngineRequest, Modality
from .schema import Status as EngineStatus

logger = get_logger(__name__)


def create_app(config: EricConfig, engine: Engine) -> FastAPI:
    app = FastAPI(title="cornserve-b200 encoder executor")
    from ...tracing import instrument_fastapi

    instrument_fastapi(app, "cornserve.eric")
    processor = Processor(engine.worker.entry.processor, config.modality)
    model_ids = set(config.model.all_model_ids)

    @app.get("/health")
    async def health():
        return Response(status_code=200 if engine.alive else 503)

    @app.get("/info")
    async def info():
        return config.model_dump(mode="json")

    @app.get("/modalities")
    async def modalities():
        return [m.value for m in engine.worker.entry.modalities]

    @app.post("/embeddings")
    async def embeddings(request: EmbeddingRequest, raw: Request):
        for d in request.data:
            if d.model_id not in model_ids:
                return EmbeddingResponse(status=Status.ERROR, error_message=f"Model {d.model_id} is not served here "
                                         f"(serving {sorted(model_ids)})")
            if d.modality.value != config.model.modality.value:
                return EmbeddingResponse(status=Status.ERROR, error_message=f"This executor encodes "
                                         f"{config.model.modality.value}, not {d.modality.value}")
        try:
            items = await processor.process([(d.id, Modality(d.modality.value), d.model_id, d.url, d.receiver_sidecar_ranks)
                                             for d in request.data])
        except Exception as e:
            logger.exception("Preprocessing failed")
            return EmbeddingResponse(status=Status.ERROR, error_message=f"Failed to load data: {e}")
        resp = await engine.embed(EngineRequest(uuid.uuid4().hex, items, inject()))
        if resp.status == EngineStatus.SUCCESS:
            return EmbeddingResponse(status=Status.SUCCESS)
        return EmbeddingResponse(status=Status.ERROR, error_message=resp.error_message)

    @app.get("/stats")
    async def stats():
        """Counters of this executor since it started (rank 0 of a tensor-parallel group; the other ranks launch the
        same kernels): this library's kernel launches, launches per fused path, batches, host-to-device bytes."""
        from ... import ops

        return {"executor": "eric", "tp_size": config.model.tp_size, "kernel_launches": ops.kernel_launches(),
                "paths": ops.path_counts(), **engine.worker.stats}

    @app.post("/profile/start")
    async def profile_start(out_dir: str = "/tmp/cornserve_profile"):
        engine.start_profile(out_dir)
        return {"status": "started", "dir": out_dir}

    @app.post("/profile/stop")
    async def profile_stop():
        engine.stop_profile()
        return {"status": "stopped"}

    from ..device_timer import add_timer_routes

    add_timer_routes(app, engine.worker.device)
    app.state.processor = processor
    return app
