"""HTTP API of the generator executor (reference: python/cornserve/task_executors/geri/router.py:26-107 and
geri/engine/client.py:154-251): ``POST /image/generate`` answers with one base64 PNG, ``POST /audio/generate``
with server-sent events whose ``data:`` lines are base64-in-JSON PCM16 chunks.  The conditioning tensor arrives
through the sidecar: the handler awaits every chunk of ``embedding_data_id`` (until the stream's end marker)
before the request enters the engine queue."""

from __future__ import annotations

import uuid

import torch
from fastapi import FastAPI, Response
from fastapi.responses import StreamingResponse

from ...logging import get_logger
from ...sidecar.api import Sidecar
from ...tracing import inject
from .api import AudioGeriRequest, BatchGeriResponse, ImageGeriRequest, Status, StreamGeriResponseChunk
from .config import GeriConfig
from .engine import Engine, collect_embed_chunks
from .schema import EngineRequest
from .schema import Status as EngineStatus

logger = get_logger(__name__)


async def receive_all_chunks(sidecar: Sidecar | None, data_id: str, skip_tokens: int = 0) -> torch.Tensor:
    """Every chunk of ``data_id`` in order; consumed chunks are released back to the producer."""
    if sidecar is None:
        raise RuntimeError("this executor has no sidecar: it cannot receive conditioning tensors")
    chunks, i = [], 0
    while True:
        c = await sidecar.recv(data_id, i)  # None once i is past the last chunk
        if c is None:
            break
        chunks.append(c.clone() if isinstance(c, torch.Tensor) else torch.as_tensor(c))
        await sidecar.mark_done(data_id, i)
        i += 1
    if not chunks:
        raise RuntimeError(f"no data arrived for {data_id}")
    return collect_embed_chunks(chunks, skip_tokens)


def create_app(config: GeriConfig, engine: Engine, sidecar: Sidecar | None) -> FastAPI:
    app = FastAPI(title="cornserve-b200 generator executor")
    from ...tracing import instrument_fastapi

    instrument_fastapi(app, "cornserve.geri")

    @app.get("/health")
    async def health():
        return Response(status_code=200 if engine.alive else 503)

    @app.get("/info")
    async def info():
        return config.model_dump(mode="json")

    @app.post("/image/generate")
    async def image_generate(request: ImageGeriRequest) -> BatchGeriResponse:
        try:
            embeds = await receive_all_chunks(sidecar, request.embedding_data_id, request.skip_tokens)
        except Exception as e:
            logger.exception("Receiving embeddings failed")
            return BatchGeriResponse(status=Status.ERROR, error_message=f"Failed to receive embeddings: {e}")
        params = {"height": request.height, "width": request.width, "num_inference_steps": request.num_inference_steps}
        resp = await engine.generate(EngineRequest(uuid.uuid4().hex, embeds, params, trace_carrier=inject()))
        if resp.status == EngineStatus.SUCCESS:
            return BatchGeriResponse(status=Status.SUCCESS, generated=resp.generated)
        return BatchGeriResponse(status=Status.ERROR, error_message=resp.error_message)

    @app.post("/audio/generate")
    async def audio_generate(request: AudioGeriRequest):
        try:
            codes = await receive_all_chunks(sidecar, request.embedding_data_id)
        except Exception as e:
            logger.exception("Receiving codes failed")
            return Response(status_code=500, content=f"Failed to receive codes: {e}")
        # codes arrive as [T, num_quantizers] rows; the vocoder wants [num_quantizers, T]
        codes = codes.long()
        if codes.dim() == 2 and codes.shape[1] == engine.model.embedding_dim and codes.shape[0] != codes.shape[1]:
            codes = codes.t()
        params = {"chunk_size": request.chunk_size, "left_context_size": request.left_context_size}
        q = engine.generate_stream(EngineRequest(uuid.uuid4().hex, codes.contiguous(), params, trace_carrier=inject()))

        async def events():
            while True:
                resp = await q.get()
                if resp.status == EngineStatus.SUCCESS:
                    yield f"data: {StreamGeriResponseChunk(resp.generated).model_dump_json()}\n\n"
                elif resp.status == EngineStatus.FINISHED:
                    return
                else:
                    logger.error("Audio generation failed: %s", resp.error_message)
                    return

        return StreamingResponse(events(), media_type="text/event-stream")

    return app
