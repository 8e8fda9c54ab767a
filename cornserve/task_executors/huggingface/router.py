"""``POST /generate``, ``GET /health``, ``GET /info`` (reference: python/cornserve/task_executors/huggingface/router.py:19-88).
Image requests get one JSON response; omni requests get newline-delimited JSON items."""

from __future__ import annotations

from fastapi import FastAPI, Response
from fastapi.responses import StreamingResponse

from .api import HuggingFaceRequest, HuggingFaceResponse, ModelType, Status
from .config import HuggingFaceConfig
from .engine import Engine


def create_app(config: HuggingFaceConfig, engine: Engine) -> FastAPI:
    app = FastAPI(title="cornserve-b200 monolithic baseline executor")
    from ...tracing import instrument_fastapi

    instrument_fastapi(app, "cornserve.huggingface")

    @app.get("/health")
    async def health():
        return Response(status_code=200 if engine.alive else 503)

    @app.get("/info")
    async def info():
        return config.model_dump(mode="json")

    @app.post("/generate")
    async def generate(request: HuggingFaceRequest):
        if config.model.model_type == ModelType.QWEN_IMAGE:
            if None in (request.prompt, request.height, request.width, request.num_inference_steps):
                return HuggingFaceResponse(status=Status.ERROR, error_message="prompt, height, width and num_inference_steps are required")
            return await engine.generate(request)

        async def lines():
            async for item in engine.stream(request):
                yield item.model_dump_json(exclude_none=True) + "\n"

        return StreamingResponse(lines(), media_type="application/x-ndjson")

    return app
