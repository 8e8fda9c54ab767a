"""Two Gemma-3 sizes answer the same question; both read their images through ONE shared vision encoder deployment
(the encoder task lists both model ids, so it loads one SigLIP tower and a projector per model).

    cornserve register examples/encoder_sharing.py
    cornserve invoke encoder_sharing '{"prompt": "What is in the image?", "image_url": "https://picsum.photos/seed/7/896/896"}'
"""

from __future__ import annotations

import asyncio

from cornserve.app.base import AppConfig, AppRequest, AppResponse
from cornserve_tasklib import MLLMTask, Modality, OpenAIChatCompletionRequest

MODELS = ["google/gemma-3-4b-it", "google/gemma-3-12b-it"]


class Request(AppRequest):
    prompt: str
    image_url: str
    max_completion_tokens: int = 128


class Response(AppResponse):
    answers: dict[str, str]


tasks = {m: MLLMTask(model_id=m, modalities=[Modality.IMAGE], encoder_model_ids=set(MODELS)) for m in MODELS}


class Config(AppConfig):
    tasks = {f"mllm_{i}": t for i, t in enumerate(tasks.values())}


async def _ask(model: str, request: Request) -> str:
    content = [{"type": "image_url", "image_url": {"url": request.image_url}}, {"type": "text", "text": request.prompt}]
    stream = await tasks[model](OpenAIChatCompletionRequest(model=model, messages=[{"role": "user", "content": content}],
                                                            max_completion_tokens=request.max_completion_tokens))
    return "".join([(c.choices[0].delta.content or "") async for c in stream if c.choices])


async def serve(request: Request) -> Response:
    texts = await asyncio.gather(*(_ask(m, request) for m in MODELS))
    return Response(answers=dict(zip(MODELS, texts)))
