"""Arena: three Gemma-3 sizes stream their answers side by side over one shared image encoder; every streamed line
names the model it came from.

    cornserve register examples/gemmarena.py
    cornserve invoke gemmarena '{"prompt": "Write a haiku about the picture.", "image_url": "https://picsum.photos/seed/3/896/896"}'
"""

from __future__ import annotations

import asyncio
from collections.abc import AsyncIterator

from cornserve.app.base import AppConfig, AppRequest, AppResponse
from cornserve_tasklib import MLLMTask, Modality, OpenAIChatCompletionRequest

MODELS = {"4b": "google/gemma-3-4b-it", "12b": "google/gemma-3-12b-it", "27b": "google/gemma-3-27b-it"}


class Request(AppRequest):
    prompt: str
    image_url: str | None = None
    max_completion_tokens: int = 256


class Delta(AppResponse):
    model: str
    text: str
    done: bool = False


arena = {k: MLLMTask(model_id=m, modalities=[Modality.IMAGE], encoder_model_ids=set(MODELS.values())) for k, m in MODELS.items()}


class Config(AppConfig):
    tasks = {f"gemma_{k}": t for k, t in arena.items()}


async def serve(request: Request) -> AsyncIterator[Delta]:
    content: list[dict] = [{"type": "text", "text": request.prompt}]
    if request.image_url:
        content.insert(0, {"type": "image_url", "image_url": {"url": request.image_url}})
    queue: asyncio.Queue[Delta] = asyncio.Queue()

    async def pump(key: str) -> None:
        try:
            stream = await arena[key](OpenAIChatCompletionRequest(model=MODELS[key], messages=[{"role": "user", "content": content}],
                                                                  max_completion_tokens=request.max_completion_tokens))
            async for chunk in stream:
                if chunk.choices and chunk.choices[0].delta.content:
                    await queue.put(Delta(model=key, text=chunk.choices[0].delta.content))
        finally:
            await queue.put(Delta(model=key, text="", done=True))

    async def merged() -> AsyncIterator[Delta]:
        pumps = [asyncio.create_task(pump(k)) for k in arena]
        remaining = len(pumps)
        while remaining:
            d = await queue.get()
            remaining -= d.done
            yield d
        await asyncio.gather(*pumps, return_exceptions=True)

    return merged()
