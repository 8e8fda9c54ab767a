"""Multimodal chat: images go to a separately deployed (and separately scaled) encoder, text generation streams back.

    cornserve register examples/mllm.py
    cornserve invoke mllm '{"prompt": "Describe the picture.", "multimodal_data": [["image", "https://picsum.photos/seed/1/640/480"]]}' \
        --aggregate-keys choices.0.delta.content
"""

from __future__ import annotations

from collections.abc import AsyncIterator

from cornserve.app.base import AppConfig, AppRequest
from cornserve_tasklib import MLLMTask, Modality, OpenAIChatCompletionChunk, OpenAIChatCompletionRequest

MODEL = "Qwen/Qwen2.5-VL-7B-Instruct"


class Request(AppRequest):
    prompt: str
    multimodal_data: list[tuple[str, str]] = []   # (modality, url)
    max_completion_tokens: int | None = None


mllm = MLLMTask(model_id=MODEL, modalities=[Modality.IMAGE], encoder_fission=True)


class Config(AppConfig):
    tasks = {"mllm": mllm}


async def serve(request: Request) -> AsyncIterator[OpenAIChatCompletionChunk]:
    content: list[dict] = [{"type": "text", "text": request.prompt}]
    for modality, url in request.multimodal_data:
        content.append({"type": f"{modality}_url", f"{modality}_url": {"url": url}})
    return await mllm(OpenAIChatCompletionRequest(model=MODEL, messages=[{"role": "user", "content": content}],
                                                  max_completion_tokens=request.max_completion_tokens))
