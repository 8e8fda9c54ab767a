"""Re-typing a stream: the app exposes plain text pieces instead of OpenAI chunk objects by transforming the task's
output stream once.

    cornserve register examples/stream_transform.py
    cornserve invoke stream_transform '{"prompt": "Count to five."}' --aggregate-keys text
"""

from __future__ import annotations

from collections.abc import AsyncIterator

from cornserve.app.base import AppConfig, AppRequest, AppResponse
from cornserve_tasklib import MLLMTask, OpenAIChatCompletionChunk, OpenAIChatCompletionRequest

MODEL = "Qwen/Qwen2.5-VL-7B-Instruct"


class Request(AppRequest):
    prompt: str


class Piece(AppResponse):
    text: str


llm = MLLMTask(model_id=MODEL, modalities=[], encoder_fission=False)


class Config(AppConfig):
    tasks = {"llm": llm}


def to_piece(chunk: OpenAIChatCompletionChunk) -> Piece:
    return Piece(text=(chunk.choices[0].delta.content or "") if chunk.choices else "")


async def serve(request: Request) -> AsyncIterator[Piece]:
    stream = await llm(OpenAIChatCompletionRequest(model=MODEL, messages=[{"role": "user", "content": request.prompt}]))
    return stream.transform(to_piece, Piece)
