"""Descriptors of the generator tasks: launch Geri and speak its ``/{modality}/generate`` API
(reference: tasklib/cornserve_tasklib/task_executors/descriptor/generator.py:37-203)."""

from __future__ import annotations

import base64
import sys
import time
from collections.abc import AsyncGenerator
from typing import Any

from cornserve.task_executors.descriptor.base import TaskExecutionDescriptor
from cornserve.task_executors.geri.api import (AudioGeriRequest, BatchGeriResponse, ImageGeriRequest, Status,
                                   StreamGeriResponseChunk)
from cornserve.services.resource import GPU
from cornserve.services.task_registry import register_descriptor
from cornserve.task.base import Stream
from cornserve_tasklib.task.unit.generator import (AudioGeneratorInput, AudioGeneratorTask, ImageGeneratorInput, ImageGeneratorOutput,
                                   ImageGeneratorTask)
from cornserve_tasklib.task.unit.llm import ChoiceDelta, ChoiceDeltaAudio, ChunkChoice, OpenAIChatCompletionChunk


async def parse_geri_chunks(response: Any) -> AsyncGenerator[str]:
    """Geri's server-sent events (``data: <base64 bytes as JSON>``) -> chat-completion chunks carrying the
    audio bytes in ``choices[0].delta.audio.data``."""
    pending = b""
    try:
        async for block in response.content.iter_chunked(1 << 16):
            pending += block
            *lines, pending = pending.split(b"\n")
            for raw in lines:
                line = raw.decode().strip()
                if not line.startswith("data: "):
                    continue
                chunk = StreamGeriResponseChunk.model_validate_json(line[6:].strip())
                if not chunk.root:
                    continue
                out = OpenAIChatCompletionChunk(
                    id="0", created=int(time.time()),
                    choices=[ChunkChoice(delta=ChoiceDelta(audio=ChoiceDeltaAudio(data=base64.b64encode(chunk.root).decode())))])
                yield out.model_dump_json()
    finally:
        response.close()


class _GeriLaunch:
    def create_executor_name(self) -> str:
        return "-".join(["geri", self.task.modality, self.task.model_id.split("/")[-1]]).lower()

    def get_entrypoint(self) -> list[str]:
        return [sys.executable, "-m", "cornserve.task_executors.geri.entrypoint"]

    def get_container_args(self, gpus: list[GPU], port: int) -> list[str]:
        return [
            "--model.id", self.task.model_id,
            "--model.modality", self.task.modality.value.upper(),
            "--server.port", str(port),
            "--server.max-batch-size", str(self.task.max_batch_size),
            "--sidecar.ranks", *[str(g.global_rank) for g in gpus],
        ]

    def get_api_url(self, base: str) -> str:
        return f"{base}/{self.task.modality.value}/generate"


@register_descriptor(ImageGeneratorTask, default=True)
class ImageGeriDescriptor(_GeriLaunch, TaskExecutionDescriptor[ImageGeneratorTask, ImageGeneratorInput, ImageGeneratorOutput]):
    def to_request(self, task_input: ImageGeneratorInput, task_output: ImageGeneratorOutput) -> dict[str, Any]:
        return ImageGeriRequest(embedding_data_id=task_input.embeddings.id, height=task_input.height,
                                width=task_input.width, num_inference_steps=task_input.num_inference_steps,
                                skip_tokens=task_input.skip_tokens).model_dump()

    async def from_response(self, task_output: ImageGeneratorOutput, response: Any) -> ImageGeneratorOutput:
        resp = BatchGeriResponse.model_validate(await response.json())
        if resp.status != Status.SUCCESS or resp.generated is None:
            raise RuntimeError(f"Error in generator task: {resp.error_message}")
        return ImageGeneratorOutput(generated=resp.generated)


@register_descriptor(AudioGeneratorTask, default=True)
class AudioGeriDescriptor(_GeriLaunch, TaskExecutionDescriptor[AudioGeneratorTask, AudioGeneratorInput,
                                                               Stream[OpenAIChatCompletionChunk]]):
    def to_request(self, task_input: AudioGeneratorInput, task_output: Stream[OpenAIChatCompletionChunk]) -> dict[str, Any]:
        return AudioGeriRequest(embedding_data_id=task_input.embeddings.id, chunk_size=task_input.chunk_size,
                                left_context_size=task_input.left_context_size).model_dump()

    async def from_response(self, task_output: Stream[OpenAIChatCompletionChunk], response: Any) -> Stream[OpenAIChatCompletionChunk]:
        return Stream[OpenAIChatCompletionChunk](async_iterator=parse_geri_chunks(response), response=response)
