"""Generator unit tasks: image and (streamed) audio generation from forwarded embeddings
(reference: tasklib/cornserve_tasklib/task/unit/generator.py:21-115)."""

from __future__ import annotations

import enum

from cornserve.services.task_registry import register_task
from cornserve.task.base import Stream, TaskInput, TaskOutput, UnitTask
from cornserve.task.forward import DataForward, Tensor
from cornserve_tasklib.task.unit.llm import OpenAIChatCompletionChunk


class Modality(enum.StrEnum):
    IMAGE = "image"
    VIDEO = "video"
    AUDIO = "audio"


class ImageGeneratorInput(TaskInput):
    """``embeddings`` are the prompt embeddings produced by the text encoder; the first ``skip_tokens``
    rows (chat-template prefix) are dropped by the generator."""

    height: int
    width: int
    num_inference_steps: int
    embeddings: DataForward[Tensor]
    skip_tokens: int = 0


class ImageGeneratorOutput(TaskOutput):
    generated: str  # base64 PNG


@register_task
class ImageGeneratorTask(UnitTask[ImageGeneratorInput, ImageGeneratorOutput]):
    model_id: str
    max_batch_size: int = 1
    modality: Modality = Modality.IMAGE

    def make_record_output(self, task_input: ImageGeneratorInput) -> ImageGeneratorOutput:
        return ImageGeneratorOutput(generated="")

    def validate_input(self, task_input: ImageGeneratorInput) -> None:
        if task_input.height <= 0 or task_input.width <= 0:
            raise ValueError("Height and width must be positive integers.")
        if task_input.num_inference_steps <= 0:
            raise ValueError("Number of inference steps must be positive.")

    def make_name(self) -> str:
        return f"generator-{self.modality.lower()}-{self.model_id.split('/')[-1].lower()}"


class AudioGeneratorInput(TaskInput):
    embeddings: DataForward[Tensor]
    chunk_size: int | None = None
    left_context_size: int | None = None


@register_task
class AudioGeneratorTask(UnitTask[AudioGeneratorInput, Stream[OpenAIChatCompletionChunk]]):
    """Streams audio chunks (``choices[0].delta.audio.data`` = base64 PCM16)."""

    model_id: str
    max_batch_size: int = 1
    modality: Modality = Modality.AUDIO

    def make_record_output(self, task_input: AudioGeneratorInput) -> Stream[OpenAIChatCompletionChunk]:
        return Stream[OpenAIChatCompletionChunk]()

    def make_name(self) -> str:
        return f"generator-{self.modality.lower()}-{self.model_id.split('/')[-1].lower()}"
