"""Monolithic ("no fission") baseline tasks served by the single-process baseline executor
(reference: tasklib/cornserve_tasklib/task/unit/huggingface.py:48-144)."""

from __future__ import annotations

import uuid

from pydantic import Field

from cornserve.services.task_registry import register_task
from cornserve.task.base import Stream, TaskInput, TaskOutput, UnitTask
from cornserve_tasklib.task.unit.llm import ChatCompletionMessageParam, OpenAIChatCompletionChunk, StreamOptions


class HuggingFaceQwenImageInput(TaskInput):
    prompt: str
    height: int
    width: int
    num_inference_steps: int


class HuggingFaceQwenImageOutput(TaskOutput):
    image: str  # base64 PNG


@register_task
class HuggingFaceQwenImageTask(UnitTask[HuggingFaceQwenImageInput, HuggingFaceQwenImageOutput]):
    """Whole text-to-image pipeline (text encoder + DiT + VAE) in one executor."""

    model_id: str = "Qwen/Qwen-Image"
    max_batch_size: int = 1

    def make_record_output(self, task_input: HuggingFaceQwenImageInput) -> HuggingFaceQwenImageOutput:
        return HuggingFaceQwenImageOutput(image="")

    def make_name(self) -> str:
        return f"hf-{self.model_id.split('/')[-1].lower()}"


class HuggingFaceQwenOmniInput(TaskInput):
    messages: list[ChatCompletionMessageParam]
    model: str
    frequency_penalty: float | None = 0.0
    max_completion_tokens: int | None = None
    presence_penalty: float | None = 0.0
    seed: int | None = None
    stream_options: StreamOptions | None = None
    temperature: float | None = None
    top_p: float | None = None
    request_id: str = Field(default_factory=lambda: uuid.uuid4().hex)
    ignore_eos: bool = False
    return_audio: bool = True


class HuggingFaceQwenOmniOutput(TaskOutput):
    """One streamed item: either an audio chunk (base64 float32 waveform) or a text chunk."""

    audio_chunk: str | None = None
    text_chunk: OpenAIChatCompletionChunk | None = None


@register_task
class HuggingFaceQwenOmniTask(UnitTask[HuggingFaceQwenOmniInput, Stream[HuggingFaceQwenOmniOutput]]):
    """Whole omni model (encoders + thinker + talker + vocoder) in one executor."""

    model_id: str = "Qwen/Qwen2.5-Omni-7B"
    max_batch_size: int = 1

    def make_record_output(self, task_input: HuggingFaceQwenOmniInput) -> Stream[HuggingFaceQwenOmniOutput]:
        return Stream[HuggingFaceQwenOmniOutput]()

    def validate_input(self, task_input: HuggingFaceQwenOmniInput) -> None:
        if task_input.model != self.model_id:
            raise ValueError(f"Model ID in task input ({task_input.model}) does not match the task model ID "
                             f"({self.model_id}).")

    def make_name(self) -> str:
        return f"hf-{self.model_id.split('/')[-1].lower().replace('.', '-')}"
