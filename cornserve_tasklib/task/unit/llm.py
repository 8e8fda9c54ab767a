"""OpenAI-compatible LLM unit tasks (reference: tasklib/cornserve_tasklib/task/unit/llm.py:27-253)."""

from __future__ import annotations

import uuid
from typing import Any, Generic, Literal, TypeVar

from pydantic import BaseModel, ConfigDict, Field

from cornserve.services.task_registry import register_task
from cornserve.task.base import Stream, TaskInput, TaskOutput, UnitTask
from cornserve.task.forward import DataForward, Tensor


class StreamOptions(BaseModel):
    include_usage: bool = True


class URL(BaseModel):
    url: str


class ChatCompletionContentPartTextParam(BaseModel):
    type: Literal["text"] = "text"
    text: str


class ChatCompletionContentPartAudioParam(BaseModel):
    type: Literal["audio_url"] = "audio_url"
    audio_url: URL


class ChatCompletionContentPartImageParam(BaseModel):
    type: Literal["image_url"] = "image_url"
    image_url: URL


class ChatCompletionContentPartVideoParam(BaseModel):
    type: Literal["video_url"] = "video_url"
    video_url: URL


ChatCompletionContentPartMultimodalParam = (
    ChatCompletionContentPartAudioParam | ChatCompletionContentPartImageParam | ChatCompletionContentPartVideoParam
)
ChatCompletionContentPartParam = ChatCompletionContentPartTextParam | ChatCompletionContentPartMultimodalParam


class ChatCompletionMessageParam(BaseModel):
    role: str
    content: str | list[ChatCompletionContentPartParam]


class OpenAIChatCompletionRequest(TaskInput):
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
    # further OpenAI fields that the LLM executor honours (absent from the request unless set)
    n: int | None = None
    stop: str | list[str] | None = None
    logprobs: bool | None = None
    top_logprobs: int | None = None
    # extensions: encoder outputs and KV-transfer parameters arrive through the sidecars
    cornserve_embeddings: list[DataForward[Tensor]] = []
    cornserve_kv_transfer_params: DataForward[dict] | None = None
    encoder_fission: bool = True


def extract_multimodal_content(messages: list[ChatCompletionMessageParam]) -> list[Any]:
    """All non-text content parts, in message order."""
    parts = []
    for msg in messages:
        if isinstance(msg.content, str):
            continue
        parts.extend(p for p in msg.content if not isinstance(p, (ChatCompletionContentPartTextParam, str)))
    return parts


def part_modality_and_url(part: Any) -> tuple[str, URL]:
    """``("image", URL)`` for an ``image_url`` part, and so on."""
    return part.type.split("_")[0], getattr(part, part.type)


# -- response chunks (the subset of the OpenAI chat.completion.chunk object that is produced) -----------
class ChoiceDeltaAudio(BaseModel):
    model_config = ConfigDict(extra="allow")
    id: str | None = None
    data: str | None = None
    transcript: str | None = None


class ChoiceDelta(BaseModel):
    model_config = ConfigDict(extra="allow")
    role: str | None = None
    content: str | None = None
    audio: ChoiceDeltaAudio | None = None


class ChunkChoice(BaseModel):
    model_config = ConfigDict(extra="allow")
    index: int = 0
    delta: ChoiceDelta = Field(default_factory=ChoiceDelta)
    finish_reason: str | None = None


class CompletionUsage(BaseModel):
    model_config = ConfigDict(extra="allow")
    prompt_tokens: int = 0
    completion_tokens: int = 0
    total_tokens: int = 0


class OpenAIChatCompletionChunk(TaskOutput):
    model_config = ConfigDict(extra="allow")
    id: str = ""
    object: str = "chat.completion.chunk"
    created: int = 0
    model: str = ""
    choices: list[ChunkChoice] = []
    usage: CompletionUsage | None = None


InputT = TypeVar("InputT", bound=TaskInput)
OutputT = TypeVar("OutputT", bound=TaskOutput)


class LLMBaseUnitTask(UnitTask[InputT, OutputT], Generic[InputT, OutputT]):
    """Root class of the LLM tasks that share one executor deployment per (model, receive_embeddings)."""

    model_id: str
    receive_embeddings: bool = True

    def make_name(self) -> str:
        return f"llm-{self.model_id.split('/')[-1].lower()}"

    def validate_input(self, task_input) -> None:
        if getattr(task_input, "model", self.model_id) != self.model_id:
            raise ValueError(f"Model ID in task input ({task_input.model}) does not match the task model ID "
                             f"({self.model_id}).")


@register_task
class LLMUnitTask(LLMBaseUnitTask[OpenAIChatCompletionRequest, Stream[OpenAIChatCompletionChunk]]):
    """Chat completion, streamed."""

    def make_record_output(self, task_input: OpenAIChatCompletionRequest) -> Stream[OpenAIChatCompletionChunk]:
        return Stream[OpenAIChatCompletionChunk]()


class LLMEmbeddingResponse(TaskOutput):
    embeddings: DataForward[Tensor]


@register_task
class LLMEmbeddingUnitTask(LLMBaseUnitTask[OpenAIChatCompletionRequest, LLMEmbeddingResponse]):
    """Runs the prompt through the LLM and forwards its hidden states instead of sampling text."""

    def make_record_output(self, task_input: OpenAIChatCompletionRequest) -> LLMEmbeddingResponse:
        return LLMEmbeddingResponse(embeddings=DataForward[Tensor]())


class PrefillChatCompletionResponse(TaskOutput):
    kv_transfer_params: DataForward[dict] | None = None
    hidden_states: DataForward[Tensor] | None = None


@register_task
class PrefillLLMUnitTask(UnitTask[OpenAIChatCompletionRequest, PrefillChatCompletionResponse]):
    """Prefill half of a disaggregated deployment: fills the KV cache and forwards how to fetch it."""

    model_id: str
    receive_embeddings: bool = True
    send_hidden_states: bool = False

    def make_name(self) -> str:
        return f"prefill-{self.model_id.split('/')[-1].lower()}"

    def make_record_output(self, task_input: OpenAIChatCompletionRequest) -> PrefillChatCompletionResponse:
        if self.send_hidden_states:
            return PrefillChatCompletionResponse(hidden_states=DataForward[Tensor]())
        return PrefillChatCompletionResponse(kv_transfer_params=DataForward[dict]())

    def validate_input(self, task_input: OpenAIChatCompletionRequest) -> None:
        if task_input.model != self.model_id:
            raise ValueError(f"Model ID in task input ({task_input.model}) does not match the task model ID "
                             f"({self.model_id}).")


@register_task
class DecodeLLMUnitTask(UnitTask[OpenAIChatCompletionRequest, Stream[OpenAIChatCompletionChunk]]):
    """Decode half of a disaggregated deployment: pulls the prefilled KV blocks, then generates."""

    model_id: str
    receive_embeddings: bool = True

    def make_name(self) -> str:
        return f"decode-{self.model_id.split('/')[-1].lower()}"

    def make_record_output(self, task_input: OpenAIChatCompletionRequest) -> Stream[OpenAIChatCompletionChunk]:
        return Stream[OpenAIChatCompletionChunk]()

    def validate_input(self, task_input: OpenAIChatCompletionRequest) -> None:
        if task_input.model != self.model_id:
            raise ValueError(f"Model ID in task input ({task_input.model}) does not match the task model ID "
                             f"({self.model_id}).")
        if not task_input.cornserve_kv_transfer_params:
            raise ValueError("KV transfer parameters must be specified in the task input.")
