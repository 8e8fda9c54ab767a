"""HTTP schema of the monolithic baseline executor (wire-compatible with
python/cornserve/task_executors/huggingface/api.py:11-90)."""

from __future__ import annotations

import enum

from pydantic import BaseModel


class ModelType(enum.StrEnum):
    QWEN_IMAGE = "QWEN_IMAGE"
    QWEN_OMNI = "QWEN_OMNI"


class StreamOptions(BaseModel):
    include_usage: bool = True


class HuggingFaceRequest(BaseModel):
    # image generation
    prompt: str | None = None
    height: int | None = None
    width: int | None = None
    num_inference_steps: int | None = None
    # omni chat
    messages: list[dict] | None = None
    model: str | None = None
    frequency_penalty: float | None = 0.0
    max_completion_tokens: int | None = None
    presence_penalty: float | None = 0.0
    seed: int | None = None
    stream_options: StreamOptions | None = None
    temperature: float | None = None
    top_p: float | None = None
    ignore_eos: bool = False
    return_audio: bool | None = None
    request_id: str | None = None
    model_type: str | None = None


class Status(enum.IntEnum):
    SUCCESS = 0
    ERROR = 1


class HuggingFaceResponse(BaseModel):
    status: Status
    image: str | None = None          # base64 PNG
    audio_chunk: str | None = None    # base64 float32 waveform
    text_chunk: dict | None = None    # OpenAI chat-completion chunk
    error_message: str | None = None
