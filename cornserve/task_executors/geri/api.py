"""HTTP schema of the generator executor (wire-compatible with python/cornserve/task_executors/geri/api.py:11-117)."""

from __future__ import annotations

import enum

from pydantic import BaseModel, ConfigDict, RootModel


class Status(enum.IntEnum):
    SUCCESS = 0
    ERROR = 1
    FINISHED = 2


class Modality(enum.StrEnum):
    IMAGE = "image"
    VIDEO = "video"
    AUDIO = "audio"


class BatchGeriRequest(BaseModel):
    """Requests answered with one response; ``embedding_data_id`` names the forwarded conditioning tensor."""

    embedding_data_id: str


class StreamGeriRequest(BaseModel):
    """Requests answered with a stream of chunks."""

    embedding_data_id: str


class ImageGeriRequest(BatchGeriRequest):
    height: int
    width: int
    num_inference_steps: int
    skip_tokens: int = 0


class AudioGeriRequest(StreamGeriRequest):
    chunk_size: int | None = None
    left_context_size: int | None = None


class BatchGeriResponse(BaseModel):
    status: Status
    generated: str | None = None  # base64 (PNG for images)
    error_message: str | None = None


class StreamGeriResponseChunk(RootModel[bytes]):
    """One unit of a streamed response; bytes travel as base64 inside JSON."""

    model_config = ConfigDict(ser_json_bytes="base64", val_json_bytes="base64")
