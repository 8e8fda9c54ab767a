"""HTTP schema of the encoder executor (wire-compatible with python/cornserve/task_executors/eric/api.py:20-60)."""

from __future__ import annotations

import enum

from pydantic import BaseModel

ID = str


class Modality(enum.StrEnum):
    IMAGE = "image"
    VIDEO = "video"
    AUDIO = "audio"


class EmbeddingData(BaseModel):
    """One item to embed.  ``receiver_sidecar_ranks`` lists the consumer groups; ``None`` = do not send."""

    id: ID
    modality: Modality
    model_id: str
    url: str
    receiver_sidecar_ranks: list[list[int]] | None = None


class EmbeddingRequest(BaseModel):
    data: list[EmbeddingData]


class Status(enum.IntEnum):
    SUCCESS = 0
    ERROR = 1


class EmbeddingResponse(BaseModel):
    status: Status
    error_message: str | None = None
