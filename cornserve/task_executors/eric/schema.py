"""Internal data model of the encoder executor (reference: python/cornserve/task_executors/eric/schema.py)."""

from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Any

import torch


class Modality(enum.StrEnum):
    IMAGE = "image"
    VIDEO = "video"
    AUDIO = "audio"


class Status(enum.IntEnum):
    SUCCESS = 0
    ERROR = 1


@dataclass
class ProcessedItem:
    """One multimodal item after CPU preprocessing: the model-specific tensors (``processed``) keyed as
    the model's ``forward`` expects them."""

    id: str
    modality: Modality
    model_id: str
    processed: dict[str, torch.Tensor | Any]
    receiver_sidecar_ranks: list[list[int]] | None = None


@dataclass
class EngineRequest:
    request_id: str
    items: list[ProcessedItem]
    trace_carrier: dict[str, str] = field(default_factory=dict)


@dataclass
class EngineResponse:
    request_id: str
    status: Status
    error_message: str | None = None


@dataclass
class Batch:
    """Items that share modality and adapter, executed in one forward pass."""

    modality: Modality
    adapter_name: str
    request_ids: list[str]
    data_ids: list[str]
    receiver_ranks: list[list[list[int]] | None]
    data: dict[str, list[Any]]
    trace_carriers: list[dict[str, str]] = field(default_factory=list)
