"""Internal data model of the generator executor (reference: python/cornserve/task_executors/geri/schema.py)."""

from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Any

import torch


class GeriMode(enum.Enum):
    BATCH = "batch"          # one response per request (images)
    STREAMING = "streaming"  # a stream of chunks per request (audio)


class Status(enum.IntEnum):
    SUCCESS = 0
    ERROR = 1
    FINISHED = 2


@dataclass
class EngineRequest:
    """One generation request; ``embeds`` are the conditioning chunks received through the sidecar (already
    concatenated and trimmed), ``params`` the modality-specific knobs that decide batch compatibility."""

    request_id: str
    embeds: torch.Tensor
    params: dict[str, Any]
    negative_embeds: torch.Tensor | None = None
    trace_carrier: dict[str, str] = field(default_factory=dict)

    def batch_key(self) -> tuple:
        return tuple(sorted((k, v) for k, v in self.params.items())) + (self.negative_embeds is not None,)


@dataclass
class EngineResponse:
    request_id: str
    status: Status
    generated: Any = None
    error_message: str | None = None


@dataclass
class Batch:
    requests: list[EngineRequest]

    @property
    def request_ids(self) -> list[str]:
        return [r.request_id for r in self.requests]

    @property
    def params(self) -> dict[str, Any]:
        return self.requests[0].params
