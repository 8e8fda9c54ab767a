"""Application configuration base (reference: python/cornserve/app/base.py:12-23).  An app module defines
``class Config(AppConfig)`` whose ``tasks`` class variable names every task the app invokes, plus an
``async def serve(request)`` that returns a response or an async iterator of responses."""

from __future__ import annotations

from typing import ClassVar

from pydantic import BaseModel, ConfigDict

from ..task.base import Task


class AppRequest(BaseModel):
    """Optional base for app request models."""


class AppResponse(BaseModel):
    """Optional base for app response models."""


class AppConfig(BaseModel):
    tasks: ClassVar[dict[str, Task]] = {}

    model_config = ConfigDict(extra="forbid")
