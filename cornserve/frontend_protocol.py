"""Messages of the gateway's WebSocket session protocol (verbs as in python/cornserve/frontend.py:22-58)."""

from __future__ import annotations

from typing import Any, Literal

from pydantic import BaseModel, Field

from .task.base import UnitTaskList


class DeclareUsedRequest(BaseModel):
    verb: Literal["declare_used"] = "declare_used"
    task_list: UnitTaskList


class DeclareNotUsedRequest(BaseModel):
    verb: Literal["declare_not_used"] = "declare_not_used"
    task_list: UnitTaskList


class HeartbeatRequest(BaseModel):
    verb: Literal["heartbeat"] = "heartbeat"


class SessionRequest(BaseModel):
    request: DeclareUsedRequest | DeclareNotUsedRequest | HeartbeatRequest = Field(discriminator="verb")


class SessionResponse(BaseModel):
    status: int
    content: Any = None
