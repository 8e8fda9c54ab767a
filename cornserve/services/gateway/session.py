"""WebSocket debug sessions (reference: python/cornserve/services/gateway/session.py:26-97; client side in
``cornserve.frontend``).  A session deploys unit tasks on behalf of a notebook; when the socket
closes everything the session deployed is released."""

from __future__ import annotations

import asyncio
import uuid
from dataclasses import dataclass, field

from ...frontend_protocol import (DeclareNotUsedRequest, DeclareUsedRequest, HeartbeatRequest, SessionRequest,
                                  SessionResponse)
from ...logging import get_logger
from ...task.base import UnitTask
from .task_manager import TaskManager

logger = get_logger(__name__)


@dataclass
class Session:
    session_id: str
    tasks: list[UnitTask] = field(default_factory=list)


class SessionManager:
    def __init__(self, task_manager: TaskManager) -> None:
        self.task_manager = task_manager
        self.lock = asyncio.Lock()
        self.sessions: dict[str, Session] = {}

    async def create_session(self) -> str:
        sid = uuid.uuid4().hex
        async with self.lock:
            self.sessions[sid] = Session(sid)
        return sid

    async def handle_request(self, session_id: str, raw: dict) -> SessionResponse:
        try:
            req = SessionRequest.model_validate(raw).request
            session = self.sessions[session_id]
            if isinstance(req, HeartbeatRequest):
                return SessionResponse(status=200, content="ok")
            if isinstance(req, DeclareUsedRequest):
                tasks = req.task_list.tasks
                ids = await self.task_manager.declare_used(tasks)
                session.tasks.extend(tasks)
                return SessionResponse(status=200, content={"task_ids": ids})
            if isinstance(req, DeclareNotUsedRequest):
                tasks = req.task_list.tasks
                await self.task_manager.declare_not_used(tasks)
                for t in tasks:
                    for s in list(session.tasks):
                        if s.is_equivalent_to(t):
                            session.tasks.remove(s)
                            break
                return SessionResponse(status=200, content="released")
            return SessionResponse(status=400, content="unknown request")
        except Exception as e:
            logger.exception("Session request failed")
            return SessionResponse(status=500, content=str(e))

    async def destroy_session(self, session_id: str) -> None:
        async with self.lock:
            session = self.sessions.pop(session_id, None)
        if session and session.tasks:
            try:
                await self.task_manager.declare_not_used(session.tasks)
            except Exception:
                logger.exception("Failed to release the tasks of session %s", session_id)
