"""Notebook / script client (reference: python/cornserve/frontend.py:60-263): a WebSocket session with the gateway
through which unit tasks are deployed and released interactively.  While the session is open a heartbeat keeps it
alive; when it closes the gateway releases everything the session deployed.  ``CORNSERVE_GATEWAY_URL`` is set so
that ``await task(input)`` dispatches through the same gateway."""

from __future__ import annotations

import json
import os
import threading
from urllib.parse import urlparse

import requests

from .constants import GATEWAY_URL
from .frontend_protocol import DeclareNotUsedRequest, DeclareUsedRequest, HeartbeatRequest, SessionRequest, SessionResponse
from .task.base import Task, UnitTaskList, discover_unit_tasks

HEARTBEAT_S = 5.0


class CornserveClient:
    def __init__(self, url: str | None = None) -> None:
        from websockets.sync.client import connect

        self.url = (url or os.environ.get("CORNSERVE_GATEWAY_URL") or GATEWAY_URL).rstrip("/")
        os.environ["CORNSERVE_GATEWAY_URL"] = self.url
        u = urlparse(self.url)
        self._ws = connect(f"{'wss' if u.scheme == 'https' else 'ws'}://{u.netloc}/session", open_timeout=30)
        self._lock = threading.Lock()
        self._closed = threading.Event()
        self._hb = threading.Thread(target=self._heartbeat, name="cornserve-heartbeat", daemon=True)
        self._hb.start()

    def _call(self, request, timeout: float = 3600.0) -> SessionResponse:
        with self._lock:
            self._ws.send(json.dumps(SessionRequest(request=request).model_dump(mode="json")))
            return SessionResponse.model_validate_json(self._ws.recv(timeout=timeout))

    def _heartbeat(self) -> None:
        while not self._closed.wait(HEARTBEAT_S):
            try:
                self._call(HeartbeatRequest(), timeout=30)
            except Exception:
                return

    def is_online(self) -> bool:
        try:
            return self._call(HeartbeatRequest(), timeout=10).status == 200
        except Exception:
            return False

    def deploy(self, task: Task) -> SessionResponse:
        """Deploy every unit task ``task`` is built from (equivalent tasks that already run are shared)."""
        units = discover_unit_tasks([task])
        return self._call(DeclareUsedRequest(task_list=UnitTaskList(tasks=units)))

    def teardown(self, task: Task) -> SessionResponse:
        units = discover_unit_tasks([task])
        return self._call(DeclareNotUsedRequest(task_list=UnitTaskList(tasks=units)))

    def deploy_tasklib(self, target: str) -> dict:
        """Upload the task classes and descriptors of a package or directory of modules."""
        from .cli.tasklib_explorer import discover_tasklib

        r = requests.post(f"{self.url}/deploy-tasks", json=discover_tasklib(target).model_dump(), timeout=300)
        r.raise_for_status()
        return r.json()

    def close(self) -> None:
        self._closed.set()
        try:
            self._ws.close()
        except Exception:
            pass

    def __enter__(self) -> "CornserveClient":
        return self

    def __exit__(self, *exc) -> None:
        self.close()
