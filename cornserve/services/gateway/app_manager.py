"""Registered applications: source loading, validation, deployment of their unit tasks, invocation
(reference: python/cornserve/services/gateway/app/manager.py:26-315)."""

from __future__ import annotations

import asyncio
import enum
import importlib.util
import inspect
import sys
import types
import uuid
from collections.abc import AsyncIterator
from dataclasses import dataclass, field
from typing import Any, get_type_hints

from pydantic import BaseModel

from ...app.base import AppConfig
from ...logging import get_logger
from ...task.base import Task, UnitTask, discover_unit_tasks
from .task_manager import TaskManager

logger = get_logger(__name__)


class AppState(enum.StrEnum):
    NOT_READY = "not ready"
    READY = "ready"


@dataclass
class AppClasses:
    request_cls: type[BaseModel]
    response_cls: type[BaseModel] | None
    config_cls: type[AppConfig]
    serve_fn: Any
    is_streaming: bool


@dataclass
class AppDefinition:
    app_id: str
    module: types.ModuleType
    source_code: str
    classes: AppClasses
    tasks: list[UnitTask] = field(default_factory=list)


def load_module_from_source(source_code: str, module_name: str) -> types.ModuleType:
    """Execute app source in a fresh module (registered in ``sys.modules`` so pydantic can resolve
    forward references)."""
    spec = importlib.util.spec_from_loader(module_name, loader=None)
    module = importlib.util.module_from_spec(spec)
    sys.modules[module_name] = module
    try:
        exec(compile(source_code, f"<app {module_name}>", "exec"), module.__dict__)
    except Exception as e:
        sys.modules.pop(module_name, None)
        raise ImportError(f"Failed to execute app source: {e}") from e
    return module


def validate_app_module(module: types.ModuleType) -> AppClasses:
    """An app needs ``class Config(AppConfig)`` and ``async def serve(request)`` whose parameter is a
    pydantic model and whose return annotation is a pydantic model or an ``AsyncIterator`` of one."""
    config = getattr(module, "Config", None)
    if not (inspect.isclass(config) and issubclass(config, AppConfig)):
        raise ValueError("App must define a `Config` class that inherits from AppConfig")
    serve = getattr(module, "serve", None)
    if serve is None or not (inspect.iscoroutinefunction(serve) or inspect.isasyncgenfunction(serve)):
        raise ValueError("App must define an `async def serve(request)` function")
    params = list(inspect.signature(serve).parameters.values())
    if len(params) != 1:
        raise ValueError("`serve` must take exactly one argument (the request)")
    hints = get_type_hints(serve)
    req_cls = hints.get(params[0].name)
    if not (inspect.isclass(req_cls) and issubclass(req_cls, BaseModel)):
        raise ValueError("The argument of `serve` must be annotated with a pydantic model")
    ret = hints.get("return")
    streaming = inspect.isasyncgenfunction(serve)
    resp_cls = None
    if ret is not None:
        origin = getattr(ret, "__origin__", None)
        if origin is not None and origin.__name__ in ("AsyncIterator", "AsyncGenerator", "AsyncIterable"):
            streaming = True
            ret = ret.__args__[0]
        if inspect.isclass(ret) and issubclass(ret, BaseModel):
            resp_cls = ret
        elif ret is not type(None) and not streaming:
            raise ValueError("`serve` must return a pydantic model (or an AsyncIterator of one)")
    for name, t in config.tasks.items():
        if not isinstance(t, Task):
            raise ValueError(f"Config.tasks[{name!r}] is not a Task")
    return AppClasses(req_cls, resp_cls, config, serve, streaming)


class AppManager:
    def __init__(self, task_manager: TaskManager) -> None:
        self.task_manager = task_manager
        self.lock = asyncio.Lock()
        self.apps: dict[str, AppDefinition] = {}
        self.app_states: dict[str, AppState] = {}
        self.running: dict[str, list[asyncio.Task]] = {}

    async def validate_and_create_app(self, source_code: str) -> tuple[str, list[str]]:
        app_id = f"app-{uuid.uuid4().hex}"
        module = load_module_from_source(source_code, app_id.replace("-", "_"))
        classes = validate_app_module(module)
        unit_tasks: list[UnitTask] = []
        for t in discover_unit_tasks(classes.config_cls.tasks.values()):
            if not any(u.is_equivalent_to(t) for u in unit_tasks):
                unit_tasks.append(t)
        async with self.lock:
            self.apps[app_id] = AppDefinition(app_id, module, source_code, classes, unit_tasks)
            self.app_states[app_id] = AppState.NOT_READY
        return app_id, [t.make_name() for t in unit_tasks]

    async def deploy_app_tasks(self, app_id: str) -> None:
        app = self.apps[app_id]
        try:
            await self.task_manager.declare_used(app.tasks)
        except Exception:
            async with self.lock:
                self.apps.pop(app_id, None)
                self.app_states.pop(app_id, None)
            sys.modules.pop(app.module.__name__, None)
            raise
        async with self.lock:
            self.app_states[app_id] = AppState.READY

    async def register_app(self, source_code: str) -> tuple[str, list[str]]:
        app_id, names = await self.validate_and_create_app(source_code)
        await self.deploy_app_tasks(app_id)
        return app_id, names

    async def unregister_app(self, app_id: str) -> None:
        async with self.lock:
            app = self.apps.pop(app_id, None)
            if app is None:
                raise KeyError(f"App {app_id} not found")
            self.app_states.pop(app_id, None)
            for t in self.running.pop(app_id, []):
                t.cancel()
        sys.modules.pop(app.module.__name__, None)
        await self.task_manager.declare_not_used(app.tasks)

    def _check_ready(self, app_id: str) -> AppDefinition:
        if app_id not in self.apps:
            raise KeyError(f"App {app_id} not found")
        if self.app_states[app_id] is not AppState.READY:
            raise ValueError(f"App {app_id} is not ready")
        return self.apps[app_id]

    def is_streaming(self, app_id: str) -> bool:
        return self._check_ready(app_id).classes.is_streaming

    async def invoke_app(self, app_id: str, request_data: dict[str, Any]) -> Any:
        """Run ``serve``.  Returns a pydantic model, or an async iterator of models for streaming apps."""
        app = self._check_ready(app_id)
        request = app.classes.request_cls(**request_data)
        if inspect.isasyncgenfunction(app.classes.serve_fn):
            return app.classes.serve_fn(request)
        job = asyncio.create_task(app.classes.serve_fn(request))
        self.running.setdefault(app_id, []).append(job)
        try:
            result = await job
        finally:
            lst = self.running.get(app_id, [])
            if job in lst:
                lst.remove(job)
        if app.classes.is_streaming and not isinstance(result, AsyncIterator) and not hasattr(result, "__aiter__"):
            raise ValueError("Streaming app did not return an async iterator")
        return result

    def list_apps(self) -> dict[str, AppState]:
        return dict(self.app_states)

    async def shutdown(self) -> None:
        for app_id in list(self.apps):
            try:
                await self.unregister_app(app_id)
            except Exception as e:
                logger.warning("Failed to unregister %s: %s", app_id, e)
