"""Task execution descriptors: how one kind of unit task is launched and called.

Reference: python/cornserve/task_executors/descriptor/base.py:21-91.  The reference builds Kubernetes
pod specs; here an executor is a local process, so a descriptor produces a :class:`LaunchSpec`
(argv + environment + GPUs).  The reference's method names (``get_container_args`` ...) are kept so
that user-written descriptors keep working; ``get_container_image`` is informational only.
"""

from __future__ import annotations

import sys
from abc import ABC, abstractmethod
from dataclasses import dataclass, field
from typing import Any, Generic, TypeVar

from pydantic import BaseModel

from ...services.resource import GPU
from ...task.base import TaskInput, TaskOutput, UnitTask

TaskT = TypeVar("TaskT", bound=UnitTask)
InputT = TypeVar("InputT", bound=TaskInput)
OutputT = TypeVar("OutputT", bound=TaskOutput)


@dataclass
class LaunchSpec:
    """Everything the task manager needs to start one executor process."""

    argv: list[str]
    env: dict[str, str] = field(default_factory=dict)
    gpus: list[int] = field(default_factory=list)
    port: int = 0
    name: str = ""


class TaskExecutionDescriptor(BaseModel, ABC, Generic[TaskT, InputT, OutputT]):
    task: TaskT

    model_config = {"arbitrary_types_allowed": True}

    @abstractmethod
    def create_executor_name(self) -> str:
        """Short name used in process names and logs."""

    def get_container_image(self) -> str:
        return "local-process"

    def get_entrypoint(self) -> list[str]:
        """Interpreter + module that implements the executor."""
        return [sys.executable, "-m", "cornserve.task_executors.generic"]

    @abstractmethod
    def get_container_args(self, gpus: list[GPU], port: int) -> list[str]:
        """Command-line arguments of the executor."""

    def get_container_volumes(self) -> list[tuple[str, str, str]]:
        return []

    def get_service_ports(self, gpus: list[GPU]) -> list[tuple[str, int]]:
        return []

    def get_container_envs(self, gpus: list[GPU]) -> list[tuple[str, str]]:
        return [("CUDA_VISIBLE_DEVICES", ",".join(str(g.local_rank) for g in gpus))]

    def get_kubernetes_envs(self, gpus: list[GPU]) -> list[Any]:
        return []

    def launch_spec(self, gpus: list[GPU], port: int, extra_args: list[str] | None = None) -> LaunchSpec:
        env = dict(self.get_container_envs(gpus))
        argv = [*self.get_entrypoint(), *self.get_container_args(gpus, port), *(extra_args or [])]
        return LaunchSpec(argv=argv, env=env, gpus=[g.global_rank for g in gpus], port=port,
                          name=self.create_executor_name())

    @abstractmethod
    def get_api_url(self, base: str) -> str:
        """URL of the executor endpoint that runs the task."""

    @abstractmethod
    def to_request(self, task_input: InputT, task_output: OutputT) -> dict[str, Any]:
        """JSON body for the executor from the task input (and the recorded output with its forwards)."""

    @abstractmethod
    async def from_response(self, task_output: OutputT, response: Any) -> OutputT:
        """Task output from the executor's HTTP response (``aiohttp.ClientResponse``)."""
