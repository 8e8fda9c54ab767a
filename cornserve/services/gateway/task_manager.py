"""Gateway-side registry of deployed unit tasks with usage counting (reference:
python/cornserve/services/gateway/task_manager.py:46-377).

``declare_used`` is transactional: instances are written to the registry and ``DeployUnitTask`` is
called for all new tasks in parallel; on any failure everything this call created is rolled back.
Equivalent tasks are deployed once and shared; ``declare_not_used`` tears a task down when its last user
leaves and cancels invocations that are still running on it.
"""

from __future__ import annotations

import asyncio
import enum
import uuid
from collections import defaultdict
from typing import Any

import aiohttp
import grpc

from ...constants import RESOURCE_MANAGER_GRPC_URL, TASK_DISPATCHER_HTTP_URL, TASK_TIMEOUT_S
from ...logging import get_logger
from ...task.base import TaskGraphDispatch, UnitTask
from ..pb import resource_manager_pb2, resource_manager_pb2_grpc
from ..task_registry.registry import TaskRegistry
from ...tracing import grpc_client_interceptors

logger = get_logger(__name__)


def _trace_configs():
    from ...tracing import aiohttp_trace_configs

    return aiohttp_trace_configs()


class TaskState(enum.StrEnum):
    DEPLOYING = "not ready"
    READY = "ready"
    TEARING_DOWN = "tearing down"


class TaskManager:
    def __init__(self, resource_manager_grpc_url: str = RESOURCE_MANAGER_GRPC_URL,
                 task_dispatcher_http_url: str = TASK_DISPATCHER_HTTP_URL, registry: TaskRegistry | None = None) -> None:
        self.registry = registry or TaskRegistry()
        self.lock = asyncio.Lock()
        self.tasks: dict[str, UnitTask] = {}          # task id (= instance name) -> task
        self.task_states: dict[str, TaskState] = {}
        self.task_usage: dict[str, int] = defaultdict(int)
        self.invocation_tasks: dict[str, list[asyncio.Task]] = defaultdict(list)
        self.dispatcher_url = task_dispatcher_http_url
        self._rm_channel = grpc.aio.insecure_channel(resource_manager_grpc_url, interceptors=grpc_client_interceptors())
        self.resource_manager = resource_manager_pb2_grpc.ResourceManagerStub(self._rm_channel)
        self._client: aiohttp.ClientSession | None = None

    @property
    def client(self) -> aiohttp.ClientSession:
        if self._client is None or self._client.closed:
            self._client = aiohttp.ClientSession(trace_configs=_trace_configs(), timeout=aiohttp.ClientTimeout(total=TASK_TIMEOUT_S),
                                                 connector=aiohttp.TCPConnector(limit=0))
        return self._client

    def _find_equivalent(self, task: UnitTask) -> str | None:
        return next((tid for tid, t in self.tasks.items() if t.is_equivalent_to(task)), None)

    async def declare_used(self, tasks: list[UnitTask]) -> list[str]:
        """Make sure every task is deployed; returns the ids of the deployments that now back them."""
        async with self.lock:
            snapshot = (dict(self.tasks), dict(self.task_states), dict(self.task_usage))
            created: list[str] = []
            ids: list[str] = []
            to_deploy: list[tuple[str, UnitTask]] = []
            try:
                for task in tasks:
                    tid = self._find_equivalent(task)
                    if tid is None:
                        tid = await self.registry.create_task_instance_from_task(task, uuid.uuid4().hex[:12])
                        created.append(tid)
                        self.tasks[tid] = task
                        self.task_states[tid] = TaskState.DEPLOYING
                        to_deploy.append((tid, task))
                    self.task_usage[tid] += 1
                    ids.append(tid)
                results = await asyncio.gather(
                    *(self.resource_manager.DeployUnitTask(resource_manager_pb2.DeployUnitTaskRequest(task_instance_name=t))
                      for t, _ in to_deploy), return_exceptions=True)
                errors = [r for r in results if isinstance(r, BaseException)]
                if errors:
                    raise RuntimeError(f"Failed to deploy {len(errors)} unit task(s): "
                                       f"{[getattr(e, 'details', lambda: str(e))() for e in errors]}")
                for tid, _ in to_deploy:
                    self.task_states[tid] = TaskState.READY
                return ids
            except BaseException:
                logger.exception("Deployment failed; rolling back %s", created)
                deployed_ok = [tid for (tid, _), r in zip(to_deploy, results if "results" in locals() else [])
                               if not isinstance(r, BaseException)]
                for tid in deployed_ok:
                    try:
                        await self.resource_manager.TeardownUnitTask(
                            resource_manager_pb2.TeardownUnitTaskRequest(task_instance_name=tid))
                    except Exception as e:
                        logger.warning("Rollback teardown of %s failed: %s", tid, e)
                for tid in created:
                    await self.registry.delete_task_instance(tid)
                self.tasks, self.task_states = snapshot[0], snapshot[1]
                self.task_usage = defaultdict(int, snapshot[2])
                raise

    async def declare_not_used(self, tasks: list[UnitTask]) -> None:
        async with self.lock:
            doomed: list[str] = []
            for task in tasks:
                tid = self._find_equivalent(task)
                if tid is None:
                    logger.warning("Task %s was not deployed", task.make_name())
                    continue
                self.task_usage[tid] -= 1
                if self.task_usage[tid] <= 0:
                    self.task_usage.pop(tid, None)
                    self.task_states[tid] = TaskState.TEARING_DOWN
                    doomed.append(tid)
            for tid in doomed:
                for t in self.invocation_tasks.pop(tid, []):
                    t.cancel()
            results = await asyncio.gather(
                *(self.resource_manager.TeardownUnitTask(resource_manager_pb2.TeardownUnitTaskRequest(task_instance_name=t))
                  for t in doomed), return_exceptions=True)
            for tid, r in zip(doomed, results):
                if isinstance(r, BaseException):
                    logger.error("Teardown of %s failed: %s", tid, r)
                self.tasks.pop(tid, None)
                self.task_states.pop(tid, None)
                await self.registry.delete_task_instance(tid)

    async def scale_unit_task(self, task_id: str, num_gpus: int) -> None:
        if task_id not in self.tasks:
            raise KeyError(f"Unit task {task_id} not found")
        await self.resource_manager.ScaleUnitTask(
            resource_manager_pb2.ScaleUnitTaskRequest(task_instance_name=task_id, num_gpus=num_gpus))

    def list_tasks(self) -> list[tuple[str, UnitTask, TaskState]]:
        return [(tid, t, self.task_states[tid]) for tid, t in self.tasks.items()]

    async def invoke_tasks(self, dispatch: TaskGraphDispatch) -> list[Any]:
        """Send a recorded graph to the task dispatcher.  Every unit task in it must be READY."""
        involved: list[str] = []
        for inv in dispatch.invocations:
            tid = self._find_equivalent(inv.task)
            if tid is None:
                raise KeyError(f"Unit task {inv.task.make_name()} is not deployed")
            if self.task_states.get(tid) is not TaskState.READY:
                raise ValueError(f"Unit task {tid} is {self.task_states.get(tid)}")
            involved.append(tid)
        current = asyncio.current_task()
        for tid in involved:
            self.invocation_tasks[tid].append(current)
        try:
            return await dispatch.dispatch(self.dispatcher_url + "/task", self.client)
        finally:
            for tid in involved:
                lst = self.invocation_tasks.get(tid, [])
                if current in lst:
                    lst.remove(current)

    async def shutdown(self) -> None:
        async with self.lock:
            for tid in list(self.tasks):
                try:
                    await self.resource_manager.TeardownUnitTask(
                        resource_manager_pb2.TeardownUnitTaskRequest(task_instance_name=tid))
                except Exception as e:
                    logger.warning("Teardown of %s during shutdown failed: %s", tid, e)
                await self.registry.delete_task_instance(tid)
            self.tasks.clear()
            self.task_states.clear()
            self.task_usage.clear()
        if self._client is not None and not self._client.closed:
            await self._client.close()
        await self._rm_channel.close()
