"""Task Dispatcher: turns a recorded task graph into executor calls.

For every invocation (reference: python/cornserve/services/task_dispatcher/dispatcher.py:153-318): find the
deployed unit task it is equivalent to, ask that task's manager for an executor (``GetRoute``), connect
the ``DataForward`` placeholders (outputs are producers, inputs are consumers: fill in source ranks and
append destination rank groups, so a forward consumed twice is broadcast), then call all executors
concurrently; each call is ``descriptor.to_request`` -> HTTP POST -> ``descriptor.from_response``.
Invocations of a unit task that is torn down are cancelled.
"""

from __future__ import annotations

import asyncio
import uuid
from collections.abc import Iterator
from dataclasses import dataclass
from typing import Any

import aiohttp
import grpc
from pydantic import BaseModel

from ...constants import TASK_TIMEOUT_S
from ...logging import get_logger
from ...task.base import Stream, TaskInvocation, TaskOutput, UnitTask
from ...task.forward import DataForward
from ...tracing import get_tracer
from ..pb import task_manager_pb2, task_manager_pb2_grpc
from ..task_registry.registry import TaskRegistry
from ...tracing import grpc_client_interceptors

logger = get_logger(__name__)


def _trace_configs():
    from ...tracing import aiohttp_trace_configs

    return aiohttp_trace_configs()
tracer = get_tracer(__name__)


def iter_data_forwards(obj: Any) -> Iterator[DataForward]:
    """Every ``DataForward`` reachable through model fields, lists, tuples and dict values, in order."""
    if isinstance(obj, DataForward):
        yield obj
    elif isinstance(obj, BaseModel):
        for name in type(obj).model_fields:
            yield from iter_data_forwards(getattr(obj, name))
        for v in (obj.model_extra or {}).values():
            yield from iter_data_forwards(v)
    elif isinstance(obj, (list, tuple)):
        for v in obj:
            yield from iter_data_forwards(v)
    elif isinstance(obj, dict):
        for v in obj.values():
            yield from iter_data_forwards(v)


def connect_forwards(executions: list["UnitTaskExecution"]) -> None:
    """Fill ``src_sidecar_ranks`` / ``dst_sidecar_ranks`` of all forwards of a graph, in place."""
    producers: dict[str, DataForward] = {}
    for ex in executions:
        for consumer in iter_data_forwards(ex.invocation.task_input):
            producer = producers.get(consumer.id)
            if producer is None:
                raise ValueError(f"DataForward {consumer.id} in the input of {type(ex.invocation.task).__name__} "
                                 "was not produced by an earlier invocation.")
            if producer.dst_sidecar_ranks is None:
                producer.dst_sidecar_ranks = []
            producer.dst_sidecar_ranks.append(ex.sidecar_ranks)
            consumer.src_sidecar_ranks = producer.src_sidecar_ranks
            consumer.dst_sidecar_ranks = producer.dst_sidecar_ranks
        for producer in iter_data_forwards(ex.invocation.task_output):
            producer.src_sidecar_ranks = ex.sidecar_ranks
            producers[producer.id] = producer
    for p in producers.values():
        if p.dst_sidecar_ranks is None:
            p.dst_sidecar_ranks = []  # produced but never consumed: nothing is sent


@dataclass
class UnitTaskExecution:
    invocation: TaskInvocation
    executor_url: str
    sidecar_ranks: list[int]

    @property
    def is_streaming(self) -> bool:
        return isinstance(self.invocation.task_output, Stream)


@dataclass
class TaskInfo:
    task: UnitTask
    instance_name: str
    task_manager_url: str
    channel: grpc.aio.Channel
    stub: task_manager_pb2_grpc.TaskManagerStub


class TaskDispatcher:
    def __init__(self, registry: TaskRegistry | None = None) -> None:
        self.registry = registry or TaskRegistry()
        self.task_lock = asyncio.Lock()
        self.task_infos: dict[str, TaskInfo] = {}
        self.ongoing_lock = asyncio.Lock()
        self.ongoing: dict[str, list[asyncio.Task]] = {}
        self._client: aiohttp.ClientSession | None = None

    @property
    def client(self) -> aiohttp.ClientSession:
        if self._client is None or self._client.closed:
            self._client = aiohttp.ClientSession(trace_configs=_trace_configs(), timeout=aiohttp.ClientTimeout(total=TASK_TIMEOUT_S),
                                                 connector=aiohttp.TCPConnector(limit=0))
        return self._client

    # -- deployment notifications ---------------------------------------------------------------------------
    async def notify_task_deployment(self, instance_name: str, task_manager_url: str) -> None:
        task = await self.registry.get_task_instance(instance_name)
        channel = grpc.aio.insecure_channel(task_manager_url, interceptors=grpc_client_interceptors())
        info = TaskInfo(task, instance_name, task_manager_url, channel, task_manager_pb2_grpc.TaskManagerStub(channel))
        async with self.task_lock:
            old = self.task_infos.pop(instance_name, None)
            self.task_infos[instance_name] = info
        if old is not None:
            await old.channel.close()
        logger.info("Registered unit task %s (manager at %s)", instance_name, task_manager_url)

    async def notify_task_teardown(self, instance_name: str) -> None:
        async with self.task_lock:
            info = self.task_infos.pop(instance_name, None)
        if info is None:
            raise ValueError(f"Unit task {instance_name} not found")
        async with self.ongoing_lock:
            for t in self.ongoing.pop(instance_name, []):
                t.cancel()
        await info.channel.close()
        logger.info("Removed unit task %s", instance_name)

    # -- invocation ----------------------------------------------------------------------------------------------
    async def invoke(self, invocations: list[TaskInvocation]) -> list[TaskOutput]:
        with tracer.start_as_current_span("TaskDispatcher.invoke"):
            async with self.task_lock:
                infos: list[TaskInfo] = []
                for inv in invocations:
                    match = next((i for i in self.task_infos.values() if i.task.is_equivalent_to(inv.task)), None)
                    if match is None:
                        raise ValueError(f"Unit task {type(inv.task).__name__}({inv.task.make_name()}) is not deployed")
                    infos.append(match)
            request_id = uuid.uuid4().hex
            routes = await asyncio.gather(*(i.stub.GetRoute(task_manager_pb2.GetRouteRequest(request_id=request_id))
                                            for i in infos))
            executions = [UnitTaskExecution(inv, r.task_executor_url, list(r.sidecar_ranks))
                          for inv, r in zip(invocations, routes)]
            connect_forwards(executions)
            current = asyncio.current_task()
            async with self.ongoing_lock:
                for i in infos:
                    self.ongoing.setdefault(i.instance_name, []).append(current)
            try:
                async with asyncio.TaskGroup() as tg:
                    jobs = [tg.create_task(self._execute(ex)) for ex in executions]
            except* Exception as eg:  # noqa: E999
                raise RuntimeError(f"Task invocation failed: {[str(e) for e in eg.exceptions]}") from eg
            finally:
                async with self.ongoing_lock:
                    for i in infos:
                        lst = self.ongoing.get(i.instance_name, [])
                        if current in lst:
                            lst.remove(current)
            return [j.result() for j in jobs]

    async def _execute(self, ex: UnitTaskExecution) -> TaskOutput:
        desc = ex.invocation.task.execution_descriptor
        body = desc.to_request(task_input=ex.invocation.task_input, task_output=ex.invocation.task_output)
        url = desc.get_api_url(ex.executor_url)
        try:
            resp = await self.client.post(url, json=body)
            if resp.status >= 400:
                text = await resp.text()
                raise RuntimeError(f"HTTP request to {url} failed with code {resp.status}: {text[:500]}")
        except aiohttp.ClientError as e:
            raise RuntimeError(f"HTTP request to {url} failed: {e}") from e
        return await desc.from_response(task_output=ex.invocation.task_output, response=resp)

    async def shutdown(self) -> None:
        async with self.ongoing_lock:
            for tasks in self.ongoing.values():
                for t in tasks:
                    t.cancel()
        async with self.task_lock:
            for i in self.task_infos.values():
                await i.channel.close()
            self.task_infos.clear()
        if self._client is not None and not self._client.closed:
            await self._client.close()
