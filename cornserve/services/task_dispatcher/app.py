"""HTTP and gRPC faces of the Task Dispatcher (reference: python/cornserve/services/task_dispatcher/
router.py:21-54 and grpc.py:21-72).  ``POST /task`` answers with the JSON list of outputs, or, for a
streaming graph, with ``text/plain`` lines: first the list of outputs, then the raw stream chunks."""

from __future__ import annotations

import json
from collections.abc import AsyncGenerator

import grpc
from fastapi import FastAPI, Request, Response
from fastapi.responses import StreamingResponse

from ...logging import get_logger
from ...task.base import Stream, TaskGraphDispatch, TaskOutput
from ..pb import common_pb2, task_dispatcher_pb2, task_dispatcher_pb2_grpc
from .dispatcher import TaskDispatcher
from ...tracing import grpc_server_interceptors

logger = get_logger(__name__)
OK, ERROR = common_pb2.STATUS_OK, common_pb2.STATUS_ERROR


def create_app(dispatcher: TaskDispatcher) -> FastAPI:
    app = FastAPI(title="cornserve-b200 task dispatcher")
    from ...tracing import instrument_fastapi

    instrument_fastapi(app, "cornserve.task-dispatcher")
    app.state.dispatcher = dispatcher

    @app.post("/task")
    async def invoke_task(request: Request):
        try:
            await dispatcher.registry.sync_watchers()
            graph = TaskGraphDispatch.model_validate(await request.json())
            results = await dispatcher.invoke(graph.invocations)
        except Exception as e:
            logger.exception("Error while invoking task")
            return Response(status_code=500, content=str(e))
        if not graph.is_streaming:
            return [r.model_dump() for r in results]

        async def lines(outs: list[TaskOutput]) -> AsyncGenerator[bytes, None]:
            yield (json.dumps([r.model_dump() for r in outs]) + "\n").encode()
            stream = outs[-1]
            assert isinstance(stream, Stream)
            async for chunk in stream.aiter_raw():
                yield (chunk if isinstance(chunk, bytes) else chunk.encode()) + b"\n"

        return StreamingResponse(lines(results), media_type="text/plain")

    @app.get("/health")
    async def health():
        return {"status": "ok", "tasks": sorted(dispatcher.task_infos)}

    return app


class TaskDispatcherServicer(task_dispatcher_pb2_grpc.TaskDispatcherServicer):
    def __init__(self, dispatcher: TaskDispatcher):
        self.dispatcher = dispatcher

    async def NotifyUnitTaskDeployment(self, request, context):
        try:
            await self.dispatcher.registry.sync_watchers()
            await self.dispatcher.notify_task_deployment(request.task_instance_name, request.task_manager.url)
        except Exception as e:
            logger.exception("NotifyUnitTaskDeployment failed")
            await context.abort(grpc.StatusCode.INTERNAL, str(e))
        return task_dispatcher_pb2.NotifyUnitTaskDeploymentResponse(status=OK)

    async def NotifyUnitTaskTeardown(self, request, context):
        try:
            await self.dispatcher.notify_task_teardown(request.task_instance_name)
        except ValueError as e:
            await context.abort(grpc.StatusCode.NOT_FOUND, str(e))
        return task_dispatcher_pb2.NotifyUnitTaskTeardownResponse(status=OK)

    async def SyncTaskRegistry(self, request, context):
        try:
            await self.dispatcher.registry.sync_watchers()
            return common_pb2.SyncTaskRegistryResponse(status=OK)
        except Exception:
            logger.exception("SyncTaskRegistry failed")
            return common_pb2.SyncTaskRegistryResponse(status=ERROR)


async def start_grpc(dispatcher: TaskDispatcher, address: str) -> grpc.aio.Server:
    server = grpc.aio.server(interceptors=grpc_server_interceptors())
    task_dispatcher_pb2_grpc.add_TaskDispatcherServicer_to_server(TaskDispatcherServicer(dispatcher), server)
    server.add_insecure_port(address)
    await server.start()
    return server
