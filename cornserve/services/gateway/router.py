"""REST / WebSocket API of the gateway (endpoints as in python/cornserve/services/gateway/router.py:99-547)."""

from __future__ import annotations

import asyncio
import contextlib
import json
from collections.abc import AsyncGenerator
from typing import Any

import grpc
from fastapi import APIRouter, FastAPI, Request, Response, WebSocket, WebSocketDisconnect
from fastapi.responses import JSONResponse, StreamingResponse
from pydantic import BaseModel

from ...constants import RESOURCE_MANAGER_GRPC_URL, TASK_DISPATCHER_GRPC_URL, TASK_DISPATCHER_HTTP_URL
from ...task_executors.profile import UnitTaskProfile, UnitTaskProfileManager
from ...logging import get_logger
from ...task.base import Stream, TaskGraphDispatch, UnitTaskList, task_manager_context
from ..pb import common_pb2, resource_manager_pb2_grpc, task_dispatcher_pb2_grpc
from ..task_registry import DESCRIPTOR_REGISTRY, TASK_CLASS_REGISTRY
from ..task_registry.registry import TaskRegistry
from .app_manager import AppManager
from .models import (AppInvocationRequest, AppRegistrationRequest, ProfilesDeploymentRequest, ReconcileRequest,
                     RegistrationErrorResponse, RegistrationFinalResponse, RegistrationInitialResponse,
                     RegistrationStatusEvent, ScaleTaskRequest, TasksDeploymentRequest)
from .session import SessionManager
from .task_manager import TaskManager

logger = get_logger(__name__)
router = APIRouter()


async def sync_control_plane(app: FastAPI) -> None:
    """Ask the resource manager and every dispatcher to catch up with the registry, then catch up here."""
    async def one(stub_cls, url):
        async with grpc.aio.insecure_channel(url) as ch:
            r = await stub_cls(ch).SyncTaskRegistry(common_pb2.SyncTaskRegistryRequest(), timeout=60)
            if r.status != common_pb2.STATUS_OK:
                raise RuntimeError(f"{url} failed to sync its task registry")

    jobs = [one(resource_manager_pb2_grpc.ResourceManagerStub, app.state.resource_manager_grpc_url)]
    jobs += [one(task_dispatcher_pb2_grpc.TaskDispatcherStub, u) for u in app.state.task_dispatcher_grpc_urls]
    await asyncio.gather(*jobs, app.state.task_registry.sync_watchers())


def _dump(obj: Any) -> Any:
    return obj.model_dump() if isinstance(obj, BaseModel) else obj


@router.post("/app/register")
async def register_app(request: AppRegistrationRequest, raw: Request):
    manager: AppManager = raw.app.state.app_manager

    async def events() -> AsyncGenerator[str]:
        app_id = None
        try:
            if not TASK_CLASS_REGISTRY.list_registered_unit_tasks() and await raw.app.state.task_registry.check_emptiness():
                raise ValueError("No task definitions are known. Deploy a task library first (`cornserve tasklib deploy`).")
            app_id, names = await manager.validate_and_create_app(request.source_code)
            yield f"data: {RegistrationStatusEvent(event=RegistrationInitialResponse(app_id=app_id, task_names=names)).model_dump_json()}\n\n"
            await manager.deploy_app_tasks(app_id)
            msg = f"Successfully deployed {len(names)} unit tasks"
            yield f"data: {RegistrationStatusEvent(event=RegistrationFinalResponse(message=msg)).model_dump_json()}\n\n"
        except Exception as e:
            logger.exception("Error during app registration for app_id '%s'", app_id)
            yield f"data: {RegistrationStatusEvent(event=RegistrationErrorResponse(message=str(e))).model_dump_json()}\n\n"

    return StreamingResponse(events(), media_type="text/event-stream",
                             headers={"Cache-Control": "no-cache", "Connection": "keep-alive"})


@router.post("/app/unregister/{app_id}")
async def unregister_app(app_id: str, raw: Request):
    try:
        await raw.app.state.app_manager.unregister_app(app_id)
        return Response(status_code=200)
    except KeyError as e:
        return Response(status_code=404, content=str(e))
    except Exception as e:
        logger.exception("Unexpected error while unregistering app")
        return Response(status_code=500, content=str(e))


@router.post("/app/invoke/{app_id}")
async def invoke_app(app_id: str, request: AppInvocationRequest, raw: Request):
    manager: AppManager = raw.app.state.app_manager
    try:
        result = await manager.invoke_app(app_id, request.request_data)
    except KeyError as e:
        return Response(status_code=404, content=str(e))
    except ValueError as e:
        return Response(status_code=400, content=str(e))
    except Exception as e:
        logger.exception("Unexpected error while running app %s", app_id)
        return Response(status_code=500, content=str(e))
    if hasattr(result, "__aiter__"):
        async def lines() -> AsyncGenerator[str]:
            try:
                async for item in result:
                    yield (item.model_dump_json() if isinstance(item, BaseModel) else json.dumps(item)) + "\n"
            except Exception as e:
                logger.exception("Streaming app %s failed", app_id)
                yield json.dumps({"error": str(e)}) + "\n"

        return StreamingResponse(lines(), media_type="text/plain")
    return JSONResponse(_dump(result))


@router.get("/app/list")
async def list_apps(raw: Request):
    return {k: v.value for k, v in raw.app.state.app_manager.list_apps().items()}


@router.websocket("/session")
async def session(socket: WebSocket):
    await socket.accept()
    sessions: SessionManager = socket.app.state.session_manager
    sid = await sessions.create_session()
    try:
        while True:
            resp = await sessions.handle_request(sid, await socket.receive_json())
            await socket.send_text(resp.model_dump_json())
    except WebSocketDisconnect:
        pass
    except Exception:
        logger.exception("Session %s failed", sid)
    finally:
        await sessions.destroy_session(sid)


@router.post("/task/register")
async def register_task(raw: Request):
    return Response(status_code=501, content="Use /deploy-tasks to upload task classes")


@router.post("/task/scale")
async def scale_task(request: ScaleTaskRequest, raw: Request):
    if request.num_gpus == 0:
        return Response(status_code=400, content="Scaling 0 GPUs has no effect.")
    try:
        await raw.app.state.task_manager.scale_unit_task(request.task_id, request.num_gpus)
        return Response(status_code=200)
    except KeyError as e:
        return Response(status_code=404, content=str(e))
    except grpc.aio.AioRpcError as e:
        return Response(status_code=400 if e.code() == grpc.StatusCode.INVALID_ARGUMENT else 500, content=e.details())
    except Exception as e:
        logger.exception("Unexpected error while scaling")
        return Response(status_code=500, content=str(e))


@router.post("/task/reconcile")
async def reconcile_task(request: ReconcileRequest, raw: Request):
    """Load-driven scaling: the task's manager converts the target load into a GPU count (not in the reference)."""
    rm = raw.app.state.resource_manager_local
    if rm is None:
        return Response(status_code=501, content="Reconcile needs an in-process resource manager")
    try:
        return {"message": await rm.reconcile(request.task_id, request.target_load)}
    except KeyError as e:
        return Response(status_code=404, content=str(e))


@router.get("/tasks/list")
async def list_tasks(raw: Request):
    return [[t.model_dump_json(), tid, st.value] for tid, t, st in raw.app.state.task_manager.list_tasks()]


@router.post("/tasks/usage")
async def declare_task_usage(raw: Request):
    try:
        tasks = UnitTaskList.model_validate(await raw.json()).tasks
        ids = await raw.app.state.task_manager.declare_used(tasks)
        return {"task_ids": ids}
    except Exception as e:
        logger.exception("Unexpected error while declaring task usage")
        return Response(status_code=500, content=str(e))


@router.delete("/tasks/usage")
async def declare_unused_tasks(raw: Request):
    try:
        tasks = UnitTaskList.model_validate(await raw.json()).tasks
        await raw.app.state.task_manager.declare_not_used(tasks)
        return Response(status_code=200)
    except Exception as e:
        logger.exception("Unexpected error while releasing tasks")
        return Response(status_code=500, content=str(e))


@router.post("/tasks/invoke")
async def invoke_tasks(raw: Request):
    """Invoke a recorded task graph on behalf of a client outside the gateway (notebooks, scripts)."""
    try:
        graph = TaskGraphDispatch.model_validate(await raw.json())
        results = await raw.app.state.task_manager.invoke_tasks(graph)
    except KeyError as e:
        return Response(status_code=404, content=str(e))
    except ValueError as e:
        return Response(status_code=400, content=str(e))
    except Exception as e:
        logger.exception("Unexpected error while invoking tasks")
        return Response(status_code=500, content=str(e))
    if not graph.is_streaming:
        return results

    async def lines() -> AsyncGenerator[bytes]:
        stream_dict = results[-1]
        it, resp = stream_dict.pop("async_iterator"), stream_dict.pop("response", None)
        yield (json.dumps(results) + "\n").encode()
        try:
            async for chunk in it:
                chunk = chunk.strip()
                if chunk:
                    yield (chunk if isinstance(chunk, bytes) else chunk.encode()) + b"\n"
        finally:
            if resp is not None:
                resp.close()

    return StreamingResponse(lines(), media_type="text/plain")


@router.get("/health")
async def health():
    return Response(status_code=200)


@router.post("/deploy-tasks")
async def deploy_tasks(request: TasksDeploymentRequest, raw: Request):
    """Upload task classes and descriptors; every control-plane process loads them through its watcher."""
    registry: TaskRegistry = raw.app.state.task_registry
    try:
        if not await registry.check_no_active_task_instance():
            return Response(status_code=409, content="Unit tasks are deployed; unregister all apps before redeploying.")
        for d in request.task_definitions:
            import base64

            await registry.create_task_definition(d.task_definition_name, d.task_class_name, d.module_name,
                                                  base64.b64decode(d.source_b64).decode(), d.is_unit_task)
        for d in request.descriptor_definitions:
            import base64

            await registry.create_execution_descriptor(d.descriptor_definition_name, d.task_class_name,
                                                       d.descriptor_class_name, d.module_name,
                                                       base64.b64decode(d.source_b64).decode(), d.is_default)
        await sync_control_plane(raw.app)
        return {"status": "ok", "unit_tasks": TASK_CLASS_REGISTRY.list_registered_unit_tasks(),
                "descriptors": DESCRIPTOR_REGISTRY.list_registered_descriptors()}
    except ValueError as e:
        return Response(status_code=409, content=str(e))
    except Exception as e:
        logger.exception("Unexpected error while deploying tasks")
        return Response(status_code=500, content=str(e))


@router.post("/deploy-profiles")
async def deploy_profiles(request: ProfilesDeploymentRequest, raw: Request):
    profiles: UnitTaskProfileManager = raw.app.state.profile_manager
    try:
        names = []
        for p in request.profiles:
            names.append(await profiles.deploy_profile(UnitTaskProfile.from_dict(p.model_dump())))
        return {"status": "ok", "profiles": names}
    except ValueError as e:
        return Response(status_code=400, content=str(e))


@router.post("/purge-tasklib")
async def purge_tasklib(raw: Request):
    registry: TaskRegistry = raw.app.state.task_registry
    if not await registry.check_no_active_task_instance():
        return Response(status_code=409, content="Unit tasks are deployed; unregister all apps first.")
    await registry.delete_all_task_definitions_and_descriptors()
    await sync_control_plane(raw.app)
    return {"status": "ok"}


def create_app(resource_manager_grpc_url: str = RESOURCE_MANAGER_GRPC_URL,
               task_dispatcher_http_url: str = TASK_DISPATCHER_HTTP_URL,
               task_dispatcher_grpc_urls: list[str] | None = None, registry: TaskRegistry | None = None,
               resource_manager_local: Any = None) -> FastAPI:
    registry = registry or TaskRegistry()

    @contextlib.asynccontextmanager
    async def lifespan(app: FastAPI):
        task_manager_context.set(app.state.task_manager)
        registry.start_watching()
        yield
        await app.state.app_manager.shutdown()
        await app.state.task_manager.shutdown()
        await registry.shutdown()

    app = FastAPI(title="cornserve-b200 gateway", lifespan=lifespan)

    from ...tracing import instrument_fastapi


    instrument_fastapi(app, "cornserve.gateway")
    app.include_router(router)
    app.state.task_registry = registry
    app.state.profile_manager = UnitTaskProfileManager(registry.store)
    app.state.task_manager = TaskManager(resource_manager_grpc_url, task_dispatcher_http_url, registry)
    app.state.app_manager = AppManager(app.state.task_manager)
    app.state.session_manager = SessionManager(app.state.task_manager)
    app.state.resource_manager_grpc_url = resource_manager_grpc_url
    app.state.task_dispatcher_grpc_urls = task_dispatcher_grpc_urls or [TASK_DISPATCHER_GRPC_URL]
    app.state.resource_manager_local = resource_manager_local
    # app code running inside the gateway dispatches through the in-process manager (no extra HTTP hop)
    task_manager_context.set(app.state.task_manager)

    return app
