"""gRPC face of a Task Manager (reference: python/cornserve/services/task_manager/grpc.py:29-135; the three
RPCs that are declared but unimplemented there are implemented here)."""

from __future__ import annotations

import grpc

from ...logging import get_logger
from ..pb import common_pb2, task_manager_pb2, task_manager_pb2_grpc
from ..resource import GPU
from ..task_registry.registry import TaskRegistry
from .manager import TaskManager
from ...tracing import grpc_server_interceptors

logger = get_logger(__name__)
OK, ERROR = common_pb2.STATUS_OK, common_pb2.STATUS_ERROR


class TaskManagerServicer(task_manager_pb2_grpc.TaskManagerServicer):
    def __init__(self, registry: TaskRegistry | None = None, manager_kwargs: dict | None = None):
        self.registry = registry or TaskRegistry()
        self.manager: TaskManager | None = None
        self.manager_kwargs = manager_kwargs or {}
        self.shutdown_requested = False

    @staticmethod
    def _gpus(msgs, action) -> list[GPU]:
        return [GPU(m.node_id, m.global_rank, m.local_rank) for m in msgs if m.action == action]

    async def RegisterTask(self, request, context):
        if self.manager is not None:
            await context.abort(grpc.StatusCode.ALREADY_EXISTS, "Task manager already registered")
        try:
            task = await self.registry.get_task_instance(request.task_instance_name)
            self.manager = await TaskManager.init(request.task_manager_id, task,
                                                  self._gpus(request.gpus, task_manager_pb2.ResourceAction.ADD),
                                                  **self.manager_kwargs)
        except Exception as e:
            logger.exception("RegisterTask failed")
            await context.abort(grpc.StatusCode.INTERNAL, f"RegisterTask failed: {e}")
        return task_manager_pb2.RegisterTaskResponse(status=OK)

    async def UpdateResources(self, request, context):
        if self.manager is None or self.manager.id != request.task_manager_id:
            await context.abort(grpc.StatusCode.FAILED_PRECONDITION, "Task manager not registered with this ID")
        try:
            await self.manager.update_resources(self._gpus(request.gpus, task_manager_pb2.ResourceAction.ADD),
                                                self._gpus(request.gpus, task_manager_pb2.ResourceAction.REMOVE))
        except Exception as e:
            logger.exception("UpdateResources failed")
            await context.abort(grpc.StatusCode.INTERNAL, f"UpdateResources failed: {e}")
        return task_manager_pb2.UpdateResourcesResponse(status=OK)

    async def Shutdown(self, request, context):
        if self.manager is not None:
            await self.manager.shutdown()
            self.manager = None
        self.shutdown_requested = True
        return task_manager_pb2.ShutdownResponse(status=OK)

    async def GetRoute(self, request, context):
        if self.manager is None:
            await context.abort(grpc.StatusCode.FAILED_PRECONDITION, "Task manager not registered")
        try:
            hint = request.routing_hint if request.HasField("routing_hint") else None
            url, ranks = await self.manager.get_route(request.request_id, hint)
        except Exception as e:
            await context.abort(grpc.StatusCode.UNAVAILABLE, str(e))
        return task_manager_pb2.GetRouteResponse(task_executor_url=url, sidecar_ranks=ranks)

    async def Healthcheck(self, request, context):
        resp = task_manager_pb2.HealthcheckResponse(status=OK)
        if self.manager is None:
            resp.status = ERROR
            return resp
        for eid, (ok, ranks) in (await self.manager.healthcheck()).items():
            st = resp.task_executor_statuses[eid]
            st.status = OK if ok else ERROR
            st.sidecar_ranks.extend(ranks)
            if not ok:
                resp.status = ERROR
        return resp

    async def GetTaskProfile(self, request, context):
        resp = task_manager_pb2.GetTaskProfileResponse()
        if self.manager is not None:
            for n, load, tp in await self.manager.get_task_profile():
                resp.profile_points.add(num_gpus=n, max_sustainable_load=load,
                                        deployment_config=task_manager_pb2.DeploymentConfig(
                                            num_replicas=1, tensor_parallel_degree=tp, pipeline_parallel_degree=1))
        return resp

    async def ReconcileTargetLoad(self, request, context):
        if self.manager is None:
            return task_manager_pb2.ReconcileTargetLoadResponse(status=ERROR, message="not registered")
        delta, msg = await self.manager.reconcile_target_load(request.target_load)
        return task_manager_pb2.ReconcileTargetLoadResponse(status=OK, message=f"delta_gpus={delta}; {msg}")

    async def SyncTaskRegistry(self, request, context):
        try:
            await self.registry.sync_watchers()
            return common_pb2.SyncTaskRegistryResponse(status=OK)
        except Exception:
            logger.exception("SyncTaskRegistry failed")
            return common_pb2.SyncTaskRegistryResponse(status=ERROR)


async def start_server(port: int, servicer: TaskManagerServicer) -> grpc.aio.Server:
    server = grpc.aio.server(interceptors=grpc_server_interceptors())
    task_manager_pb2_grpc.add_TaskManagerServicer_to_server(servicer, server)
    server.add_insecure_port(f"127.0.0.1:{port}")
    await server.start()
    return server
