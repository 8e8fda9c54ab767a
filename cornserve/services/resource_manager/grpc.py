"""gRPC face of the Resource Manager (reference: python/cornserve/services/resource_manager/grpc.py:18-135)."""

from __future__ import annotations

import grpc

from ...logging import get_logger
from ..pb import common_pb2, resource_manager_pb2, resource_manager_pb2_grpc
from .manager import ResourceManager
from ...tracing import grpc_server_interceptors

logger = get_logger(__name__)
OK, ERROR = common_pb2.STATUS_OK, common_pb2.STATUS_ERROR


class ResourceManagerServicer(resource_manager_pb2_grpc.ResourceManagerServicer):
    def __init__(self, manager: ResourceManager):
        self.manager = manager

    async def DeployUnitTask(self, request, context):
        try:
            await self.manager.registry.sync_watchers()
            task = await self.manager.registry.get_task_instance(request.task_instance_name)
            await self.manager.deploy_unit_task(request.task_instance_name, task)
        except Exception as e:
            logger.exception("DeployUnitTask failed")
            await context.abort(grpc.StatusCode.INTERNAL, f"DeployUnitTask failed: {e}")
        return resource_manager_pb2.DeployUnitTaskResponse(status=OK)

    async def TeardownUnitTask(self, request, context):
        try:
            await self.manager.teardown_unit_task(request.task_instance_name)
        except ValueError as e:
            await context.abort(grpc.StatusCode.NOT_FOUND, str(e))
        except Exception as e:
            logger.exception("TeardownUnitTask failed")
            await context.abort(grpc.StatusCode.INTERNAL, f"TeardownUnitTask failed: {e}")
        return resource_manager_pb2.TeardownUnitTaskResponse(status=OK)

    async def ScaleUnitTask(self, request, context):
        try:
            await self.manager.scale_unit_task(request.task_instance_name, request.num_gpus)
        except ValueError as e:
            await context.abort(grpc.StatusCode.INVALID_ARGUMENT, str(e))
        except Exception as e:
            logger.exception("ScaleUnitTask failed")
            await context.abort(grpc.StatusCode.INTERNAL, f"ScaleUnitTask failed: {e}")
        return resource_manager_pb2.ScaleUnitTaskResponse(status=OK)

    async def Healthcheck(self, request, context):
        ok, statuses = await self.manager.healthcheck()
        resp = resource_manager_pb2.HealthcheckResponse(status=OK if ok else ERROR)
        for name, good in statuses.items():
            resp.task_manager_statuses.add(task_instance_name=name, status=OK if good else ERROR)
        return resp

    async def SyncTaskRegistry(self, request, context):
        try:
            await self.manager.registry.sync_watchers()
            return common_pb2.SyncTaskRegistryResponse(status=OK)
        except Exception:
            logger.exception("SyncTaskRegistry failed")
            return common_pb2.SyncTaskRegistryResponse(status=ERROR)


async def start_server(manager: ResourceManager, address: str) -> grpc.aio.Server:
    server = grpc.aio.server(interceptors=grpc_server_interceptors())
    resource_manager_pb2_grpc.add_ResourceManagerServicer_to_server(ResourceManagerServicer(manager), server)
    server.add_insecure_port(address)
    await server.start()
    return server
