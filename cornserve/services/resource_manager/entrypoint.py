"""``python -m cornserve.services.resource_manager.entrypoint``"""

from __future__ import annotations

import asyncio
import os
import signal

import cornserve_tasklib  # noqa: F401

from ...constants import RESOURCE_MANAGER_GRPC_URL, TASK_DISPATCHER_GRPC_URL
from ...logging import get_logger
from ...tracing import configure_otel
from .grpc import start_server
from .manager import ResourceManager

logger = get_logger(__name__)


async def serve() -> None:
    configure_otel("resource_manager")
    dispatchers = os.environ.get("CORNSERVE_TASK_DISPATCHER_GRPC_URLS", TASK_DISPATCHER_GRPC_URL).split(",")
    manager = await ResourceManager.init(dispatcher_urls=[d for d in dispatchers if d],
                                         sidecar_device=os.environ.get("SIDECAR_DEVICE"))
    manager.registry.start_watching()
    server = await start_server(manager, RESOURCE_MANAGER_GRPC_URL)
    logger.info("Resource manager listening on %s", RESOURCE_MANAGER_GRPC_URL)
    stop = asyncio.Event()
    for s in (signal.SIGTERM, signal.SIGINT):
        asyncio.get_running_loop().add_signal_handler(s, stop.set)
    await stop.wait()
    await server.stop(2.0)
    await manager.shutdown()
    await manager.registry.shutdown()


def main() -> None:
    asyncio.run(serve())


if __name__ == "__main__":
    main()
