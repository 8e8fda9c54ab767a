"""``python -m cornserve.services.task_dispatcher.entrypoint``: HTTP (task graphs) + gRPC (notifications)."""

from __future__ import annotations

import asyncio
import signal
from urllib.parse import urlparse

import uvicorn

import cornserve_tasklib  # noqa: F401

from ...constants import TASK_DISPATCHER_GRPC_URL, TASK_DISPATCHER_HTTP_URL
from ...logging import get_logger
from ...tracing import configure_otel
from .app import create_app, start_grpc
from .dispatcher import TaskDispatcher

logger = get_logger(__name__)


async def serve() -> None:
    configure_otel("task_dispatcher")
    dispatcher = TaskDispatcher()
    dispatcher.registry.start_watching()
    grpc_server = await start_grpc(dispatcher, TASK_DISPATCHER_GRPC_URL)
    u = urlparse(TASK_DISPATCHER_HTTP_URL)
    server = uvicorn.Server(uvicorn.Config(create_app(dispatcher), host=u.hostname or "127.0.0.1", port=u.port or 8001,
                                           log_level="warning"))
    loop = asyncio.get_running_loop()
    for s in (signal.SIGTERM, signal.SIGINT):
        loop.add_signal_handler(s, lambda: setattr(server, "should_exit", True))
    logger.info("Task dispatcher: HTTP %s, gRPC %s", TASK_DISPATCHER_HTTP_URL, TASK_DISPATCHER_GRPC_URL)
    await server.serve()
    await grpc_server.stop(2.0)
    await dispatcher.shutdown()
    await dispatcher.registry.shutdown()


def main() -> None:
    asyncio.run(serve())


if __name__ == "__main__":
    main()
