"""``python -m cornserve.services.task_manager.entrypoint --port P``: a Task Manager as its own process
(the resource manager can also host task managers in-process)."""

from __future__ import annotations

import argparse
import asyncio

import cornserve_tasklib  # noqa: F401  (registers the built-in task classes)

from ...logging import get_logger
from ...tracing import configure_otel
from .grpc import TaskManagerServicer, start_server

logger = get_logger(__name__)


async def serve(port: int) -> None:
    configure_otel("task_manager")
    servicer = TaskManagerServicer()
    servicer.registry.start_watching()
    server = await start_server(port, servicer)
    logger.info("Task manager listening on %d", port)
    while not servicer.shutdown_requested:
        await asyncio.sleep(0.2)
    await server.stop(2.0)
    await servicer.registry.shutdown()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--port", type=int, required=True)
    asyncio.run(serve(ap.parse_args().port))


if __name__ == "__main__":
    main()
