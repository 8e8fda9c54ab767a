"""``python -m cornserve.services.gateway.entrypoint``"""

from __future__ import annotations

import os

import uvicorn

import cornserve_tasklib  # noqa: F401

from ...constants import GATEWAY_HOST, GATEWAY_HTTP_PORT, TASK_DISPATCHER_GRPC_URL
from ...tracing import configure_otel
from .router import create_app


def main() -> None:
    configure_otel("gateway")
    dispatchers = os.environ.get("CORNSERVE_TASK_DISPATCHER_GRPC_URLS", TASK_DISPATCHER_GRPC_URL).split(",")
    app = create_app(task_dispatcher_grpc_urls=[d for d in dispatchers if d])
    uvicorn.run(app, host=GATEWAY_HOST, port=GATEWAY_HTTP_PORT, log_level="warning")


if __name__ == "__main__":
    main()
