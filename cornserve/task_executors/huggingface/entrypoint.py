"""``python -m cornserve.task_executors.huggingface.entrypoint --model.id ... --model.model-type QWEN_IMAGE --server.port ...``"""

from __future__ import annotations

import tyro
import uvicorn

from ...tracing import configure_otel
from ... import ops
from ..eric.worker import pick_device
from .config import HuggingFaceConfig
from .engine import Engine
from .router import create_app


def main(argv: list[str] | None = None) -> None:
    config = tyro.cli(HuggingFaceConfig, args=argv)
    configure_otel("huggingface")
    device = pick_device(0)
    ops.bind_thread(device)
    engine = Engine(config, device)
    uvicorn.run(create_app(config, engine), host=config.server.host, port=config.server.port, log_level="warning")


if __name__ == "__main__":
    main()
