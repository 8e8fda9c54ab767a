"""``python -m cornserve.task_executors.eric.entrypoint --model.id ... --server.port ...``"""

from __future__ import annotations

import os
import subprocess
import sys

import tyro
import uvicorn

from ...logging import get_logger
from ...parallel.state import init_distributed
from ...services.process import free_port
from ...tracing import configure_otel
from ...utils.threads import maybe_start_sampler, tune_interpreter
from .config import EricConfig
from .engine import Engine
from .router import create_app
from .worker import pick_device

logger = get_logger(__name__)


def main(argv: list[str] | None = None) -> None:
    config = tyro.cli(EricConfig, args=argv)
    tune_interpreter()
    configure_otel("eric")
    maybe_start_sampler()
    tp = config.model.tp_size
    group = None
    children: list[subprocess.Popen] = []
    if tp > 1:
        port = free_port()
        for r in range(1, tp):
            code = ("from cornserve.task_executors.eric.worker import tp_worker_main; import sys; "
                    "tp_worker_main(sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4]))")
            children.append(subprocess.Popen([sys.executable, "-c", code, config.model_dump_json(), str(r), str(tp), str(port)],
                                             env=dict(os.environ)))
        dev = pick_device(0)
        group = init_distributed(0, tp, master_port=port, local_device=dev.index if dev.type == "cuda" else None,
                                 backend=None if dev.type == "cuda" else "gloo")
    engine = Engine(config, group)
    try:
        uvicorn.run(create_app(config, engine), host=config.server.host, port=config.server.port, log_level="warning")
    finally:
        engine.shutdown()
        for c in children:
            try:
                c.wait(timeout=10)
            except subprocess.TimeoutExpired:
                c.kill()


if __name__ == "__main__":
    main()
