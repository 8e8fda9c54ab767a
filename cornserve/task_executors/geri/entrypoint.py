"""``python -m cornserve.task_executors.geri.entrypoint --model.id ... --model.modality IMAGE --server.port ...``"""

from __future__ import annotations

import os
import subprocess
import sys

import tyro
import uvicorn

from ...logging import get_logger
from ...parallel.state import init_distributed
from ...services.process import free_port
from ...sidecar.api import Sidecar
from ...sidecar.schema import SidecarConfig
from ...tracing import configure_otel
from ... import ops
from ..eric.worker import pick_device
from .config import GeriConfig
from .engine import Engine
from .loader import find_embedding_dim, resolve_entry
from .router import create_app

logger = get_logger(__name__)


def main(argv: list[str] | None = None) -> None:
    config = tyro.cli(GeriConfig, args=argv)
    configure_otel("geri")
    sp = config.model.sp_size
    group = None
    children: list[subprocess.Popen] = []
    device = pick_device(0)
    ops.bind_thread(device)  # also for the sidecar client: forwarded tensors are mapped onto the current GPU
    if sp > 1:
        port = free_port()
        for r in range(1, sp):
            code = ("from cornserve.task_executors.geri.engine import sp_worker_main; import sys; "
                    "sp_worker_main(sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4]))")
            children.append(subprocess.Popen([sys.executable, "-c", code, config.model_dump_json(), str(r), str(sp), str(port)],
                                             env=dict(os.environ)))
        group = init_distributed(0, sp, master_port=port, local_device=device.index if device.type == "cuda" else None,
                                 backend=None if device.type == "cuda" else "gloo")
    engine = Engine(config, device, group)
    sidecar = None
    if config.sidecar.ranks:
        entry, _ = resolve_entry(config.model.id)
        sidecar = Sidecar(SidecarConfig(sidecar_rank=config.sidecar.ranks[0], group=list(config.sidecar.ranks), whole_group=True,
                                        recv_tensor_dtype=entry.embedding_dtype,
                                        recv_tensor_shape=(-1, find_embedding_dim(config.model.id))))
    try:
        uvicorn.run(create_app(config, engine, sidecar), host=config.server.host, port=config.server.port, log_level="warning")
    finally:
        engine.shutdown()
        if sidecar is not None:
            sidecar.shutdown_sync()
        for c in children:
            try:
                c.wait(timeout=10)
            except subprocess.TimeoutExpired:
                c.kill()


if __name__ == "__main__":
    main()
