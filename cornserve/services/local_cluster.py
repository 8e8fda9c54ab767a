"""One-machine control plane: resource manager (which starts one sidecar per GPU), task dispatcher and gateway in
one process, serving on localhost.  This is what ``cornserve up`` runs; it replaces applying the reference's
Kubernetes manifests (kubernetes/kustomize/cornserve/base: gateway, resource-manager, task-dispatcher deployments)."""

from __future__ import annotations

import asyncio
import contextlib
import signal

import uvicorn

from ..constants import GATEWAY_HTTP_PORT
from ..logging import get_logger
from .process import free_port

logger = get_logger(__name__)


class LocalCluster:
    def __init__(self, num_gpus: int | None = None, cpu: bool = False, gateway_port: int | None = None,
                 store_path: str | None = None, tm_manager_kwargs: dict | None = None, sidecar_slab_bytes: int | None = None):
        self.num_gpus, self.cpu = num_gpus, cpu
        self.gateway_port = gateway_port or GATEWAY_HTTP_PORT
        self.store_path = store_path
        self.tm_kwargs = tm_manager_kwargs or {}
        self.slab = sidecar_slab_bytes
        self._closers: list = []
        self.rm = None
        self.url = f"http://127.0.0.1:{self.gateway_port}"

    async def _serve(self, app, port: int):
        server = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="warning"))
        task = asyncio.create_task(server.serve())
        while not server.started:
            await asyncio.sleep(0.02)
            if task.done():
                task.result()
        return server, task

    async def start(self) -> "LocalCluster":
        import torch

        import cornserve_tasklib  # noqa: F401  (registers the built-in tasks and descriptors)
        from .gateway.router import create_app
        from .resource_manager.grpc import start_server as start_rm
        from .resource_manager.manager import ResourceManager
        from .store import LocalStore
        from .task_dispatcher.app import create_app as create_td_app
        from .task_dispatcher.app import start_grpc as start_td_grpc
        from .task_dispatcher.dispatcher import TaskDispatcher
        from .task_registry.registry import TaskRegistry

        cpu = self.cpu or not torch.cuda.is_available()
        n = self.num_gpus or (torch.cuda.device_count() if not cpu else 2)
        # one store for the whole deployment: the path given, else $CORNSERVE_STORE_PATH (what default_store() opens
        # in every other process of the deployment), else the per-user state directory
        import os

        store = LocalStore(self.store_path or os.environ.get("CORNSERVE_STORE_PATH"))
        registry = TaskRegistry(store)
        dispatcher = TaskDispatcher(registry)
        td_grpc_addr = f"127.0.0.1:{free_port()}"
        td_grpc = await start_td_grpc(dispatcher, td_grpc_addr)
        td_port = free_port()
        td_server, td_task = await self._serve(create_td_app(dispatcher), td_port)
        kw = {"sidecar_slab_bytes": self.slab} if self.slab else {}
        # adopt=True: sidecars and executors that a previous control plane over the same store left running are taken
        # over instead of being started again
        rm = await ResourceManager.init(num_gpus=n, sidecar_device="cpu" if cpu else None, registry=registry, adopt=True,
                                        dispatcher_urls=[td_grpc_addr], tm_manager_kwargs=self.tm_kwargs, **kw)
        rm_addr = f"127.0.0.1:{free_port()}"
        rm_server = await start_rm(rm, rm_addr)
        gw_app = create_app(rm_addr, f"http://127.0.0.1:{td_port}", [td_grpc_addr], registry)
        self.rm = rm

        @gw_app.get("/cluster/executors")
        async def cluster_executors():
            """What runs where: one entry per task executor with its URL, GPUs and health (a view for operators and
            benchmarks; the reference offers ``kubectl get pods`` for this)."""
            return self.executors()

        gw_server, gw_task = await self._serve(gw_app, self.gateway_port)
        logger.info("Control plane is up: gateway %s, %d %s", self.url, n, "CPU ranks" if cpu else "GPUs")

        async def close():
            gw_server.should_exit = True
            td_server.should_exit = True
            await asyncio.gather(gw_task, td_task, return_exceptions=True)
            await rm_server.stop(0.5)
            await td_grpc.stop(0.5)
            await rm.shutdown()
            await dispatcher.shutdown()
            await registry.shutdown()
            store.close()

        self._closers.append(close)
        return self

    def executors(self) -> list[dict]:
        out, seen = [], set()
        for name, st in self.rm.task_managers.items():
            tm = getattr(getattr(st, "servicer", None), "manager", None)
            if tm is None or id(tm) in seen:
                continue
            seen.add(id(tm))
            for d in tm.executors.values():
                out.append({"task": name, "task_class": type(st.task).__name__, "executor_id": d.executor_id, "url": d.url,
                            "gpus": d.sidecar_ranks, "healthy": d.healthy,
                            "pid": getattr(getattr(d.process, "popen", None), "pid", None)})
        return out

    async def stop(self) -> None:
        for c in reversed(self._closers):
            with contextlib.suppress(Exception):
                await c()
        self._closers.clear()


def run_forever(num_gpus: int | None = None, cpu: bool = False, gateway_port: int | None = None) -> None:
    async def main():
        cluster = await LocalCluster(num_gpus, cpu, gateway_port).start()
        print(f"cornserve control plane ready at {cluster.url}  (CORNSERVE_GATEWAY_URL={cluster.url})", flush=True)
        stop = asyncio.Event()
        loop = asyncio.get_running_loop()
        for s in (signal.SIGINT, signal.SIGTERM):
            loop.add_signal_handler(s, stop.set)
        await stop.wait()
        await cluster.stop()

    asyncio.run(main())
