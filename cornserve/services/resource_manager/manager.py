"""Resource Manager: owns the GPUs of the box, the sidecar processes and one Task Manager per deployed
unit task (reference: python/cornserve/services/resource_manager/manager.py:171-845, with local
processes in place of pods).

``deploy_unit_task`` is idempotent by task equivalence and transactional: GPUs are allocated, a Task
Manager is started and registered, the Task Dispatchers are told, and any failure on the way rolls all
of it back.  ``scale_unit_task`` grows or shrinks a task's GPU set in chunks that its profile allows.
``healthcheck`` fans out to the Task Managers; ``reconcile`` lets a Task Manager's load target drive
scaling (declared but not implemented in the reference).
"""

from __future__ import annotations

import asyncio
import os
import sys
import uuid
from dataclasses import dataclass, field

import grpc

from ...constants import (KIND_EXECUTOR_RECORD, KIND_SIDECAR_RECORD, KIND_TASK_MANAGER_RECORD, SIDECAR_HEALTHY_TIMEOUT_S,
                          TASK_DISPATCHER_GRPC_URL)
from ...task_executors.profile import UnitTaskProfileManager
from ...logging import get_logger
from ...task.base import UnitTask
from ..pb import (common_pb2, task_dispatcher_pb2, task_dispatcher_pb2_grpc, task_manager_pb2,
                  task_manager_pb2_grpc)
from ..process import ManagedProcess, free_port, spawn, terminate
from ..resource import GPU, Resource
from ..sidecar import launch as sidecar_launch
from ..task_manager.grpc import TaskManagerServicer, start_server
from ..task_registry.registry import TaskRegistry
from ...tracing import grpc_client_interceptors

logger = get_logger(__name__)


@dataclass
class TaskManagerState:
    id: str
    task_instance_name: str
    task: UnitTask
    url: str
    gpus: list[GPU]
    server: grpc.aio.Server | None = None        # in-process hosting
    servicer: TaskManagerServicer | None = None
    process: ManagedProcess | None = None        # subprocess hosting
    channel: grpc.aio.Channel | None = None
    stub: task_manager_pb2_grpc.TaskManagerStub | None = None
    lock: asyncio.Lock = field(default_factory=asyncio.Lock)


def detect_num_gpus() -> int:
    if "CORNSERVE_NUM_GPUS" in os.environ:
        return int(os.environ["CORNSERVE_NUM_GPUS"])
    try:
        import torch

        return torch.cuda.device_count()
    except Exception:
        return 0


class ResourceManager:
    def __init__(self, resource: Resource, registry: TaskRegistry | None = None,
                 dispatcher_urls: list[str] | None = None, tm_in_process: bool = True,
                 tm_manager_kwargs: dict | None = None, sidecar_processes: list | None = None):
        self.resource = resource
        self.registry = registry or TaskRegistry()
        self.profiles = UnitTaskProfileManager(self.registry.store)
        self.dispatcher_urls = dispatcher_urls if dispatcher_urls is not None else [TASK_DISPATCHER_GRPC_URL]
        self.tm_in_process = tm_in_process
        self.tm_manager_kwargs = tm_manager_kwargs or {}
        self.sidecars = sidecar_processes or []
        self.task_managers: dict[str, TaskManagerState] = {}   # keyed by task instance name
        self.lock = asyncio.Lock()
        self._dispatcher_channels: dict[str, grpc.aio.Channel] = {}

    # -- start-up ----------------------------------------------------------------------------------------------
    @classmethod
    async def init(cls, num_gpus: int | None = None, spawn_sidecars: bool = True, sidecar_slab_bytes: int | None = None,
                   sidecar_device: str | None = None, adopt: bool = False, **kw) -> "ResourceManager":
        """Enumerate the GPUs of this box, start one sidecar per GPU (ranks 0..n-1) and wait until every
        sidecar reports ``ALL_GOOD``."""
        n = num_gpus if num_gpus is not None else detect_num_gpus()
        if n <= 0:
            raise RuntimeError("No GPUs found (set CORNSERVE_NUM_GPUS to run a CPU-only deployment)")
        resource = Resource.single_node(n)
        procs = []
        store = (kw.get("registry") or TaskRegistry()).store if adopt else None
        if kw.get("registry") is None and adopt:
            kw["registry"] = TaskRegistry(store)
        adopted_pids: list[int] = []
        if spawn_sidecars:
            slab = sidecar_slab_bytes or int(os.environ.get("SIDECAR_SHM_SIZE", str(1 << 30)))
            for r in range(n):
                # a sidecar left running by a previous control plane (same rank, same ports) is taken over as it is:
                # executors that are adopted below have its slab mapped
                if adopt and await asyncio.to_thread(sidecar_launch.check_health, r, 1.0) == 0:   # HEALTH_ALL_GOOD
                    try:
                        adopted_pids.append(int(store.get(KIND_SIDECAR_RECORD, f"sidecar-{r}").spec["pid"]))
                        logger.info("Adopted sidecar %d (pid %d)", r, adopted_pids[-1])
                        continue
                    except Exception:  # noqa: BLE001  (answers but is not ours to manage: start none, it holds the port)
                        logger.warning("Sidecar %d answers but has no record; using it without managing it", r)
                        continue
                from ...constants import LOG_DIR

                os.makedirs(LOG_DIR, exist_ok=True)
                p = sidecar_launch.spawn_sidecar(r, n, slab, device=sidecar_device, log_path=os.path.join(LOG_DIR, f"sidecar-{r}.log"))
                procs.append(p)
                if store is not None:
                    store.update(KIND_SIDECAR_RECORD, f"sidecar-{r}", {"pid": p.pid, "rank": r}, True)
            ok = await asyncio.to_thread(sidecar_launch.wait_all_good, list(range(n)), SIDECAR_HEALTHY_TIMEOUT_S, procs)
            if not ok:
                for p in procs:
                    p.terminate()
                tails = []
                for r in range(n):
                    try:
                        tails.append(f"sidecar-{r}: " + " | ".join(open(os.path.join(LOG_DIR, f"sidecar-{r}.log"), errors="replace").read().splitlines()[-5:]))
                    except OSError:
                        pass
                raise RuntimeError("Sidecars did not become healthy\n" + "\n".join(tails))
            logger.info("All %d sidecars are healthy", n)
        rm = cls(resource, sidecar_processes=procs, **kw)
        rm.adopted_sidecar_pids = adopted_pids
        rm.persist = adopt
        if adopt:
            await rm.adopt_running()
        logger.info("Cluster:\n%s", resource.render())
        return rm

    # -- taking over what a previous control plane left running ---------------------------------------------------------
    async def adopt_running(self) -> list[str]:
        """Rebuild the task managers of unit tasks whose executors are still running (the control plane was restarted,
        its executors and sidecars were not): the recorded GPUs are marked as owned again, every executor that answers
        ``/health`` is taken over, the task dispatchers are told.  Returns the adopted task instance names.  The
        reference leaves this as a TODO (python/cornserve/services/resource_manager/grpc.py:44-46)."""
        store = self.registry.store
        records = await asyncio.to_thread(store.list, KIND_TASK_MANAGER_RECORD)
        executors = await asyncio.to_thread(store.list, KIND_EXECUTOR_RECORD)
        adopted = []
        for rec in records:
            name, spec = rec.name, rec.spec
            try:
                task = await self.registry.get_task_instance(name)
                gpus = [g for g in self.resource.gpus if g.global_rank in set(spec["gpus"])]
                if len(gpus) != len(spec["gpus"]) or any(not g.is_free for g in gpus):
                    raise RuntimeError("its GPUs are not available")
                mine = {e.name: e.spec for e in executors if e.spec.get("task_manager_id") == spec["tm_id"]}
                for g in gpus:
                    g.allocate_to(spec["tm_id"])
                port = free_port()
                st = TaskManagerState(spec["tm_id"], name, task, f"127.0.0.1:{port}", gpus)
                st.servicer = TaskManagerServicer(self.registry, {"profile_manager": self.profiles, **self.tm_manager_kwargs})
                from ..task_manager.manager import TaskManager

                st.servicer.manager = await TaskManager.adopt(spec["tm_id"], task, gpus, mine,
                                                              **{"profile_manager": self.profiles, **self.tm_manager_kwargs})
                st.server = await start_server(port, st.servicer)
                st.channel = grpc.aio.insecure_channel(st.url, interceptors=grpc_client_interceptors())
                st.stub = task_manager_pb2_grpc.TaskManagerStub(st.channel)
                await asyncio.wait_for(st.channel.channel_ready(), timeout=60)
                self.task_managers[name] = st
                await self._notify_dispatchers(deployed=True, name=name, url=st.url)
                adopted.append(name)
                logger.info("Adopted unit task %s with %d executors", name, len(st.servicer.manager.executors))
            except Exception as e:  # noqa: BLE001
                logger.warning("Could not adopt unit task %s: %s; dropping its record", name, e)
                for g in self.resource.gpus:
                    if g.owner == spec.get("tm_id"):
                        g.free()
                await asyncio.to_thread(self._drop_record, name)
        return adopted

    def _drop_record(self, name: str) -> None:
        try:
            self.registry.store.delete(KIND_TASK_MANAGER_RECORD, name)
        except Exception:  # noqa: BLE001
            pass

    def _save_record(self, st: "TaskManagerState") -> None:
        if getattr(self, "persist", False):
            self.registry.store.update(KIND_TASK_MANAGER_RECORD, st.task_instance_name,
                                       {"tm_id": st.id, "gpus": [g.global_rank for g in st.gpus]}, True)

    # -- deploy / teardown ----------------------------------------------------------------------------------------
    async def deploy_unit_task(self, task_instance_name: str, task: UnitTask) -> None:
        async with self.lock:
            if task_instance_name in self.task_managers:
                logger.info("Unit task %s is already deployed", task_instance_name)
                return
            for st in self.task_managers.values():
                if st.task.is_equivalent_to(task):
                    logger.info("An equivalent unit task (%s) is already deployed", st.task_instance_name)
                    self.task_managers[task_instance_name] = st
                    return
            st = await self._spawn_task_manager(task_instance_name, task)
            self.task_managers[task_instance_name] = st
        try:
            await self._notify_dispatchers(deployed=True, name=task_instance_name, url=st.url)
        except Exception:
            logger.exception("Dispatcher notification failed; rolling back %s", task_instance_name)
            async with self.lock:
                self.task_managers.pop(task_instance_name, None)
                await self._stop_task_manager(st)
            raise

    async def _spawn_task_manager(self, task_instance_name: str, task: UnitTask) -> TaskManagerState:
        profile = await self.profiles.get_profile(task)
        tm_id = f"tm-{task.make_name()}-{uuid.uuid4().hex[:8]}"
        gpus = self.resource.allocate(profile.min_gpus(), owner=tm_id)
        logger.info("Allocated GPUs %s to %s\n%s", [g.global_rank for g in gpus], tm_id, self.resource.render())
        port = free_port()
        st = TaskManagerState(tm_id, task_instance_name, task, f"127.0.0.1:{port}", gpus)
        try:
            if self.tm_in_process:
                # in-process task managers read profiles from the same store as this resource manager
                st.servicer = TaskManagerServicer(self.registry, {"profile_manager": self.profiles, **self.tm_manager_kwargs})
                st.server = await start_server(port, st.servicer)
            else:
                st.process = spawn(tm_id, [sys.executable, "-m", "cornserve.services.task_manager.entrypoint",
                                           "--port", str(port)], port=port)
            st.channel = grpc.aio.insecure_channel(st.url, interceptors=grpc_client_interceptors())
            st.stub = task_manager_pb2_grpc.TaskManagerStub(st.channel)
            await asyncio.wait_for(st.channel.channel_ready(), timeout=60)
            await st.stub.SyncTaskRegistry(common_pb2.SyncTaskRegistryRequest())
            req = task_manager_pb2.RegisterTaskRequest(task_manager_id=tm_id, task_instance_name=task_instance_name)
            for g in gpus:
                req.gpus.add(action=task_manager_pb2.ResourceAction.ADD, node_id=g.node, global_rank=g.global_rank,
                             local_rank=g.local_rank)
            resp = await st.stub.RegisterTask(req)
            if resp.status != common_pb2.STATUS_OK:
                raise RuntimeError("RegisterTask returned an error status")
            await asyncio.to_thread(self._save_record, st)
            return st
        except Exception:
            logger.exception("Failed to start task manager %s; releasing its GPUs", tm_id)
            await self._stop_task_manager(st)
            raise

    async def _stop_task_manager(self, st: TaskManagerState) -> None:
        await asyncio.to_thread(self._drop_record, st.task_instance_name)
        try:
            if st.stub is not None:
                await asyncio.wait_for(st.stub.Shutdown(task_manager_pb2.ShutdownRequest()), timeout=60)
        except Exception as e:
            logger.warning("Shutdown RPC to %s failed: %s", st.id, e)
        if st.channel is not None:
            await st.channel.close()
        if st.server is not None:
            await st.server.stop(1.0)
        if st.process is not None:
            await terminate(st.process)
        self.resource.release(st.gpus)
        st.gpus = []

    async def teardown_unit_task(self, task_instance_name: str) -> None:
        async with self.lock:
            st = self.task_managers.pop(task_instance_name, None)
            if st is None:
                raise ValueError(f"Unit task {task_instance_name} is not deployed")
            shared = any(o is st for o in self.task_managers.values())
        try:
            await self._notify_dispatchers(deployed=False, name=task_instance_name)
        except Exception:
            logger.exception("Teardown notification failed for %s", task_instance_name)
        if not shared:
            async with st.lock:
                await self._stop_task_manager(st)
            logger.info("Tore down %s\n%s", task_instance_name, self.resource.render())

    # -- scaling ------------------------------------------------------------------------------------------------------
    async def scale_unit_task(self, task_instance_name: str, num_gpus: int) -> None:
        """Positive ``num_gpus`` adds, negative removes.  GPUs move in chunks of sizes the profile allows
        (largest first), so a request that cannot be tiled exactly is rounded down."""
        st = self.task_managers.get(task_instance_name)
        if st is None:
            raise ValueError(f"Unit task {task_instance_name} is not deployed")
        if num_gpus == 0:
            return
        async with st.lock:
            sizes = sorted((await self.profiles.get_profile(st.task)).gpu_counts(), reverse=True)
            remaining, chunks = abs(num_gpus), []
            for s in sizes:
                while remaining >= s:
                    chunks.append(s)
                    remaining -= s
            if not chunks:
                raise ValueError(f"{abs(num_gpus)} GPUs cannot be formed from executor sizes {sizes}")
            req = task_manager_pb2.UpdateResourcesRequest(task_manager_id=st.id)
            if num_gpus > 0:
                added: list[GPU] = []
                try:
                    for s in chunks:
                        added.extend(self.resource.allocate(s, owner=st.id))
                except Exception:
                    self.resource.release(added)
                    raise
                for g in added:
                    req.gpus.add(action=task_manager_pb2.ResourceAction.ADD, node_id=g.node, global_rank=g.global_rank,
                                 local_rank=g.local_rank)
                try:
                    await st.stub.UpdateResources(req)
                except Exception:
                    self.resource.release(added)
                    raise
                st.gpus.extend(added)
            else:
                count = sum(chunks)
                if count >= len(st.gpus):
                    raise ValueError("Scaling down would remove every GPU of the task; tear it down instead")
                removed = st.gpus[-count:]
                for g in removed:
                    req.gpus.add(action=task_manager_pb2.ResourceAction.REMOVE, node_id=g.node,
                                 global_rank=g.global_rank, local_rank=g.local_rank)
                await st.stub.UpdateResources(req)
                st.gpus = st.gpus[:-count]
                self.resource.release(removed)
        await asyncio.to_thread(self._save_record, st)
        logger.info("Scaled %s by %+d GPUs\n%s", task_instance_name, num_gpus, self.resource.render())

    async def reconcile(self, task_instance_name: str, target_load: float) -> str:
        """Ask the task's manager how many GPUs the load needs and scale accordingly."""
        st = self.task_managers[task_instance_name]
        resp = await st.stub.ReconcileTargetLoad(task_manager_pb2.ReconcileTargetLoadRequest(
            task_id=task_instance_name, target_load=target_load))
        delta = int(resp.message.split(";")[0].split("=")[1]) if resp.message.startswith("delta_gpus=") else 0
        if delta > 0:
            delta = min(delta, self.resource.num_free())
        if delta != 0:
            try:
                await self.scale_unit_task(task_instance_name, delta)
            except ValueError as e:
                return f"{resp.message}; not applied: {e}"
        return resp.message

    # -- health ------------------------------------------------------------------------------------------------------
    async def healthcheck(self) -> tuple[bool, dict[str, bool]]:
        statuses: dict[str, bool] = {}

        async def probe(name: str, st: TaskManagerState) -> None:
            try:
                r = await asyncio.wait_for(st.stub.Healthcheck(task_manager_pb2.HealthcheckRequest()), timeout=1.0)
                statuses[name] = r.status == common_pb2.STATUS_OK
            except Exception:
                statuses[name] = False

        await asyncio.gather(*(probe(n, s) for n, s in list(self.task_managers.items())))
        sidecars_ok = all(p.poll() is None for p in self.sidecars)
        return sidecars_ok and all(statuses.values()), statuses

    # -- dispatchers ----------------------------------------------------------------------------------------------------
    async def _notify_dispatchers(self, deployed: bool, name: str, url: str = "") -> None:
        async def one(addr: str) -> None:
            ch = self._dispatcher_channels.get(addr)
            if ch is None:
                ch = self._dispatcher_channels[addr] = grpc.aio.insecure_channel(addr, interceptors=grpc_client_interceptors())
            stub = task_dispatcher_pb2_grpc.TaskDispatcherStub(ch)
            await stub.SyncTaskRegistry(common_pb2.SyncTaskRegistryRequest(), timeout=60)
            if deployed:
                await stub.NotifyUnitTaskDeployment(task_dispatcher_pb2.NotifyUnitTaskDeploymentRequest(
                    task_instance_name=name, task_manager=task_dispatcher_pb2.TaskManagerDeployment(url=url)), timeout=60)
            else:
                await stub.NotifyUnitTaskTeardown(task_dispatcher_pb2.NotifyUnitTaskTeardownRequest(
                    task_instance_name=name), timeout=60)

        await asyncio.gather(*(one(a) for a in self.dispatcher_urls))

    async def shutdown(self) -> None:
        async with self.lock:
            seen = set()
            for st in list(self.task_managers.values()):
                if id(st) not in seen:
                    seen.add(id(st))
                    await self._stop_task_manager(st)
            self.task_managers.clear()
        for ch in self._dispatcher_channels.values():
            await ch.close()
        for pid in [p.pid for p in self.sidecars] + list(getattr(self, "adopted_sidecar_pids", [])):
            try:
                os.killpg(pid, 15)
            except (ProcessLookupError, PermissionError):
                pass
        if getattr(self, "persist", False):
            for r in range(len(self.resource.gpus)):
                try:
                    self.registry.store.delete(KIND_SIDECAR_RECORD, f"sidecar-{r}")
                except Exception:  # noqa: BLE001
                    pass
        for p in self.sidecars:
            try:
                p.wait(timeout=10)
            except Exception:
                p.kill()
