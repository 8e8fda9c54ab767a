"""Task Manager: owns the executors of one unit task.

Reference behaviour (python/cornserve/services/task_manager/manager.py:69-586) with processes instead of
pods: ``update_resources`` kills every executor that touches a removed GPU, then packs the free GPUs,
per node, into executors of the largest feasible size listed in the task's profile; ``get_route`` is
round robin over healthy executors; spawning waits for ``GET /health`` and reports the tail of the
executor's log when it dies early.  The RPCs the reference leaves unimplemented (``Healthcheck``,
``GetTaskProfile``, ``ReconcileTargetLoad``) are provided.
"""

from __future__ import annotations

import asyncio
import itertools
import os
import time
import uuid
from collections import defaultdict
from dataclasses import dataclass, field

import aiohttp

from ...constants import EXECUTOR_HEALTH_POLL_S, EXECUTOR_HEALTHY_TIMEOUT_S, KIND_EXECUTOR_RECORD
from ...task_executors.profile import UnitTaskProfile, UnitTaskProfileManager
from ...logging import get_logger
from ...task.base import UnitTask
from ..process import ManagedProcess, adopt, free_port, spawn, terminate, to_strict_name
from ..resource import GPU

logger = get_logger(__name__)


def _trace_configs():
    from ...tracing import aiohttp_trace_configs

    return aiohttp_trace_configs()


@dataclass
class ExecutorDeployment:
    executor_id: str
    url: str
    gpus: list[GPU]
    process: ManagedProcess | None
    healthy: bool = True
    spawned_at: float = field(default_factory=time.monotonic)

    @property
    def sidecar_ranks(self) -> list[int]:
        return [g.global_rank for g in self.gpus]


def plan_executors(free_gpus: list[GPU], feasible_sizes: list[int]) -> tuple[list[list[GPU]], list[GPU]]:
    """Split free GPUs into executor-sized groups: per node, largest feasible size first.

    With sizes {1, 2, 4}: 3 GPUs -> [2, 1]; 7 -> [4, 2, 1]; 8 -> [4, 4].  Returns the groups and the GPUs
    that no feasible size could use."""
    sizes = sorted(set(feasible_sizes), reverse=True)
    by_node: dict[str, list[GPU]] = defaultdict(list)
    for g in free_gpus:
        by_node[g.node].append(g)
    groups: list[list[GPU]] = []
    leftover: list[GPU] = []
    for node in sorted(by_node):
        gpus = sorted(by_node[node], key=lambda g: g.global_rank)
        for n in sizes:
            while len(gpus) >= n:
                groups.append(gpus[:n])
                gpus = gpus[n:]
        leftover.extend(gpus)
    return groups, leftover


class TaskManager:
    def __init__(self, task_manager_id: str, task: UnitTask, profile_manager: UnitTaskProfileManager | None = None,
                 spawn_fn=None, health_timeout_s: float | None = None):
        self.id = task_manager_id
        self.task = task
        self.descriptor = task.execution_descriptor
        self.profiles = profile_manager or UnitTaskProfileManager()
        self.gpus: list[GPU] = []
        self.executors: dict[str, ExecutorDeployment] = {}
        self.lock = asyncio.Lock()
        self._rr = itertools.count()
        self._spawn_fn = spawn_fn  # tests inject a fake: async (executor_id, gpus, port, launch_args) -> (url, process|None)
        self._health_timeout = health_timeout_s if health_timeout_s is not None else EXECUTOR_HEALTHY_TIMEOUT_S
        self._http: aiohttp.ClientSession | None = None
        self.target_load: float | None = None

    # -- lifecycle ---------------------------------------------------------------------------------------
    @classmethod
    async def init(cls, task_manager_id: str, task: UnitTask, gpus: list[GPU], **kw) -> "TaskManager":
        tm = cls(task_manager_id, task, **kw)
        await tm.update_resources(add_gpus=gpus)
        return tm

    # -- records: what a restarted control plane needs to find this task's executors again ---------------------------
    def _record(self, dep: ExecutorDeployment) -> None:
        if dep.process is None:
            return
        try:
            self.profiles.store.update(KIND_EXECUTOR_RECORD, dep.executor_id, {
                "task_manager_id": self.id, "url": dep.url, "pid": dep.process.pid, "log_path": str(dep.process.log_path),
                "gpus": [[g.node, g.global_rank, g.local_rank] for g in dep.gpus]}, True)
        except Exception as e:  # noqa: BLE001
            logger.warning("could not record executor %s: %s", dep.executor_id, e)

    def _forget(self, executor_id: str) -> None:
        try:
            self.profiles.store.delete(KIND_EXECUTOR_RECORD, executor_id)
        except Exception:  # noqa: BLE001
            pass

    @classmethod
    async def adopt(cls, task_manager_id: str, task: UnitTask, gpus: list[GPU], records: dict[str, dict], **kw) -> "TaskManager":
        """A task manager around executors that are already running (their control plane was restarted): every recorded
        executor that still answers ``/health`` is taken over as it is, the others are forgotten and their GPUs get new
        executors."""
        tm = cls(task_manager_id, task, **kw)
        client = await tm._client()
        by_rank = {g.global_rank: g for g in gpus}
        for eid, rec in records.items():
            mine = [by_rank[r[1]] for r in rec.get("gpus", []) if r[1] in by_rank]
            ok = False
            if len(mine) == len(rec.get("gpus", [])) and mine:
                try:
                    async with client.get(f"{rec['url']}/health", timeout=aiohttp.ClientTimeout(total=2)) as r:
                        ok = r.status == 200
                except (aiohttp.ClientError, asyncio.TimeoutError):
                    ok = False
            if ok:
                proc = adopt(eid, int(rec["pid"]), log_path=rec.get("log_path", ""))
                tm.executors[eid] = ExecutorDeployment(eid, rec["url"], mine, proc)
                logger.info("Adopted task executor %s at %s (pid %s)", eid, rec["url"], rec["pid"])
            else:
                logger.warning("Recorded task executor %s is gone; its GPUs will get a new one", eid)
                try:
                    os.killpg(int(rec["pid"]), 15)   # whatever is left of it
                except (ProcessLookupError, PermissionError, KeyError, ValueError):
                    pass
                tm._forget(eid)
        await tm.update_resources(add_gpus=gpus)   # GPUs without a live executor are filled as on a first start
        return tm

    async def _client(self) -> aiohttp.ClientSession:
        if self._http is None or self._http.closed:
            self._http = aiohttp.ClientSession(trace_configs=_trace_configs(), timeout=aiohttp.ClientTimeout(total=5))
        return self._http

    async def shutdown(self) -> None:
        async with self.lock:
            await asyncio.gather(*(self._kill_executor(e) for e in list(self.executors)), return_exceptions=True)
            self.gpus.clear()
        if self._http is not None and not self._http.closed:
            await self._http.close()

    # -- resources ------------------------------------------------------------------------------------------
    async def update_resources(self, add_gpus: list[GPU] | None = None, remove_gpus: list[GPU] | None = None) -> None:
        add_gpus, remove_gpus = add_gpus or [], remove_gpus or []
        async with self.lock:
            have = {g.global_rank for g in self.gpus}
            if any(g.global_rank not in have for g in remove_gpus):
                raise ValueError("Cannot remove GPUs that are not allocated")
            if any(g.global_rank in have for g in add_gpus):
                raise ValueError("Cannot add GPUs that are already allocated")
            gone = {g.global_rank for g in remove_gpus}
            self.gpus = [g for g in self.gpus if g.global_rank not in gone] + list(add_gpus)
            # executors that lose any GPU are stopped as a whole (no draining, as in the reference)
            doomed = [eid for eid, d in self.executors.items() if any(g.global_rank in gone for g in d.gpus)]
            results = await asyncio.gather(*(self._kill_executor(e) for e in doomed), return_exceptions=True)
            for r in results:
                if isinstance(r, BaseException):
                    logger.error("Failed to kill task executor: %s", r)
            busy = {g.global_rank for d in self.executors.values() for g in d.gpus}
            free = [g for g in self.gpus if g.global_rank not in busy]
            profile = await self.profiles.get_profile(self.task)
            groups, leftover = plan_executors(free, profile.gpu_counts())
            if leftover:
                logger.warning("%d GPUs stay unused: the profile of %s allows only %s GPUs per executor",
                               len(leftover), self.task.make_name(), profile.gpu_counts())
            results = await asyncio.gather(*(self._spawn_executor(g, profile) for g in groups), return_exceptions=True)
            errors = [str(r) for r in results if isinstance(r, BaseException)]
            if errors:
                raise RuntimeError("Failed to spawn task executors:\n" + ",\n".join(errors))

    async def _spawn_executor(self, gpus: list[GPU], profile: UnitTaskProfile) -> ExecutorDeployment:
        ranks = "-".join(str(g.global_rank) for g in gpus)
        executor_id = to_strict_name(f"te-{self.descriptor.create_executor_name()}-{ranks}")
        launch_args = profile.num_gpus_to_profile[len(gpus)].launch_args
        port = free_port()
        if self._spawn_fn is not None:
            url, proc = await self._spawn_fn(executor_id, gpus, port, launch_args)
        else:
            spec = self.descriptor.launch_spec(gpus, port, launch_args)
            env = dict(spec.env)
            # all GPUs stay visible so that peer memory of other executors can be mapped; the executor
            # selects its devices through CORNSERVE_LOCAL_GPUS
            if "CUDA_VISIBLE_DEVICES" in env:
                env["CORNSERVE_LOCAL_GPUS"] = env.pop("CUDA_VISIBLE_DEVICES")
            proc = spawn(executor_id, spec.argv, env, port)
            url = f"http://127.0.0.1:{port}"
        dep = ExecutorDeployment(executor_id, url, gpus, proc)
        try:
            await self._wait_healthy(dep)
        except Exception:
            if proc is not None:
                await terminate(proc, 2.0)
            raise
        self.executors[executor_id] = dep
        self._record(dep)
        logger.info("Task executor %s is healthy at %s", executor_id, url)
        return dep

    async def _wait_healthy(self, dep: ExecutorDeployment) -> None:
        client = await self._client()
        deadline = time.monotonic() + self._health_timeout
        while time.monotonic() < deadline:
            if dep.process is not None and not dep.process.alive():
                raise RuntimeError(f"Task executor {dep.executor_id} exited with code {dep.process.returncode()}.\n"
                                   f"Last log lines:\n{dep.process.tail(100)}")
            try:
                async with client.get(f"{dep.url}/health") as resp:
                    if resp.status == 200:
                        return
            except (aiohttp.ClientError, asyncio.TimeoutError):
                pass
            await asyncio.sleep(EXECUTOR_HEALTH_POLL_S)
        raise TimeoutError(f"Task executor {dep.executor_id} did not become healthy in {self._health_timeout:.0f} s")

    async def _kill_executor(self, executor_id: str) -> None:
        dep = self.executors.pop(executor_id, None)
        if dep is None:
            return
        self._forget(executor_id)
        if dep.process is not None:
            await terminate(dep.process)
            logger.info("Task executor %s stopped (log kept at %s)", executor_id, dep.process.log_path)

    # -- routing & health ----------------------------------------------------------------------------------------
    async def get_route(self, request_id: str, routing_hint: str | None = None) -> tuple[str, list[int]]:
        """Round robin; a routing hint pins equal hints to the same executor."""
        live = [d for d in self.executors.values() if d.healthy]
        if not live:
            raise RuntimeError(f"No task executors are deployed for {self.task.make_name()}")
        live.sort(key=lambda d: d.executor_id)
        idx = (hash(routing_hint) if routing_hint else next(self._rr)) % len(live)
        d = live[idx]
        return d.url, d.sidecar_ranks

    async def healthcheck(self) -> dict[str, tuple[bool, list[int]]]:
        """Probe every executor; an executor whose process died or whose ``/health`` fails is unhealthy."""
        client = await self._client()
        out: dict[str, tuple[bool, list[int]]] = {}

        async def probe(d: ExecutorDeployment) -> None:
            ok = d.process is None or d.process.alive()
            if ok:
                try:
                    async with client.get(f"{d.url}/health", timeout=aiohttp.ClientTimeout(total=1)) as r:
                        ok = r.status == 200
                except (aiohttp.ClientError, asyncio.TimeoutError):
                    ok = False
            d.healthy = ok
            out[d.executor_id] = (ok, d.sidecar_ranks)

        await asyncio.gather(*(probe(d) for d in list(self.executors.values())))
        return out

    async def respawn_unhealthy(self) -> list[str]:
        """Replace executors that failed the last health check on the same GPUs (elastic recovery)."""
        replaced = []
        async with self.lock:
            profile = await self.profiles.get_profile(self.task)
            for eid, d in list(self.executors.items()):
                if d.healthy:
                    continue
                await self._kill_executor(eid)
                try:
                    await self._spawn_executor(d.gpus, profile)
                    replaced.append(eid)
                except Exception as e:
                    logger.error("Could not replace %s: %s", eid, e)
        return replaced

    async def get_task_profile(self) -> list[tuple[int, float, int]]:
        """``(num_gpus, max_sustainable_load, tensor_parallel_degree)`` per profiled size."""
        profile = await self.profiles.get_profile(self.task)
        return [(n, float(info.max_sustainable_load or 0.0), n) for n, info in sorted(profile.num_gpus_to_profile.items())]

    async def reconcile_target_load(self, target_load: float) -> tuple[int, str]:
        """How many more (+) or fewer (-) GPUs this task should hold to sustain ``target_load`` requests/s,
        from the profiled load of the most efficient executor size.  The resource manager acts on it."""
        self.target_load = target_load
        points = [(n, l) for n, l, _ in await self.get_task_profile() if l > 0]
        if not points:
            return 0, "no sustainable-load figures in the profile; keeping the current allocation"
        n_best, l_best = max(points, key=lambda p: p[1] / p[0])
        executors_needed = max(1, -(-target_load // l_best))
        want = int(executors_needed) * n_best
        delta = want - len(self.gpus)
        return delta, f"target {target_load:.2f} req/s needs {want} GPUs ({int(executors_needed)} x {n_best}); have {len(self.gpus)}"
