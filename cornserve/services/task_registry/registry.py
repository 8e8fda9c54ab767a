"""Store-backed task registry: persists task definitions, execution descriptors and unit-task instances,
and replicates uploaded classes into every service process through watches.

Same object kinds and spec field names as the reference's custom resources
(python/cornserve/services/task_registry/registry.py:53-616), kept in the local store instead of the
Kubernetes API server.  ``sync_watchers`` blocks until this process has applied every definition /
descriptor event up to the version recorded in the ``LatestTasklibRV`` singleton, which is how a
service makes sure it can resolve the classes named in a request it was just sent.
"""

from __future__ import annotations

import asyncio
import base64
from typing import Any

from ...constants import (KIND_EXECUTION_DESCRIPTOR, KIND_LATEST_TASKLIB_RV, KIND_TASK_DEFINITION,
                          KIND_UNIT_TASK_INSTANCE, SYNC_WATCHERS_TIMEOUT_S)
from ...logging import get_logger
from ...task.base import UnitTask
from ..store import AlreadyExists, LocalStore, NotFound, default_store
from .descriptor_registry import DESCRIPTOR_REGISTRY
from .task_class_registry import TASK_CLASS_REGISTRY
from .utils import purge_tasklib_modules_and_delete_dir

logger = get_logger(__name__)

LATEST_RV_NAME = "latest-tasklib-rv"


class TaskRegistry:
    def __init__(self, store: LocalStore | None = None) -> None:
        self.store = store or default_store()
        self._applied_rv = 0
        self._watch_task: asyncio.Task | None = None
        self._applied = asyncio.Event()

    # -- writers -----------------------------------------------------------------------------------------
    async def create_task_definition(self, name: str, task_class_name: str, module_name: str, source_code: str,
                                     is_unit_task: bool = True) -> dict[str, Any]:
        spec = {
            "taskClassName": task_class_name,
            "moduleName": module_name,
            "sourceCode": base64.b64encode(source_code.encode()).decode(),
            "isUnitTask": is_unit_task,
        }
        try:
            obj = await asyncio.to_thread(self.store.create, KIND_TASK_DEFINITION, name, spec)
        except AlreadyExists:
            raise ValueError(f"Task definition {name} already exists") from None
        await self._bump_latest(max_task_rv=obj.resource_version)
        return spec

    async def create_execution_descriptor(self, name: str, task_class_name: str, descriptor_class_name: str,
                                          module_name: str, source_code: str, is_default: bool = True) -> dict[str, Any]:
        spec = {
            "taskClassName": task_class_name,
            "descriptorClassName": descriptor_class_name,
            "moduleName": module_name,
            "sourceCode": base64.b64encode(source_code.encode()).decode(),
            "isDefault": is_default,
        }
        try:
            obj = await asyncio.to_thread(self.store.create, KIND_EXECUTION_DESCRIPTOR, name, spec)
        except AlreadyExists:
            raise ValueError(f"Execution descriptor {name} already exists") from None
        await self._bump_latest(max_descriptor_rv=obj.resource_version)
        return spec

    async def create_task_instance_from_task(self, task: UnitTask, task_uuid: str) -> str:
        name = f"{type(task).__name__.lower()}-{task_uuid}"
        spec = {
            "definitionRef": type(task).__name__,
            "config": task.model_dump(mode="json"),
            "executionDescriptorName": task.execution_descriptor_name,
        }
        try:
            await asyncio.to_thread(self.store.create, KIND_UNIT_TASK_INSTANCE, name, spec)
        except AlreadyExists:
            raise ValueError(f"Task instance {name} already exists") from None
        return name

    async def get_task_instance(self, instance_name: str) -> UnitTask:
        try:
            obj = await asyncio.to_thread(self.store.get, KIND_UNIT_TASK_INSTANCE, instance_name)
        except NotFound:
            raise ValueError(f"Task instance {instance_name} not found") from None
        task_cls, _, _ = TASK_CLASS_REGISTRY.get_unit_task(obj.spec["definitionRef"])
        return task_cls.model_validate(obj.spec["config"])

    async def delete_task_instance(self, instance_name: str) -> None:
        try:
            await asyncio.to_thread(self.store.delete, KIND_UNIT_TASK_INSTANCE, instance_name)
        except NotFound:
            logger.warning("Task instance %s was already gone", instance_name)

    async def list_task_instances(self) -> list[str]:
        return [o.name for o in await asyncio.to_thread(self.store.list, KIND_UNIT_TASK_INSTANCE)]

    async def check_emptiness(self) -> bool:
        """True when no task definition has been uploaded."""
        return not await asyncio.to_thread(self.store.list, KIND_TASK_DEFINITION, 1)

    async def check_no_active_task_instance(self) -> bool:
        return not await asyncio.to_thread(self.store.list, KIND_UNIT_TASK_INSTANCE, 1)

    async def delete_all_task_definitions_and_descriptors(self) -> None:
        for kind in (KIND_EXECUTION_DESCRIPTOR, KIND_TASK_DEFINITION):
            await asyncio.to_thread(self.store.delete_all, kind)
        await self._bump_latest(max_task_rv=self.store.resource_version(),
                                max_descriptor_rv=self.store.resource_version())

    # -- LatestTasklibRV singleton -------------------------------------------------------------------------
    async def _bump_latest(self, max_task_rv: int | None = None, max_descriptor_rv: int | None = None) -> None:
        def run():
            try:
                cur = self.store.get(KIND_LATEST_TASKLIB_RV, LATEST_RV_NAME).spec
            except NotFound:
                cur = {"maxTaskClassRV": 0, "maxDescriptorRV": 0}
            if max_task_rv is not None:
                cur["maxTaskClassRV"] = max(cur["maxTaskClassRV"], max_task_rv)
            if max_descriptor_rv is not None:
                cur["maxDescriptorRV"] = max(cur["maxDescriptorRV"], max_descriptor_rv)
            self.store.update(KIND_LATEST_TASKLIB_RV, LATEST_RV_NAME, cur, create=True)

        await asyncio.to_thread(run)

    async def get_latest_tasklib_rv(self) -> tuple[int, int]:
        try:
            spec = (await asyncio.to_thread(self.store.get, KIND_LATEST_TASKLIB_RV, LATEST_RV_NAME)).spec
            return int(spec["maxTaskClassRV"]), int(spec["maxDescriptorRV"])
        except NotFound:
            return 0, 0

    # -- replication into this process -------------------------------------------------------------------------
    def _handle_object(self, kind: str, event_type: str, spec: dict[str, Any]) -> None:
        if event_type == "DELETED":
            # a purge invalidates everything that was uploaded; built-in classes register again on demand
            logger.info("Tasklib object deleted: purging uploaded task classes")
            purge_tasklib_modules_and_delete_dir()
            return
        try:
            if kind == KIND_TASK_DEFINITION:
                TASK_CLASS_REGISTRY.load_from_source(spec["sourceCode"], spec["taskClassName"], spec["moduleName"],
                                                     spec.get("isUnitTask", True))
            elif kind == KIND_EXECUTION_DESCRIPTOR:
                DESCRIPTOR_REGISTRY.load_from_source(spec["sourceCode"], spec["descriptorClassName"], spec["moduleName"],
                                                     spec["taskClassName"], spec.get("isDefault", False))
        except Exception:
            logger.exception("Failed to load %s %s", kind, spec.get("taskClassName"))

    async def watch_updates(self) -> None:
        """Apply definition / descriptor events forever (run as a background task)."""
        kinds = (KIND_TASK_DEFINITION, KIND_EXECUTION_DESCRIPTOR)
        while True:
            try:
                async for ev in self.store.watch(None, since=self._applied_rv):
                    if ev.object.kind in kinds:
                        self._handle_object(ev.object.kind, ev.type, ev.object.spec)
                    self._applied_rv = ev.object.resource_version
                    self._applied.set()
            except asyncio.CancelledError:
                raise
            except Exception:
                logger.exception("Registry watch failed; retrying in 5 s")
                await asyncio.sleep(5)

    def start_watching(self) -> asyncio.Task:
        if self._watch_task is None or self._watch_task.done():
            self._watch_task = asyncio.create_task(self.watch_updates())
        return self._watch_task

    async def sync_watchers(self, timeout_s: float = SYNC_WATCHERS_TIMEOUT_S) -> None:
        """Return once every tasklib event up to the recorded latest version has been applied here."""
        want = max(await self.get_latest_tasklib_rv())
        if want == 0:
            return
        self.start_watching()
        deadline = asyncio.get_running_loop().time() + timeout_s
        while self._applied_rv < want:
            remaining = deadline - asyncio.get_running_loop().time()
            if remaining <= 0:
                raise TimeoutError(f"registry watchers did not reach version {want} (at {self._applied_rv})")
            self._applied.clear()
            try:
                await asyncio.wait_for(self._applied.wait(), timeout=min(remaining, 1.0))
            except asyncio.TimeoutError:
                pass

    async def shutdown(self) -> None:
        if self._watch_task is not None:
            self._watch_task.cancel()
            try:
                await self._watch_task
            except (asyncio.CancelledError, Exception):
                pass
            self._watch_task = None
