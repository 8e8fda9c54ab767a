"""Registry of execution descriptors: task class name -> {descriptor name -> class} plus a default
(reference: python/cornserve/services/task_registry/descriptor_registry.py:20-161).  Descriptors that
arrive before their task class are parked until the class is registered."""

from __future__ import annotations

import base64
import inspect
from typing import Any

from ...logging import get_logger
from .utils import write_to_file_and_import

logger = get_logger(__name__)


class TaskExecutionDescriptorRegistry:
    def __init__(self) -> None:
        self._by_task: dict[str, dict[str, type]] = {}
        self._default: dict[str, type] = {}
        self._pending: dict[str, list[tuple[str, str, str, bool]]] = {}

    def register(self, task: type | str, descriptor: type, name: str | None = None, default: bool = False) -> None:
        task_name = task if isinstance(task, str) else task.__name__
        name = name or descriptor.__name__
        table = self._by_task.setdefault(task_name, {})
        table[name] = descriptor
        if default or task_name not in self._default:
            self._default[task_name] = descriptor

    def load_from_source(self, source_code: str, descriptor_class_name: str, module_name: str, task_class_name: str,
                         is_default: bool = False) -> None:
        from .task_class_registry import TASK_CLASS_REGISTRY

        if task_class_name not in TASK_CLASS_REGISTRY:
            logger.info("Queued execution descriptor %s for task %s until task class is loaded",
                        descriptor_class_name, task_class_name)
            self._pending.setdefault(task_class_name, []).append(
                (source_code, descriptor_class_name, module_name, is_default))
            return
        self._install(source_code, descriptor_class_name, module_name, task_class_name, is_default)

    def _install(self, source_b64: str, class_name: str, module_name: str, task_class_name: str, is_default: bool) -> None:
        module = write_to_file_and_import(module_name, base64.b64decode(source_b64).decode("utf-8"))
        cls = getattr(module, class_name, None)
        if cls is None or not inspect.isclass(cls):
            raise ValueError(f"Descriptor class {class_name} not found in its source code")
        self.register(task_class_name, cls, class_name, is_default)

    def bind_pending_descriptor_for_task_class(self, task: type) -> None:
        for item in self._pending.pop(task.__name__, []):
            src, cls_name, mod_name, is_default = item
            try:
                self._install(src, cls_name, mod_name, task.__name__, is_default)
            except Exception as e:
                logger.warning("Could not bind descriptor %s to %s: %s", cls_name, task.__name__, e)

    def get(self, task: type | str, name: str | None = None) -> type:
        task_name = task if isinstance(task, str) else task.__name__
        if task_name not in self._by_task:
            raise ValueError(f"No descriptors registered for task {task_name}")
        if name is None:
            return self._default[task_name]
        try:
            return self._by_task[task_name][name]
        except KeyError:
            raise ValueError(f"Descriptor {name} not registered for task {task_name}") from None

    def list_registered_descriptors(self) -> dict[str, list[str]]:
        return {t: sorted(d) for t, d in self._by_task.items()}

    def pending(self) -> dict[str, list[str]]:
        return {t: [i[1] for i in items] for t, items in self._pending.items()}

    def clear(self) -> None:
        self._by_task.clear()
        self._default.clear()
        self._pending.clear()


DESCRIPTOR_REGISTRY = TaskExecutionDescriptorRegistry()


def register_descriptor(task: Any, default: bool = False, name: str | None = None):
    """Class decorator binding a descriptor class to a (root) unit task class."""

    def deco(cls):
        DESCRIPTOR_REGISTRY.register(task, cls, name, default)
        return cls

    return deco
