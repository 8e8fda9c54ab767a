"""In-process registry of task classes, keyed by class name.

Classes arrive either by direct registration (the built-in tasklib registers itself on import) or as
uploaded module sources (reference: python/cornserve/services/task_registry/task_class_registry.py:21-203).
Sources whose imports are not satisfiable yet are parked and retried whenever another module lands.
"""

from __future__ import annotations

import base64
import inspect
from typing import Any

from ...logging import get_logger
from ...task.base import Task, TaskInput, TaskOutput, UnitTask
from .utils import write_to_file_and_import

logger = get_logger(__name__)


def unit_task_io_types(cls: type[UnitTask]) -> tuple[type[TaskInput], type[TaskOutput]] | None:
    """(Input, Output) models from the ``UnitTask[In, Out]`` parametrisation in the class hierarchy."""
    for anc in cls.mro():
        meta = getattr(anc, "__pydantic_generic_metadata__", None)
        origin = meta.get("origin") if meta else None
        # a parametrisation of UnitTask itself or of a generic UnitTask subclass that keeps the
        # (Input, Output) parameter order, e.g. LLMBaseUnitTask[Request, Stream[Chunk]]
        if origin is not None and inspect.isclass(origin) and issubclass(origin, UnitTask) and len(meta["args"]) == 2:
            a, b = meta["args"]
            if inspect.isclass(a) and inspect.isclass(b) and issubclass(a, TaskInput) and issubclass(b, TaskOutput):
                return a, b
    return None


class TaskClassRegistry:
    def __init__(self) -> None:
        self._unit: dict[str, tuple[type[UnitTask], type[TaskInput], type[TaskOutput]]] = {}
        self._composite: dict[str, type[Task]] = {}
        self._pending: list[tuple[str, str, str, bool]] = []

    # -- direct registration ----------------------------------------------------------------------
    def register(self, cls: type[Task], name: str | None = None) -> None:
        name = name or cls.__name__
        if inspect.isclass(cls) and issubclass(cls, UnitTask):
            io = unit_task_io_types(cls)
            if io is None:
                logger.warning("Task class %s has no valid generic type arguments", name)
                return
            self._unit[name] = (cls, io[0], io[1])
            from .descriptor_registry import DESCRIPTOR_REGISTRY

            DESCRIPTOR_REGISTRY.bind_pending_descriptor_for_task_class(cls)
        else:
            self._composite[name] = cls

    # -- uploaded sources ---------------------------------------------------------------------------
    def load_from_source(self, source_code: str, task_class_name: str, module_name: str, is_unit_task: bool = True) -> None:
        """``source_code`` is the base64 of the module source."""
        try:
            self._install(source_code, task_class_name, module_name, is_unit_task)
        except (ImportError, ModuleNotFoundError, NameError) as e:
            logger.info("Deferring task class %s (%s)", task_class_name, e)
            self._pending.append((source_code, task_class_name, module_name, is_unit_task))
            return
        self._retry_pending()

    def _install(self, source_b64: str, class_name: str, module_name: str, is_unit_task: bool) -> None:
        module = write_to_file_and_import(module_name, base64.b64decode(source_b64).decode("utf-8"))
        cls = getattr(module, class_name, None)
        if cls is None or not inspect.isclass(cls):
            raise ValueError(f"Task class {class_name} not found in its source code")
        if is_unit_task and not issubclass(cls, UnitTask):
            raise ValueError(f"{class_name} is not a UnitTask")
        self.register(cls, class_name)

    def _retry_pending(self) -> None:
        progress = True
        while progress and self._pending:
            progress = False
            for item in list(self._pending):
                try:
                    self._install(*item)
                except (ImportError, ModuleNotFoundError, NameError):
                    continue
                self._pending.remove(item)
                progress = True

    # -- lookup ----------------------------------------------------------------------------------------
    def get_unit_task(self, name: str) -> tuple[type[UnitTask], type[TaskInput], type[TaskOutput]]:
        if name not in self._unit:
            raise KeyError(f"Unit task {name} not found in task class registry")
        return self._unit[name]

    def get_composite(self, name: str) -> type[Task]:
        return self._composite[name]

    def __contains__(self, name: str) -> bool:
        return name in self._unit or name in self._composite

    def clear(self) -> None:
        self._unit.clear()
        self._composite.clear()
        self._pending.clear()

    def list_registered_unit_tasks(self) -> list[str]:
        return sorted(self._unit)

    def pending(self) -> list[str]:
        return [p[1] for p in self._pending]


TASK_CLASS_REGISTRY = TaskClassRegistry()


def register_task(cls: Any) -> Any:
    """Class decorator: make a task class resolvable by name in this process."""
    TASK_CLASS_REGISTRY.register(cls)
    return cls
