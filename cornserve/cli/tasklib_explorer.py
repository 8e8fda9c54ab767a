"""Finds task classes and execution descriptors in a package (or directory of modules) and packs their module
sources for upload to the gateway (reference: python/cornserve/cli/tasklib_explorer.py:53-195).  A task module
is any module that defines ``Task`` subclasses; a descriptor module defines ``TaskExecutionDescriptor`` subclasses,
whose task class is read from the generic arguments of the descriptor base."""

from __future__ import annotations

import base64
import importlib
import importlib.util
import inspect
import pkgutil
import sys
import typing
from pathlib import Path
from types import ModuleType

from ..task_executors.descriptor.base import TaskExecutionDescriptor
from ..services.gateway.models import DescriptorDefinitionPayload, TaskDefinitionPayload, TasksDeploymentRequest
from ..task.base import Task, UnitTask


def _iter_modules(target: str) -> list[ModuleType]:
    """Modules of an importable package name, or of the ``.py`` files below a directory."""
    p = Path(target)
    mods: list[ModuleType] = []
    if p.exists():
        files = [p] if p.is_file() else sorted(f for f in p.rglob("*.py") if f.name != "__init__.py")
        root = p.parent if p.is_file() else p
        for f in files:
            name = "cornserve_user_tasklib." + ".".join(f.relative_to(root).with_suffix("").parts)
            spec = importlib.util.spec_from_file_location(name, f)
            m = importlib.util.module_from_spec(spec)
            sys.modules[name] = m
            spec.loader.exec_module(m)
            mods.append(m)
        return mods
    pkg = importlib.import_module(target)
    mods.append(pkg)
    if hasattr(pkg, "__path__"):
        for info in pkgutil.walk_packages(pkg.__path__, pkg.__name__ + "."):
            mods.append(importlib.import_module(info.name))
    return mods


def descriptor_task_class(desc_cls: type) -> type | None:
    """The task class a descriptor serves: first generic argument of its ``TaskExecutionDescriptor[...]`` base."""
    meta = getattr(desc_cls, "__pydantic_generic_metadata__", None)
    if meta and meta.get("args"):
        return meta["args"][0]
    for klass in desc_cls.__mro__:
        m = getattr(klass, "__pydantic_generic_metadata__", None)
        if m and m.get("args") and isinstance(m["args"][0], type):
            return m["args"][0]
        for base in getattr(klass, "__orig_bases__", ()):
            args = typing.get_args(base)
            if args and isinstance(args[0], type) and issubclass(args[0], Task):
                return args[0]
    return None


def discover_tasklib(target: str) -> TasksDeploymentRequest:
    tasks: list[TaskDefinitionPayload] = []
    descs: list[DescriptorDefinitionPayload] = []
    for mod in _iter_modules(target):
        try:
            src = base64.b64encode(inspect.getsource(mod).encode()).decode()
        except (OSError, TypeError):
            continue
        for name, obj in vars(mod).items():
            if not inspect.isclass(obj) or obj.__module__ != mod.__name__:
                continue
            if issubclass(obj, Task) and obj not in (Task, UnitTask):
                tasks.append(TaskDefinitionPayload(source_b64=src, task_class_name=name, task_definition_name=name.lower(),
                                                   module_name=mod.__name__, is_unit_task=issubclass(obj, UnitTask)))
            elif issubclass(obj, TaskExecutionDescriptor) and obj is not TaskExecutionDescriptor:
                task_cls = descriptor_task_class(obj)
                if task_cls is None:
                    continue
                descs.append(DescriptorDefinitionPayload(
                    source_b64=src, descriptor_class_name=name, descriptor_definition_name=name.lower(),
                    module_name=mod.__name__, task_class_name=task_cls.__name__,
                    is_default=not any(d.task_class_name == task_cls.__name__ for d in descs)))
    return TasksDeploymentRequest(task_definitions=tasks, descriptor_definitions=descs)
