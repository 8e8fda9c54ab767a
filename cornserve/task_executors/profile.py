"""Unit-task deployment profiles: which GPU counts an executor of a task may use and which extra launch
arguments go with each count (reference: python/cornserve/task_executors/profile.py:35-314; JSON examples
under profiles/).  Profiles live in the object store; lookup is by task equivalence and the default is
"one GPU, no extra arguments"."""

from __future__ import annotations

import asyncio
import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any

from pydantic import BaseModel

from ..constants import KIND_UNIT_TASK_PROFILE
from ..logging import get_logger
from ..services.store import LocalStore, default_store
from ..services.task_registry import TASK_CLASS_REGISTRY
from ..task.base import UnitTask

logger = get_logger(__name__)


class ProfileInfo(BaseModel):
    launch_args: list[str] = []
    # measured sustainable load (requests/s) for this GPU count, when known; used by ReconcileTargetLoad
    max_sustainable_load: float | None = None


@dataclass
class UnitTaskProfile:
    task: UnitTask
    num_gpus_to_profile: dict[int, ProfileInfo] = field(default_factory=lambda: {1: ProfileInfo()})

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "UnitTaskProfile":
        try:
            task_data = dict(data["task"])
            task_cls, _, _ = TASK_CLASS_REGISTRY.get_unit_task(task_data.pop("__class__"))
            task = task_cls.model_validate(task_data)
            table = {int(k): ProfileInfo(**v) for k, v in data["num_gpus_to_profile"].items()}
        except (KeyError, ValueError, TypeError) as e:
            raise ValueError(f"Invalid profile: {e}") from e
        if not table:
            raise ValueError("Invalid profile: no GPU counts")
        return cls(task, table)

    @classmethod
    def from_json_file(cls, path: Path) -> "UnitTaskProfile":
        try:
            return cls.from_dict(json.loads(Path(path).read_text()))
        except json.JSONDecodeError as e:
            raise ValueError(f"Invalid profile file format in {path}: {e}") from e

    def to_dict(self) -> dict[str, Any]:
        task = json.loads(self.task.model_dump_json(exclude={"id", "subtask_attr_names"}))
        task["__class__"] = type(self.task).__name__
        return {"task": task,
                "num_gpus_to_profile": {str(k): v.model_dump(exclude_none=True) for k, v in self.num_gpus_to_profile.items()}}

    def to_json_file(self, path: Path) -> None:
        path = Path(path)
        path.parent.mkdir(parents=True, exist_ok=True)
        path.write_text(json.dumps(self.to_dict(), indent=2))

    def gpu_counts(self) -> list[int]:
        return sorted(self.num_gpus_to_profile)

    def min_gpus(self) -> int:
        return min(self.num_gpus_to_profile)


class UnitTaskProfileManager:
    def __init__(self, store: LocalStore | None = None):
        self.store = store or default_store()

    async def deploy_profile(self, profile: UnitTaskProfile, name: str | None = None) -> str:
        name = name or f"{profile.task.make_name()}-{abs(hash(json.dumps(profile.to_dict(), sort_keys=True))) % 10**8:08d}"
        await asyncio.to_thread(self.store.update, KIND_UNIT_TASK_PROFILE, name, profile.to_dict(), True)
        return name

    async def deploy_directory(self, directory: Path, dry_run: bool = False) -> list[str]:
        names = []
        for f in sorted(Path(directory).glob("*.json")):
            profile = UnitTaskProfile.from_json_file(f)
            names.append(f.stem)
            if not dry_run:
                await self.deploy_profile(profile, f.stem)
        return names

    async def list_profiles(self) -> list[UnitTaskProfile]:
        out = []
        for obj in await asyncio.to_thread(self.store.list, KIND_UNIT_TASK_PROFILE):
            try:
                out.append(UnitTaskProfile.from_dict(obj.spec))
            except ValueError as e:
                logger.warning("Skipping profile %s: %s", obj.name, e)
        return out

    async def get_profile(self, task: UnitTask) -> UnitTaskProfile:
        """Profile of the first stored task equivalent to ``task``; default ``{1: ProfileInfo()}``."""
        for p in await self.list_profiles():
            if p.task.is_equivalent_to(task):
                return p
        return UnitTaskProfile(task)
