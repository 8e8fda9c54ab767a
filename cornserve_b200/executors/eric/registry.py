"""Which encoder class serves which Hugging Face ``model_type`` and how its checkpoint is sliced
(reference: python/cornserve/task_executors/eric/models/registry.py:12-233)."""

from __future__ import annotations

import importlib
from dataclasses import dataclass, field

from .schema import Modality


@dataclass
class WeightInfo:
    required_prefixes: list[str]
    ignored_prefixes: list[str] = field(default_factory=list)
    adapter_prefixes: list[str] = field(default_factory=list)
    strip_prefixes: bool = True


@dataclass
class RegistryEntry:
    module: str            # module under cornserve_b200.models
    class_name: str
    config_class: str
    weight: WeightInfo
    modalities: tuple[Modality, ...]
    processor: str         # name of the preprocessing recipe in executors.eric.processor
    adapter_attr: str | None = None

    def load_classes(self):
        mod = importlib.import_module(f"cornserve_b200.models.{self.module}")
        return getattr(mod, self.class_name), getattr(mod, self.config_class)


_QWEN_VL_PREFIXES = ["visual.", "model.visual."]

MODEL_REGISTRY: dict[str, RegistryEntry] = {
    "qwen2_5_vl": RegistryEntry("qwen2_5_vl", "Qwen25VisionTransformer", "Qwen25VisionConfig",
                                WeightInfo(_QWEN_VL_PREFIXES), (Modality.IMAGE, Modality.VIDEO), "qwen2_vl"),
}


def register_model(model_type: str, entry: RegistryEntry) -> None:
    MODEL_REGISTRY[model_type] = entry
