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
    module: str            # module under cornserve.models
    class_name: str
    config_class: str
    weight: WeightInfo
    modalities: tuple[Modality, ...]
    processor: str         # name of the preprocessing recipe in executors.eric.processor
    adapter_attr: str | None = None

    def load_classes(self):
        mod = importlib.import_module(f"cornserve.models.{self.module}")
        return getattr(mod, self.class_name), getattr(mod, self.config_class)


_QWEN_VL_PREFIXES = ["visual.", "model.visual."]
_IMG_VID = (Modality.IMAGE, Modality.VIDEO)

MODEL_REGISTRY: dict[str, RegistryEntry] = {
    "qwen2_vl": RegistryEntry("qwen2_vl", "Qwen2VisionTransformer", "Qwen2VisionConfig",
                              WeightInfo(_QWEN_VL_PREFIXES), _IMG_VID, "qwen2_vl"),
    "qwen2_5_vl": RegistryEntry("qwen2_5_vl", "Qwen25VisionTransformer", "Qwen25VisionConfig",
                                WeightInfo(_QWEN_VL_PREFIXES), _IMG_VID, "qwen2_vl"),
    "qwen3_vl": RegistryEntry("qwen3_vl", "Qwen3VisionTransformer", "Qwen3VisionConfig",
                              WeightInfo(_QWEN_VL_PREFIXES), _IMG_VID, "qwen3_vl"),
    "qwen3_vl_moe": RegistryEntry("qwen3_vl", "Qwen3VisionTransformer", "Qwen3VisionConfig",
                                  WeightInfo(_QWEN_VL_PREFIXES), _IMG_VID, "qwen3_vl"),
    "qwen2_5_omni": RegistryEntry("qwen_omni", "Qwen25OmniEncoder", "OmniEncoderConfig",
                                  WeightInfo(["thinker."], ignored_prefixes=["model.", "lm_head."]),
                                  (Modality.IMAGE, Modality.VIDEO, Modality.AUDIO), "qwen2_5_omni"),
    "qwen3_omni_moe": RegistryEntry("qwen_omni", "Qwen3OmniEncoder", "OmniEncoderConfig",
                                    WeightInfo(["thinker."], ignored_prefixes=["model.", "lm_head."]),
                                    (Modality.IMAGE, Modality.VIDEO, Modality.AUDIO), "qwen3_omni"),
    "gemma3": RegistryEntry("siglip", "Gemma3VisionEncoder", "Gemma3VisionConfig",
                            WeightInfo(["vision_tower.", "multi_modal_projector.", "model.vision_tower.", "model.multi_modal_projector."],
                                       adapter_prefixes=["multi_modal_projector.", "model.multi_modal_projector."], strip_prefixes=False),
                            (Modality.IMAGE,), "gemma3", adapter_attr="add_adapter"),
    "llava_onevision": RegistryEntry("siglip", "LlavaOnevisionEncoder", "LlavaOnevisionVisionConfig",
                                     WeightInfo(["vision_tower.", "multi_modal_projector.", "image_newline", "model.vision_tower.",
                                                 "model.multi_modal_projector.", "model.image_newline"], strip_prefixes=False),
                                     _IMG_VID, "llava_onevision"),
    "internvl_chat": RegistryEntry("internvl", "InternVLEncoder", "InternVLVisionConfig",
                                   WeightInfo(["vision_model.", "mlp1."], strip_prefixes=False), _IMG_VID, "internvl"),
}


def register_model(model_type: str, entry: RegistryEntry) -> None:
    MODEL_REGISTRY[model_type] = entry
