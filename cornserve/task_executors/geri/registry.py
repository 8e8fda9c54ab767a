"""Which generator class serves which checkpoint (reference:
python/cornserve/task_executors/geri/models/registry.py:14-55).  Diffusers-style checkpoints are recognised by the
``_class_name`` of ``model_index.json``, transformers-style ones by ``model_type`` of ``config.json``."""

from __future__ import annotations

import importlib
from dataclasses import dataclass

import torch

from .api import Modality
from .schema import GeriMode


@dataclass
class RegistryEntry:
    module: str
    class_name: str
    mode: GeriMode
    modality: Modality
    embedding_dtype: torch.dtype     # dtype of the tensors that arrive through the sidecar
    builder: str                     # name of the function in executors.geri.loader that builds + loads the model

    def load_class(self):
        return getattr(importlib.import_module(f"cornserve.models.{self.module}"), self.class_name)


MODEL_REGISTRY: dict[str, RegistryEntry] = {
    "QwenImagePipeline": RegistryEntry("qwen_image", "QwenImageModel", GeriMode.BATCH, Modality.IMAGE, torch.bfloat16,
                                       "build_qwen_image"),
    "qwen3_omni_moe": RegistryEntry("code2wav", "Code2Wav", GeriMode.STREAMING, Modality.AUDIO, torch.int64,
                                    "build_code2wav"),
}
