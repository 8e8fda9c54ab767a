"""Encoders of the Omni models: one module that owns a vision tower and an audio tower and routes by modality
(reference: python/cornserve/task_executors/eric/models/qwen2_5_omni.py and qwen3_omni_moe.py).

* Qwen2.5-Omni: the Qwen2.5-VL vision tower (checkpoint stores q, k, v separately) + the Conv1d-stem audio tower.
* Qwen3-Omni: the Qwen3-VL vision tower (deep-stack outputs concatenated) + the Conv2d-stem audio tower.
Checkpoint prefixes ``thinker.visual.`` / ``thinker.audio_tower.`` are stripped by the loader; here the names start
with ``visual.`` or ``audio_tower.``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable

import torch
from torch import nn

from ..parallel.state import ParallelGroup, single_group
from .omni_audio import AudioEncoder, AudioEncoderConfig
from .qwen2_5_vl import Qwen25VisionConfig, Qwen25VisionTransformer
from .qwen3_vl import Qwen3VisionConfig, Qwen3VisionTransformer


@dataclass
class OmniEncoderConfig:
    vision: object
    audio: AudioEncoderConfig
    generation: int  # 2 = Qwen2.5-Omni, 3 = Qwen3-Omni

    @classmethod
    def from_hf(cls, cfg: dict) -> "OmniEncoderConfig":
        gen = 3 if "qwen3" in cfg.get("model_type", "") else 2
        thinker = cfg.get("thinker_config", cfg)
        vcfg = thinker.get("vision_config", {})
        vision = (Qwen3VisionConfig if gen == 3 else Qwen25VisionConfig).from_hf({"vision_config": vcfg})
        return cls(vision, AudioEncoderConfig.from_hf({"audio_config": thinker.get("audio_config", {})}, gen == 3), gen)


class _OmniEncoder(nn.Module):
    modalities = ("image", "video", "audio")

    def __init__(self, cfg: OmniEncoderConfig, group: ParallelGroup | None = None, device="cpu"):
        super().__init__()
        self.cfg = cfg
        self.group = group or single_group(device)
        vis_cls = Qwen3VisionTransformer if cfg.generation == 3 else Qwen25VisionTransformer
        self.visual = vis_cls(cfg.vision, self.group, device)
        self.audio_tower = AudioEncoder(cfg.audio, self.group, device)

    @property
    def dtype(self) -> torch.dtype:
        return self.visual.dtype

    @property
    def device(self) -> torch.device:
        return self.visual.device

    @property
    def chunk_shape(self) -> tuple[int, ...]:
        return self.visual.chunk_shape

    def forward(self, modality: str, adapter_name: str | None, batch: dict[str, list]) -> list[torch.Tensor]:
        if modality == "audio":
            return self.audio_tower(modality, adapter_name, batch)
        return self.visual(modality, adapter_name, batch)

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        vis, aud = [], []
        for name, t in weights:
            if name.startswith("visual."):
                vis.append((name[len("visual."):], t))
            elif name.startswith("audio_tower."):
                aud.append((name[len("audio_tower."):], t))
        return {"visual." + n for n in self.visual.load_weights(vis)} | \
               {"audio_tower." + n for n in self.audio_tower.load_weights(aud)}


class Qwen25OmniEncoder(_OmniEncoder):
    pass


class Qwen3OmniEncoder(_OmniEncoder):
    pass
