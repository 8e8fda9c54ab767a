"""Command-line configuration of the encoder executor, parsed with tyro
(flags as in python/cornserve/task_executors/eric/config.py:20-156: ``--model.id --model.tp-size
--model.modality --server.port --server.max-batch-size --sidecar.ranks [--model.adapter-model-ids]``)."""

from __future__ import annotations

from typing import Annotated

from pydantic import BaseModel, Field, model_validator

from .schema import Modality


class ModelConfig(BaseModel):
    id: str
    adapter_model_ids: list[str] = []
    tp_size: int = 1
    modality: Modality = Modality.IMAGE

    @property
    def all_model_ids(self) -> list[str]:
        return [self.id, *self.adapter_model_ids]


class ServerConfig(BaseModel):
    host: str = "127.0.0.1"
    port: int = 8000
    max_batch_size: int | None = 1


class ImageDataConfig(BaseModel):
    pass


class VideoDataConfig(BaseModel):
    max_num_frames: int = 32


class AudioDataConfig(BaseModel):
    sampling_rate: int = 16000


class ModalityConfig(BaseModel):
    num_workers: int = 12
    image_config: ImageDataConfig = ImageDataConfig()
    video_config: VideoDataConfig = VideoDataConfig()
    audio_config: AudioDataConfig = AudioDataConfig()


class SidecarConfig(BaseModel):
    ranks: list[int] = Field(default_factory=list)


class EricConfig(BaseModel):
    model: ModelConfig
    server: ServerConfig = ServerConfig()
    modality: ModalityConfig = ModalityConfig()
    sidecar: SidecarConfig = SidecarConfig()

    @model_validator(mode="after")
    def _check(self):
        if self.sidecar.ranks and len(self.sidecar.ranks) != self.model.tp_size:
            raise ValueError("The number of sidecar ranks must equal the tensor-parallel degree")
        return self
