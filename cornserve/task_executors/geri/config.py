"""Command-line configuration of the generator executor, parsed with tyro (flags as in
python/cornserve/task_executors/geri/config.py:17-61: ``--model.id --model.modality --server.port
--server.max-batch-size --sidecar.ranks``).  The reference accepts exactly one sidecar rank because its
generators are single-GPU; here ``--model.sp-size N`` runs the diffusion transformer sequence-parallel over N
GPUs and then N sidecar ranks are expected."""

from __future__ import annotations

from pydantic import BaseModel, Field, model_validator

from .api import Modality


class ModelConfig(BaseModel):
    id: str
    modality: Modality = Modality.IMAGE
    sp_size: int = 1
    true_cfg_scale: float = 4.0
    """Classifier-free guidance scale used when a request carries negative embeddings."""
    seed: int = 0


class ServerConfig(BaseModel):
    host: str = "127.0.0.1"
    port: int = 8000
    max_batch_size: int = 1


class SidecarConfig(BaseModel):
    ranks: list[int] = Field(default_factory=list)


class GeriConfig(BaseModel):
    model: ModelConfig
    server: ServerConfig = ServerConfig()
    sidecar: SidecarConfig = SidecarConfig()

    @model_validator(mode="after")
    def _check(self):
        if self.server.max_batch_size < 1:
            raise ValueError("max_batch_size must be at least 1")
        if self.sidecar.ranks and len(self.sidecar.ranks) != self.model.sp_size:
            raise ValueError("The number of sidecar ranks must equal the sequence-parallel degree")
        return self
