"""Flags of the monolithic baseline executor (reference: python/cornserve/task_executors/huggingface/config.py:10-40):
``--model.id --model.model-type --server.port --server.max-batch-size`` (batch size must be 1)."""

from __future__ import annotations

from pydantic import BaseModel, model_validator

from .api import ModelType


class ModelConfig(BaseModel):
    id: str
    model_type: ModelType
    text_encoder_id: str = "Qwen/Qwen2.5-VL-7B-Instruct"
    """Language model used as the text encoder of the image pipeline when the checkpoint has no ``text_encoder/``."""


class ServerConfig(BaseModel):
    host: str = "127.0.0.1"
    port: int = 8000
    max_batch_size: int = 1


class HuggingFaceConfig(BaseModel):
    model: ModelConfig
    server: ServerConfig = ServerConfig()

    @model_validator(mode="after")
    def _check(self):
        if self.server.max_batch_size != 1:
            raise ValueError("The monolithic baseline executor serves one request at a time (max_batch_size must be 1)")
        return self
