"""Placeholders for data that flows executor -> executor through the sidecars, never through the
control plane (reference: python/cornserve/task/forward.py:12-62).  A ``DataForward[T]`` carries an id,
the kind of payload and, once the dispatcher has wired producer and consumers, the sidecar ranks of
the producer and of every consumer group (several groups = broadcast)."""

from __future__ import annotations

import enum
import uuid
from typing import Generic, TypeVar

from pydantic import BaseModel, Field, model_validator


class Tensor:
    """Marker type: ``DataForward[Tensor]`` forwards a tensor."""


class ForwardableType(enum.StrEnum):
    BYTES = "bytes"
    STR = "str"
    INT = "int"
    FLOAT = "float"
    BOOL = "bool"
    TENSOR = "Tensor"
    DICT = "dict"


DataT = TypeVar("DataT")


class DataForward(BaseModel, Generic[DataT]):
    id: str = Field(default_factory=lambda: uuid.uuid4().hex)
    data_type: ForwardableType = Field(init=False, default=ForwardableType.TENSOR)
    src_sidecar_ranks: list[int] | None = Field(init=False, default=None)
    dst_sidecar_ranks: list[list[int]] | None = Field(init=False, default=None)

    @model_validator(mode="after")
    def _set_data_type(self):
        meta = type(self).__pydantic_generic_metadata__
        if meta["origin"] is None:
            raise ValueError("Generic type argument is missing.")
        (arg,) = meta["args"]
        self.data_type = ForwardableType(arg.__name__)
        return self
