"""Descriptors of the encoder tasks: launch Eric and speak its ``/embeddings`` API
(reference: tasklib/cornserve_tasklib/task_executors/descriptor/encoder.py:29-170)."""

from __future__ import annotations

import sys
import uuid
from typing import Any

from cornserve.task_executors.descriptor.base import TaskExecutionDescriptor
from cornserve.task_executors.eric.api import EmbeddingData, EmbeddingRequest, EmbeddingResponse, Modality, Status
from cornserve.services.resource import GPU
from cornserve.services.task_registry import register_descriptor
from cornserve_tasklib.task.unit.encoder import DummyEncoderOutput, DummyEncoderTask, EncoderInput, EncoderOutput, EncoderTask


class _EricLaunch:
    """Process launch shared by the real and the dummy encoder descriptors."""

    def create_executor_name(self) -> str:
        first = sorted(self.task.model_ids)[0].split("/")[-1].lower()
        return "-".join(["eric", self.task.modality, first]).lower()

    def get_entrypoint(self) -> list[str]:
        return [sys.executable, "-m", "cornserve.task_executors.eric.entrypoint"]

    def get_container_args(self, gpus: list[GPU], port: int) -> list[str]:
        ids = sorted(self.task.model_ids)
        args = [
            "--model.id", ids[0],
            "--model.tp-size", str(len(gpus)),
            "--model.modality", self.task.modality.value.upper(),
            "--server.port", str(port),
            "--server.max-batch-size", str(self.task.max_batch_size),
            "--sidecar.ranks", *[str(g.global_rank) for g in gpus],
        ]
        if len(ids) > 1:
            args += ["--model.adapter-model-ids", *ids[1:]]
        return args

    def get_api_url(self, base: str) -> str:
        return f"{base}/embeddings"


@register_descriptor(EncoderTask, default=True)
class EricDescriptor(_EricLaunch, TaskExecutionDescriptor[EncoderTask, EncoderInput, EncoderOutput]):
    def to_request(self, task_input: EncoderInput, task_output: EncoderOutput) -> dict[str, Any]:
        data = []
        for url, fwd in zip(task_input.data_urls, task_output.embeddings, strict=True):
            if fwd.dst_sidecar_ranks is None:
                raise ValueError("Destination sidecar ranks must be specified for each forward.")
            data.append(EmbeddingData(id=fwd.id, modality=Modality(self.task.modality.value), model_id=task_input.model_id,
                                      url=url, receiver_sidecar_ranks=fwd.dst_sidecar_ranks))
        return EmbeddingRequest(data=data).model_dump()

    async def from_response(self, task_output: EncoderOutput, response: Any) -> EncoderOutput:
        resp = EmbeddingResponse.model_validate(await response.json())
        if resp.status != Status.SUCCESS:
            raise RuntimeError(f"Error in encoder task: {resp.error_message}")
        return EncoderOutput(embeddings=task_output.embeddings)


@register_descriptor(DummyEncoderTask, default=True)
class DummyEricDescriptor(_EricLaunch, TaskExecutionDescriptor[DummyEncoderTask, EncoderInput, DummyEncoderOutput]):
    def to_request(self, task_input: EncoderInput, task_output: DummyEncoderOutput) -> dict[str, Any]:
        data = [EmbeddingData(id=uuid.uuid4().hex, modality=Modality(self.task.modality.value),
                              model_id=task_input.model_id, url=url, receiver_sidecar_ranks=None)
                for url in task_input.data_urls]
        return EmbeddingRequest(data=data).model_dump()

    async def from_response(self, task_output: DummyEncoderOutput, response: Any) -> DummyEncoderOutput:
        resp = EmbeddingResponse.model_validate(await response.json())
        if resp.status != Status.SUCCESS:
            raise RuntimeError(f"Error in encoder task: {resp.error_message}")
        return DummyEncoderOutput()
