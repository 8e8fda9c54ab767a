"""Descriptors of the talker tasks (reference: tasklib/cornserve_tasklib/task_executors/descriptor/omni.py:63-221).
The talker runs in the LLM executor with ``--run-talker`` (and ``--run-vocoder`` when it also vocodes)."""

from __future__ import annotations

from typing import Any, ClassVar

from cornserve.task_executors.descriptor.base import TaskExecutionDescriptor
from cornserve.services.resource import GPU
from cornserve.services.task_registry import register_descriptor
from cornserve.task.base import Stream
from cornserve_tasklib.task.unit.llm import OpenAIChatCompletionChunk
from cornserve_tasklib.task.unit.omni import (OmniTalkerEmbeddingResponse, OmniTalkerEmbeddingTask, OmniTalkerVocoderInput,
                              OmniTalkerVocoderTask)
from cornserve_tasklib.task_executors.descriptor.llm import _CONTROL_FIELDS, _LLMLaunch, parse_stream_to_completion_chunks


class _TalkerLaunch(_LLMLaunch):
    TALKER_FLAGS: ClassVar[list[str]] = ["--run-talker", "--no-enable-chunked-prefill", "--max-num-batched-tokens", "124000",
                    "--disable-chunked-mm-input"]

    def create_executor_name(self) -> str:
        return "-".join(["talker", self.task.model_id.split("/")[-1]]).lower().replace(".", "-")

    def get_container_args(self, gpus: list[GPU], port: int) -> list[str]:
        return [*super().get_container_args(gpus, port), *self.TALKER_FLAGS]

    def _base_request(self, task_input: OmniTalkerVocoderInput) -> dict[str, Any]:
        req = task_input.model_dump(exclude=_CONTROL_FIELDS | {"thinker_hidden_states"})
        req["vllm_xargs"] = {"cornserve_hidden_states_recv_id": task_input.thinker_hidden_states.id}
        return req


@register_descriptor(OmniTalkerVocoderTask, default=True)
class OmniTalkerVocoderDescriptor(_TalkerLaunch, TaskExecutionDescriptor[OmniTalkerVocoderTask, OmniTalkerVocoderInput,
                                                                          Stream[OpenAIChatCompletionChunk]]):
    TALKER_FLAGS: ClassVar[list[str]] = [*_TalkerLaunch.TALKER_FLAGS, "--run-vocoder"]

    def to_request(self, task_input: OmniTalkerVocoderInput, task_output: Stream[OpenAIChatCompletionChunk]) -> dict[str, Any]:
        req = self._base_request(task_input)
        req["stream"] = True
        req["cornserve_return_audio"] = True
        return req

    async def from_response(self, task_output: Stream[OpenAIChatCompletionChunk], response: Any) -> Stream[OpenAIChatCompletionChunk]:
        return Stream[OpenAIChatCompletionChunk](async_iterator=parse_stream_to_completion_chunks(response),
                                                 response=response)


@register_descriptor(OmniTalkerEmbeddingTask, default=True)
class OmniTalkerEmbeddingDescriptor(_TalkerLaunch, TaskExecutionDescriptor[OmniTalkerEmbeddingTask, OmniTalkerVocoderInput,
                                                                            OmniTalkerEmbeddingResponse]):
    def to_request(self, task_input: OmniTalkerVocoderInput, task_output: OmniTalkerEmbeddingResponse) -> dict[str, Any]:
        req = self._base_request(task_input)
        req["stream"] = False
        req["vllm_xargs"].update({
            "cornserve_residual_codes_forward_id": task_output.embeddings.id,
            "cornserve_residual_codes_forward_ranks": str(task_output.embeddings.dst_sidecar_ranks),
        })
        return req

    async def from_response(self, task_output: OmniTalkerEmbeddingResponse, response: Any) -> OmniTalkerEmbeddingResponse:
        await response.read()
        return OmniTalkerEmbeddingResponse(embeddings=task_output.embeddings)
