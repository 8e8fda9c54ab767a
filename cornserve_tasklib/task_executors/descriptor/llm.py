"""Descriptors of the LLM tasks: launch the LLM executor and speak its OpenAI-compatible API.

Request rewriting is wire-compatible with the reference
(tasklib/cornserve_tasklib/task_executors/descriptor/llm.py:68-563): multimodal URLs become
``data:{modality}/uuid;data_id={forward id};url={original},`` when embeddings arrive through the
sidecars, and forwarding instructions travel in ``vllm_xargs``.  The executor itself is this
repository's own (``cornserve.task_executors.llm.server``), not vLLM; prefill/decode disaggregation
moves KV pages GPU-to-GPU over NVLink instead of NIXL.
"""

from __future__ import annotations

import sys
from collections.abc import AsyncGenerator
from typing import Any, ClassVar

from cornserve.task_executors.descriptor.base import TaskExecutionDescriptor
from cornserve.logging import get_logger
from cornserve.services.resource import GPU
from cornserve.services.task_registry import register_descriptor
from cornserve.task.base import Stream, TaskOutput
from cornserve_tasklib.task.unit.llm import (DecodeLLMUnitTask, LLMBaseUnitTask, LLMEmbeddingResponse, OpenAIChatCompletionChunk,
                             OpenAIChatCompletionRequest, PrefillChatCompletionResponse, PrefillLLMUnitTask,
                             extract_multimodal_content, part_modality_and_url)

logger = get_logger(__name__)

_CONTROL_FIELDS = {"cornserve_embeddings", "cornserve_kv_transfer_params", "encoder_fission"}


async def parse_stream_to_completion_chunks(response: Any) -> AsyncGenerator[str]:
    """OpenAI server-sent events -> one JSON chunk per yielded line (stops at ``[DONE]``)."""
    try:
        async for raw in response.content:
            line = raw.decode().strip()
            if not line:
                continue
            if not line.startswith("data: "):
                logger.warning("Skipping unexpected line in chat completion stream: %s", line)
                continue
            line = line[6:].strip()
            if line.startswith("[DONE]"):
                break
            try:
                OpenAIChatCompletionChunk.model_validate_json(line)
            except Exception:
                logger.exception("Failed to parse chat completion chunk: %s", line)
                break
            yield line
    finally:
        response.close()


def rewrite_multimodal_urls(task_input: OpenAIChatCompletionRequest) -> None:
    """Point every multimodal content part at the forwarded embedding that replaces it."""
    parts = extract_multimodal_content(task_input.messages)
    if len(parts) != len(task_input.cornserve_embeddings):
        raise ValueError(f"The number of multimodal data in messages {len(parts)} != "
                         f"{len(task_input.cornserve_embeddings)} the number of embeddings provided.")
    for part, fwd in zip(parts, task_input.cornserve_embeddings, strict=True):
        modality, url = part_modality_and_url(part)
        url.url = f"data:{modality}/uuid;data_id={fwd.id};url={url.url},"


class _LLMLaunch:
    ROLE_FLAGS: ClassVar[list[str]] = []

    def get_entrypoint(self) -> list[str]:
        return [sys.executable, "-m", "cornserve.task_executors.llm.server"]

    def get_container_envs(self, gpus: list[GPU]) -> list[tuple[str, str]]:
        envs = [("CUDA_VISIBLE_DEVICES", ",".join(str(g.local_rank) for g in gpus))]
        if getattr(self.task, "receive_embeddings", False):
            envs.append(("CORNSERVE_VLLM_DISABLE_MULTIMODAL", "1"))
        return envs

    def get_container_args(self, gpus: list[GPU], port: int) -> list[str]:
        return [
            self.task.model_id,
            "--tensor-parallel-size", str(len(gpus)),
            "--port", str(port),
            "--trust-remote-code",
            "--cornserve-sidecar-ranks", *[str(g.global_rank) for g in gpus],
            "--enforce-eager", "--no-enable-prefix-caching", "--disable-mm-preprocessor-cache",
            "--gpu-memory-utilization", "0.93",
            *self.ROLE_FLAGS,
        ]

    def get_api_url(self, base: str) -> str:
        return f"{base}/v1/chat/completions"


@register_descriptor(LLMBaseUnitTask, default=True)
class VLLMDescriptor(_LLMLaunch, TaskExecutionDescriptor[LLMBaseUnitTask, OpenAIChatCompletionRequest, TaskOutput]):
    """Default descriptor of ``LLMUnitTask`` and ``LLMEmbeddingUnitTask`` (the name is kept for
    compatibility with apps that select descriptors by name)."""

    def create_executor_name(self) -> str:
        return "-".join(["llm", self.task.model_id.split("/")[-1]]).lower()

    def to_request(self, task_input: OpenAIChatCompletionRequest, task_output: TaskOutput) -> dict[str, Any]:
        if self.task.receive_embeddings:
            rewrite_multimodal_urls(task_input)
        req = task_input.model_dump(exclude=_CONTROL_FIELDS)
        if isinstance(task_output, Stream):
            req["stream"] = True
        if isinstance(task_output, LLMEmbeddingResponse):
            req["vllm_xargs"] = {
                "cornserve_hidden_states_forward_id": task_output.embeddings.id,
                "cornserve_hidden_states_forward_ranks": str(task_output.embeddings.dst_sidecar_ranks),
            }
        return req

    async def from_response(self, task_output: TaskOutput, response: Any) -> TaskOutput:
        if isinstance(task_output, Stream):
            return Stream[OpenAIChatCompletionChunk](async_iterator=parse_stream_to_completion_chunks(response),
                                                     response=response)
        if isinstance(task_output, LLMEmbeddingResponse):
            await response.read()
            return LLMEmbeddingResponse(embeddings=task_output.embeddings)
        raise ValueError(f"Expected task output to be Stream or LLMEmbeddingResponse, got {type(task_output)}")


@register_descriptor(PrefillLLMUnitTask, default=True)
class PrefillVLLMDescriptor(_LLMLaunch, TaskExecutionDescriptor[PrefillLLMUnitTask, OpenAIChatCompletionRequest,
                                                                 PrefillChatCompletionResponse]):
    ROLE_FLAGS: ClassVar[list[str]] = ["--kv-transfer-config", '{"kv_connector":"P2PConnector","kv_role":"kv_producer"}']

    def create_executor_name(self) -> str:
        return "-".join(["prefill", self.task.model_id.split("/")[-1]]).lower()

    def to_request(self, task_input: OpenAIChatCompletionRequest, task_output: PrefillChatCompletionResponse) -> dict[str, Any]:
        if self.task.receive_embeddings:
            rewrite_multimodal_urls(task_input)
        req = task_input.model_dump(exclude=_CONTROL_FIELDS)
        req["max_completion_tokens"] = 1  # a prefill executor produces exactly one token
        req["stream"] = False
        xargs: dict[str, str] = {}
        if task_output.kv_transfer_params is not None:
            xargs["cornserve_kv_transfer_params_forward_id"] = task_output.kv_transfer_params.id
            xargs["cornserve_kv_transfer_params_forward_ranks"] = str(task_output.kv_transfer_params.dst_sidecar_ranks)
        if task_output.hidden_states is not None:
            xargs["cornserve_hidden_states_forward_id"] = task_output.hidden_states.id
            xargs["cornserve_hidden_states_forward_ranks"] = str(task_output.hidden_states.dst_sidecar_ranks)
        req["vllm_xargs"] = xargs
        req["kv_transfer_params"] = {"do_remote_decode": True}
        return req

    async def from_response(self, task_output: PrefillChatCompletionResponse, response: Any) -> PrefillChatCompletionResponse:
        await response.read()
        return PrefillChatCompletionResponse(kv_transfer_params=task_output.kv_transfer_params,
                                             hidden_states=task_output.hidden_states)


@register_descriptor(DecodeLLMUnitTask, default=True)
class DecodeVLLMDescriptor(_LLMLaunch, TaskExecutionDescriptor[DecodeLLMUnitTask, OpenAIChatCompletionRequest,
                                                                Stream[OpenAIChatCompletionChunk]]):
    ROLE_FLAGS: ClassVar[list[str]] = ["--kv-transfer-config", '{"kv_connector":"P2PConnector","kv_role":"kv_consumer"}']

    def create_executor_name(self) -> str:
        return "-".join(["decode", self.task.model_id.split("/")[-1]]).lower()

    def to_request(self, task_input: OpenAIChatCompletionRequest, task_output: Stream[OpenAIChatCompletionChunk]) -> dict[str, Any]:
        if self.task.receive_embeddings:
            rewrite_multimodal_urls(task_input)
        if task_input.cornserve_kv_transfer_params is None:
            raise ValueError("KV transfer parameters must be specified in the task input.")
        req = task_input.model_dump(exclude=_CONTROL_FIELDS)
        req["stream"] = True
        req["vllm_xargs"] = {"cornserve_kv_transfer_params_recv_id": task_input.cornserve_kv_transfer_params.id}
        return req

    async def from_response(self, task_output: Stream[OpenAIChatCompletionChunk], response: Any) -> Stream[OpenAIChatCompletionChunk]:
        return Stream[OpenAIChatCompletionChunk](async_iterator=parse_stream_to_completion_chunks(response),
                                                 response=response)
