"""Descriptors of the monolithic baseline tasks (reference:
tasklib/cornserve_tasklib/task_executors/descriptor/huggingface.py:28-150)."""

from __future__ import annotations

import sys
from collections.abc import AsyncGenerator
from typing import Any, ClassVar

from cornserve.task_executors.descriptor.base import TaskExecutionDescriptor
from cornserve.services.resource import GPU
from cornserve.services.task_registry import register_descriptor
from cornserve.task.base import Stream
from cornserve_tasklib.task.unit.huggingface import (HuggingFaceQwenImageInput, HuggingFaceQwenImageOutput, HuggingFaceQwenImageTask,
                                     HuggingFaceQwenOmniInput, HuggingFaceQwenOmniOutput, HuggingFaceQwenOmniTask)


class _MonolithLaunch:
    MODEL_TYPE: ClassVar[str] = ""

    def create_executor_name(self) -> str:
        return "-".join(["hf", self.task.model_id.split("/")[-1]]).lower().replace(".", "-")

    def get_entrypoint(self) -> list[str]:
        return [sys.executable, "-m", "cornserve.task_executors.huggingface.entrypoint"]

    def get_container_args(self, gpus: list[GPU], port: int) -> list[str]:
        return ["--model.id", self.task.model_id, "--model.model-type", self.MODEL_TYPE,
                "--server.port", str(port), "--server.max-batch-size", str(self.task.max_batch_size)]

    def get_api_url(self, base: str) -> str:
        return f"{base}/generate"


@register_descriptor(HuggingFaceQwenImageTask, default=True)
class HuggingFaceQwenImageDescriptor(_MonolithLaunch, TaskExecutionDescriptor[HuggingFaceQwenImageTask,
                                                                              HuggingFaceQwenImageInput,
                                                                              HuggingFaceQwenImageOutput]):
    MODEL_TYPE: ClassVar[str] = "QWEN_IMAGE"

    def to_request(self, task_input: HuggingFaceQwenImageInput, task_output: HuggingFaceQwenImageOutput) -> dict[str, Any]:
        return {"model_type": "qwen_image", **task_input.model_dump()}

    async def from_response(self, task_output: HuggingFaceQwenImageOutput, response: Any) -> HuggingFaceQwenImageOutput:
        body = await response.json()
        if body.get("status", 0) != 0 or not body.get("image"):
            raise RuntimeError(f"Error in monolithic image task: {body.get('error_message')}")
        return HuggingFaceQwenImageOutput(image=body["image"])


async def _ndjson_lines(response: Any) -> AsyncGenerator[str]:
    try:
        async for raw in response.content:
            line = raw.decode().strip()
            if line:
                yield line
    finally:
        response.close()


@register_descriptor(HuggingFaceQwenOmniTask, default=True)
class HuggingFaceQwenOmniDescriptor(_MonolithLaunch, TaskExecutionDescriptor[HuggingFaceQwenOmniTask,
                                                                             HuggingFaceQwenOmniInput,
                                                                             Stream[HuggingFaceQwenOmniOutput]]):
    MODEL_TYPE: ClassVar[str] = "QWEN_OMNI"

    def to_request(self, task_input: HuggingFaceQwenOmniInput, task_output: Stream[HuggingFaceQwenOmniOutput]) -> dict[str, Any]:
        return {"model_type": "qwen_omni", **task_input.model_dump()}

    async def from_response(self, task_output: Stream[HuggingFaceQwenOmniOutput], response: Any) -> Stream[HuggingFaceQwenOmniOutput]:
        return Stream[HuggingFaceQwenOmniOutput](async_iterator=_ndjson_lines(response), response=response)
