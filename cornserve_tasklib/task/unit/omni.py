"""Talker tasks of Qwen3-Omni-style models (reference: tasklib/cornserve_tasklib/task/unit/omni.py:16-76).
The talker consumes the thinker's hidden states and produces codec codes, either vocoded in the same
executor (``OmniTalkerVocoderTask``) or forwarded to a separate vocoder (``OmniTalkerEmbeddingTask``)."""

from __future__ import annotations

from cornserve.services.task_registry import register_task
from cornserve.task.base import Stream, TaskOutput, UnitTask
from cornserve.task.forward import DataForward, Tensor
from cornserve_tasklib.task.unit.llm import OpenAIChatCompletionChunk, OpenAIChatCompletionRequest

OMNI_MODEL_ID = "Qwen/Qwen3-Omni-30B-A3B-Instruct"


class OmniTalkerVocoderInput(OpenAIChatCompletionRequest):
    thinker_hidden_states: DataForward[Tensor]


def _talker_name(model_id: str) -> str:
    return f"llm-{model_id.split('/')[-1].lower().replace('.', '-')}-talker"


@register_task
class OmniTalkerVocoderTask(UnitTask[OmniTalkerVocoderInput, Stream[OpenAIChatCompletionChunk]]):
    model_id: str = OMNI_MODEL_ID

    def make_name(self) -> str:
        return _talker_name(self.model_id)

    def make_record_output(self, task_input: OmniTalkerVocoderInput) -> Stream[OpenAIChatCompletionChunk]:
        return Stream[OpenAIChatCompletionChunk]()


class OmniTalkerEmbeddingResponse(TaskOutput):
    embeddings: DataForward[Tensor]


@register_task
class OmniTalkerEmbeddingTask(UnitTask[OmniTalkerVocoderInput, OmniTalkerEmbeddingResponse]):
    model_id: str = OMNI_MODEL_ID

    def make_name(self) -> str:
        return _talker_name(self.model_id)

    def make_record_output(self, task_input: OmniTalkerVocoderInput) -> OmniTalkerEmbeddingResponse:
        return OmniTalkerEmbeddingResponse(embeddings=DataForward[Tensor]())
