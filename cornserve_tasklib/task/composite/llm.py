"""Composite multimodal-LLM tasks (reference: tasklib/cornserve_tasklib/task/composite/llm.py:29-321).

All three graphs start the same way, by turning the multimodal parts of the chat messages into encoder
invocations whose outputs are attached to the LLM request, so that part lives in ``_EncoderFanout``.
"""

from __future__ import annotations

from collections import defaultdict

from cornserve.services.task_registry import register_task
from cornserve.task.base import Stream, Task
from cornserve.task.forward import DataForward, Tensor
from cornserve_tasklib.task.unit.encoder import EncoderInput, EncoderTask, Modality
from cornserve_tasklib.task.unit.llm import (DecodeLLMUnitTask, LLMEmbeddingResponse, LLMEmbeddingUnitTask, LLMUnitTask,
                        OpenAIChatCompletionChunk, OpenAIChatCompletionRequest, PrefillLLMUnitTask,
                        extract_multimodal_content, part_modality_and_url)


class _EncoderFanout:
    """Mixin: ``self.encoders`` (modality -> EncoderTask) and ``_encode`` which runs them for a request.

    With ``coalesce_encoder_invocations`` all URLs of one modality go into a single invocation,
    otherwise there is one invocation per URL.  The returned forwards are in message order.
    """

    def _make_encoders(self) -> None:
        self.encoders = {
            m: EncoderTask(model_ids=self.encoder_model_ids or {self.model_id}, modality=m) for m in self.modalities
        }

    def _encode(self, request: OpenAIChatCompletionRequest) -> list[DataForward[Tensor]]:
        parts = extract_multimodal_content(request.messages)
        by_modality: dict[Modality, list[str]] = defaultdict(list)
        for p in parts:
            mod, url = part_modality_and_url(p)
            by_modality[Modality(mod)].append(url.url)
        if missing := set(by_modality) - set(self.modalities):
            raise ValueError("The following modalities in the input are not specified in the task: "
                             f"{sorted(m.value for m in missing)}")
        forwards: list[DataForward[Tensor]] = []
        if self.coalesce_encoder_invocations:
            queues: dict[Modality, list[DataForward[Tensor]]] = {}
            for mod, enc in self.encoders.items():
                if mod in by_modality:
                    out = enc.invoke(EncoderInput(model_id=request.model, data_urls=by_modality[mod]))
                    queues[mod] = list(out.embeddings)
            for p in parts:
                forwards.append(queues[Modality(part_modality_and_url(p)[0])].pop(0))
        else:
            for p in parts:
                mod, url = part_modality_and_url(p)
                out = self.encoders[Modality(mod)].invoke(EncoderInput(model_id=request.model, data_urls=[url.url]))
                forwards.append(out.embeddings[0])
        return forwards


@register_task
class MLLMTask(Task[OpenAIChatCompletionRequest, Stream[OpenAIChatCompletionChunk]], _EncoderFanout):
    """Encoders (when ``encoder_fission``) followed by a streaming chat completion."""

    model_id: str
    modalities: list[Modality] = []
    encoder_fission: bool = True
    coalesce_encoder_invocations: bool = False
    encoder_model_ids: set[str] | None = None

    def post_init(self) -> None:
        if self.encoder_fission:
            self._make_encoders()
        self.llm = LLMUnitTask(model_id=self.model_id, receive_embeddings=self.encoder_fission)

    def invoke(self, task_input: OpenAIChatCompletionRequest) -> Stream[OpenAIChatCompletionChunk]:
        if self.encoder_fission:
            task_input.cornserve_embeddings = self._encode(task_input)
        return self.llm.invoke(task_input)


@register_task
class MLLMEmbeddingTask(Task[OpenAIChatCompletionRequest, LLMEmbeddingResponse], _EncoderFanout):
    """Like ``MLLMTask`` but ends in the LLM's hidden states (forwarded) instead of text."""

    model_id: str
    modalities: list[Modality] = []
    encoder_fission: bool = True
    coalesce_encoder_invocations: bool = False
    encoder_model_ids: set[str] | None = None

    def post_init(self) -> None:
        if self.encoder_fission:
            self._make_encoders()
        self.llm = LLMEmbeddingUnitTask(model_id=self.model_id, receive_embeddings=self.encoder_fission)

    def invoke(self, task_input: OpenAIChatCompletionRequest) -> LLMEmbeddingResponse:
        if self.encoder_fission:
            task_input.cornserve_embeddings = self._encode(task_input)
        return self.llm.invoke(task_input)


@register_task
class DisaggregatedMLLMTask(Task[OpenAIChatCompletionRequest, Stream[OpenAIChatCompletionChunk]], _EncoderFanout):
    """Encoders -> prefill executor -> decode executor; the prefill's KV-transfer parameters reach the
    decode executor as a forwarded dict."""

    model_id: str
    modalities: list[Modality] = []
    encoder_fission: bool = True
    coalesce_encoder_invocations: bool = False
    encoder_model_ids: set[str] | None = None

    def post_init(self) -> None:
        if self.encoder_fission:
            self._make_encoders()
        self.prefill = PrefillLLMUnitTask(model_id=self.model_id, receive_embeddings=self.encoder_fission)
        self.decode = DecodeLLMUnitTask(model_id=self.model_id, receive_embeddings=self.encoder_fission)

    def invoke(self, task_input: OpenAIChatCompletionRequest) -> Stream[OpenAIChatCompletionChunk]:
        if self.encoder_fission:
            task_input.cornserve_embeddings = self._encode(task_input)
        prefill_out = self.prefill.invoke(task_input)
        decode_in = task_input.model_copy(deep=True)
        decode_in.cornserve_kv_transfer_params = prefill_out.kv_transfer_params
        return self.decode.invoke(decode_in)
