"""Any-to-any task for Qwen3-Omni-style models (reference: tasklib/cornserve_tasklib/task/composite/omni.py:44-122):
thinker (text) alone, or thinker hidden states -> talker -> vocoder for spoken answers."""

from __future__ import annotations

from cornserve.services.task_registry import register_task
from cornserve.task.base import Stream, Task
from cornserve_tasklib.task.unit.encoder import Modality
from cornserve_tasklib.task.unit.generator import AudioGeneratorInput, AudioGeneratorTask
from cornserve_tasklib.task.unit.llm import ChatCompletionMessageParam, OpenAIChatCompletionChunk, OpenAIChatCompletionRequest
from cornserve_tasklib.task.unit.omni import OMNI_MODEL_ID, OmniTalkerEmbeddingTask, OmniTalkerVocoderInput, OmniTalkerVocoderTask
from cornserve_tasklib.task.composite.llm import MLLMEmbeddingTask, MLLMTask


class OmniInput(OpenAIChatCompletionRequest):
    return_audio: bool = True


@register_task
class OmniTask(Task[OmniInput, Stream[OpenAIChatCompletionChunk]]):
    model_id: str = OMNI_MODEL_ID
    modalities: list[Modality] = []
    encoder_fission: bool = True
    vocoder_fission: bool = True
    coalesce_encoder_invocations: bool = True

    def post_init(self) -> None:
        common = dict(model_id=self.model_id, encoder_fission=self.encoder_fission, modalities=self.modalities,
                      coalesce_encoder_invocations=self.coalesce_encoder_invocations)
        self.thinker_text = MLLMTask(**common)
        self.thinker_embedding = MLLMEmbeddingTask(**common)
        if self.vocoder_fission:
            self.talker_embedding = OmniTalkerEmbeddingTask(model_id=self.model_id)
            self.vocoder_geri = AudioGeneratorTask(model_id=self.model_id)
            self.talker_vocoder = None
        else:
            self.talker_vocoder = OmniTalkerVocoderTask(model_id=self.model_id)
            self.talker_embedding = None
            self.vocoder_geri = None

    def invoke(self, task_input: OmniInput) -> Stream[OpenAIChatCompletionChunk]:
        fields = task_input.model_dump(exclude={"return_audio"})
        thinker_in = OpenAIChatCompletionRequest.model_validate(fields)
        if not task_input.return_audio:
            return self.thinker_text.invoke(thinker_in)
        hidden = self.thinker_embedding.invoke(thinker_in).embeddings
        talker_in = OmniTalkerVocoderInput.model_validate({**fields, "thinker_hidden_states": hidden})
        # the talker continues an assistant turn that starts with the TTS pad token
        talker_in.messages.append(ChatCompletionMessageParam(role="assistant", content="<tts_pad>"))
        if self.vocoder_fission:
            codes = self.talker_embedding.invoke(talker_in).embeddings
            return self.vocoder_geri.invoke(AudioGeneratorInput(embeddings=codes))
        return self.talker_vocoder.invoke(talker_in)
