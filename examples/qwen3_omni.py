"""Any-to-any assistant: text, images, video or audio in; text, or speech streamed as PCM, out.  With speech the graph
is thinker (hidden states) -> talker (codec codes) -> vocoder in the generator executor.

    cornserve register examples/qwen3_omni.py
    cornserve invoke qwen3_omni '{"prompt": "Say hello.", "return_audio": true}' --audio-key choices.0.delta.audio.data --save-audio-path hello.wav
"""

from __future__ import annotations

from collections.abc import AsyncIterator

from cornserve.app.base import AppConfig, AppRequest
from cornserve_tasklib import Modality, OmniInput, OmniTask, OpenAIChatCompletionChunk

MODEL = "Qwen/Qwen3-Omni-30B-A3B-Instruct"


class Request(AppRequest):
    prompt: str
    multimodal_data: list[tuple[str, str]] = []
    return_audio: bool = True
    max_completion_tokens: int | None = None


omni = OmniTask(model_id=MODEL, modalities=[Modality.IMAGE, Modality.VIDEO, Modality.AUDIO])


class Config(AppConfig):
    tasks = {"omni": omni}


async def serve(request: Request) -> AsyncIterator[OpenAIChatCompletionChunk]:
    content: list[dict] = [{"type": "text", "text": request.prompt}]
    for modality, url in request.multimodal_data:
        content.append({"type": f"{modality}_url", f"{modality}_url": {"url": url}})
    return await omni(OmniInput(model=MODEL, messages=[{"role": "user", "content": content}], return_audio=request.return_audio,
                                max_completion_tokens=request.max_completion_tokens))
