"""Spoken answers end to end on the CPU with real executors: thinker (LLM executor, MoE decoder) -> talker (LLM executor
in talker mode) -> vocoder, either inside the talker executor or in the generator executor (vocoder fission).  Tiny
random-weight Qwen3-Omni-shaped model; the check is on the plumbing: audio arrives as PCM16 chunks, and both
deployments, which run the same models on the same seeds with greedy decoding, produce the same samples."""

import base64

import numpy as np
import pytest

from test_config1_e2e import _serve_app

APP = '''
from collections.abc import AsyncIterator
from cornserve.app.base import AppConfig, AppRequest
from cornserve_tasklib import OpenAIChatCompletionChunk
from cornserve_tasklib.task.composite.omni import OmniInput, OmniTask

class Request(AppRequest):
    prompt: str
    image_url: str = ""

omni = OmniTask(model_id="cornserve-b200/tiny-omni", modalities=[], vocoder_fission=%s)

class Config(AppConfig):
    tasks = {"omni": omni}

async def serve(request: Request) -> AsyncIterator[OpenAIChatCompletionChunk]:
    return await omni(OmniInput(model="cornserve-b200/tiny-omni", ignore_eos=True, temperature=0.0, max_completion_tokens=6, return_audio=True,
                                messages=[{"role": "user", "content": request.prompt}]))
'''


def _audio_of(chunks):
    data = b"".join(base64.b64decode(ch["choices"][0]["delta"]["audio"]["data"]) for ch in chunks
                    if ch.get("choices") and (ch["choices"][0]["delta"].get("audio") or {}).get("data"))
    assert data, chunks
    return data


@pytest.mark.gpu
@pytest.mark.timeout(900)
def test_omni_task_streams_audio_across_gpus(tmp_path, monkeypatch):
    """Thinker on one B200, talker + vocoder on another (bf16 kernels, MoE layers through the fused expert path)."""
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    monkeypatch.setenv("CORNSERVE_TALKER_GREEDY", "1")
    monkeypatch.setenv("CORNSERVE_TALKER_MIN_FRAMES", "30")
    waves = _serve_app(tmp_path, monkeypatch, APP % False, num_gpus=2, device="cuda", collect=_audio_of)
    assert len(waves) == 5 and all(np.frombuffer(w, dtype=np.int16).size > 100 for w in waves)


@pytest.mark.timeout(900)
@pytest.mark.parametrize("fission", [False, True])
def test_omni_task_streams_audio(tmp_path, monkeypatch, fission):
    monkeypatch.setenv("CORNSERVE_TALKER_GREEDY", "1")
    monkeypatch.setenv("CORNSERVE_TALKER_MIN_FRAMES", "30")   # random weights may prefer the end token at once
    waves = _serve_app(tmp_path, monkeypatch, APP % fission, num_gpus=3 if fission else 2, collect=_audio_of)
    assert len(waves) == 4
    for w in waves:
        pcm = np.frombuffer(w, dtype=np.int16)
        assert pcm.size > 100 and np.abs(pcm.astype(np.int32)).max() > 0
