"""Monolithic baseline executor on CPU with tiny random-weight models."""

import base64
import json

import pytest
import torch


@pytest.fixture
def cpu(monkeypatch):
    monkeypatch.setenv("CORNSERVE_DEVICE", "cpu")


def test_image_monolith_generates_png(cpu):
    from fastapi.testclient import TestClient

    from cornserve.task_executors.huggingface.config import HuggingFaceConfig, ModelConfig
    from cornserve.task_executors.huggingface.engine import Engine
    from cornserve.task_executors.huggingface.router import create_app

    cfg = HuggingFaceConfig(model=ModelConfig(id="cornserve-b200/tiny-image-generator", model_type="QWEN_IMAGE",
                                              text_encoder_id="cornserve-b200/tiny-vlm"))
    client = TestClient(create_app(cfg, Engine(cfg, torch.device("cpu"))))
    assert client.get("/health").status_code == 200
    r = client.post("/generate", json={"prompt": "a red cube on a table", "height": 32, "width": 32, "num_inference_steps": 2}).json()
    assert r["status"] == 0, r
    assert base64.b64decode(r["image"])[:8] == b"\x89PNG\r\n\x1a\n"
    assert client.post("/generate", json={"prompt": "x"}).json()["status"] == 1
    with pytest.raises(ValueError):
        HuggingFaceConfig(model=cfg.model, server={"max_batch_size": 2})


def test_omni_monolith_streams_text(cpu):
    from fastapi.testclient import TestClient

    from cornserve.task_executors.huggingface.config import HuggingFaceConfig, ModelConfig
    from cornserve.task_executors.huggingface.engine import Engine
    from cornserve.task_executors.huggingface.router import create_app

    cfg = HuggingFaceConfig(model=ModelConfig(id="cornserve-b200/tiny-vlm", model_type="QWEN_OMNI"))
    client = TestClient(create_app(cfg, Engine(cfg, torch.device("cpu"))))
    body = {"messages": [{"role": "user", "content": "hello there"}], "max_completion_tokens": 6, "ignore_eos": True, "return_audio": False}
    with client.stream("POST", "/generate", json=body) as r:
        items = [json.loads(line) for line in r.iter_lines() if line]
    assert items and all(i["status"] == 0 for i in items)
    assert sum(1 for i in items if i["text_chunk"]["choices"][0]["finish_reason"]) == 1
    with client.stream("POST", "/generate", json={**body, "return_audio": True}) as r:
        items = [json.loads(line) for line in r.iter_lines() if line]
    assert items[-1]["status"] == 1 and "text only" in items[-1]["error_message"]


def test_omni_monolith_speaks(cpu):
    """Thinker, talker and vocoder in one process: text chunks first, then the spoken answer as PCM16."""
    from fastapi.testclient import TestClient

    from cornserve.task_executors.huggingface.config import HuggingFaceConfig, ModelConfig
    from cornserve.task_executors.huggingface.engine import Engine
    from cornserve.task_executors.huggingface.router import create_app

    cfg = HuggingFaceConfig(model=ModelConfig(id="cornserve-b200/tiny-omni", model_type="QWEN_OMNI"))
    client = TestClient(create_app(cfg, Engine(cfg, torch.device("cpu"))))
    body = {"messages": [{"role": "user", "content": "hello there"}], "max_completion_tokens": 5, "ignore_eos": True, "return_audio": True}
    with client.stream("POST", "/generate", json=body) as r:
        items = [json.loads(line) for line in r.iter_lines() if line]
    assert items and all(i["status"] == 0 for i in items), items[-1]
    deltas = [i["text_chunk"]["choices"][0]["delta"] for i in items]
    assert any(d.get("content") for d in deltas)
    audio = b"".join(base64.b64decode(d["audio"]["data"]) for d in deltas if d.get("audio"))
    # sampled speech: its length is open, but the talker cannot stop before a frame and every frame is 48 samples here
    assert len(audio) % 2 == 0
    assert items[-1]["text_chunk"]["choices"][0]["finish_reason"] == "stop"
