"""Generator executor: scheduler policy, and the HTTP API end to end on CPU with tiny random-weight models and
the file-backed mock sidecar standing in for the tensor transport."""

import base64
import json

import pytest
import torch

from cornserve.task_executors.geri.api import StreamGeriResponseChunk
from cornserve.task_executors.geri.schema import EngineRequest
from cornserve.task_executors.geri.scheduler import Scheduler


def _req(i, **params):
    return EngineRequest(f"r{i}", torch.zeros(1, 1), params)


def test_scheduler_batches_compatible_prefix():
    s = Scheduler(max_batch_size=3)
    a = dict(height=64, width=64, num_inference_steps=2)
    b = dict(height=128, width=64, num_inference_steps=2)
    for i, p in enumerate([a, a, b, a, a, a, a]):
        s.enqueue(_req(i, **p))
    assert s.schedule().request_ids == ["r0", "r1"]          # stops at the incompatible request
    assert s.schedule().request_ids == ["r2"]
    assert s.schedule().request_ids == ["r3", "r4", "r5"]    # capped by max_batch_size
    assert s.schedule().request_ids == ["r6"]
    assert s.schedule() is None and not s.has_waiting_requests()


def test_scheduler_fcfs_and_abort():
    s = Scheduler(max_batch_size=1)
    for i in range(3):
        s.enqueue(_req(i, chunk_size=4, left_context_size=2))
    with pytest.raises(ValueError):
        s.enqueue(_req(1, chunk_size=4, left_context_size=2))
    assert s.abort("r1") and not s.abort("nope")
    assert [s.schedule().request_ids[0] for _ in range(2)] == ["r0", "r2"]


def test_negative_embeds_split_batches():
    s = Scheduler(max_batch_size=4)
    p = dict(height=64, width=64, num_inference_steps=2)
    s.enqueue(EngineRequest("a", torch.zeros(1, 1), p))
    s.enqueue(EngineRequest("b", torch.zeros(1, 1), p, negative_embeds=torch.zeros(1, 1)))
    assert s.schedule().request_ids == ["a"]


@pytest.fixture
def mock_sidecar(tmp_path, monkeypatch):
    monkeypatch.setenv("CORNSERVE_MOCK_SIDECAR", "1")
    monkeypatch.setenv("CORNSERVE_MOCK_SIDECAR_DIR", str(tmp_path))
    monkeypatch.setenv("CORNSERVE_DEVICE", "cpu")
    return tmp_path


def _client(model_id, modality, mock_dir, dtype, dim, max_batch=2):
    from fastapi.testclient import TestClient

    from cornserve.task_executors.geri.config import GeriConfig, ModelConfig, ServerConfig, SidecarConfig as GSC
    from cornserve.task_executors.geri.engine import Engine
    from cornserve.task_executors.geri.router import create_app
    from cornserve.sidecar.api import Sidecar
    from cornserve.sidecar.schema import SidecarConfig

    cfg = GeriConfig(model=ModelConfig(id=model_id, modality=modality), server=ServerConfig(max_batch_size=max_batch),
                     sidecar=GSC(ranks=[0]))
    engine = Engine(cfg, torch.device("cpu"))
    sidecar = Sidecar(SidecarConfig(sidecar_rank=0, recv_tensor_dtype=dtype, recv_tensor_shape=(-1, dim)))
    return TestClient(create_app(cfg, engine, sidecar)), engine


def test_image_generate_endpoint(mock_sidecar):
    client, engine = _client("cornserve-b200/tiny-image-generator", "image", mock_sidecar, torch.bfloat16, 256)
    try:
        # the conditioning tensor arrives in two chunks; the first two rows are skipped
        torch.save(torch.randn(5, 256).bfloat16(), mock_sidecar / "emb1-0.pt")
        torch.save(torch.randn(3, 256).bfloat16(), mock_sidecar / "emb1-1.pt")
        assert client.get("/health").status_code == 200
        assert client.get("/info").json()["model"]["id"] == "cornserve-b200/tiny-image-generator"
        r = client.post("/image/generate", json={"embedding_data_id": "emb1", "height": 32, "width": 48,
                                                 "num_inference_steps": 2, "skip_tokens": 2})
        body = r.json()
        assert r.status_code == 200 and body["status"] == 0, body
        png = base64.b64decode(body["generated"])
        assert png[:8] == b"\x89PNG\r\n\x1a\n"
        bad = client.post("/image/generate", json={"embedding_data_id": "missing", "height": 32, "width": 32,
                                                   "num_inference_steps": 1}).json()
        assert bad["status"] == 1 and "missing" in bad["error_message"]
    finally:
        engine.shutdown()


def test_audio_generate_streams_pcm(mock_sidecar):
    client, engine = _client("cornserve-b200/tiny-vocoder", "audio", mock_sidecar, torch.int64, 4)
    try:
        torch.save(torch.randint(0, 32, (9, 4)), mock_sidecar / "codes-0.pt")  # [T, num_quantizers]
        with client.stream("POST", "/audio/generate", json={"embedding_data_id": "codes", "chunk_size": 4,
                                                           "left_context_size": 2}) as r:
            assert r.status_code == 200
            chunks = [StreamGeriResponseChunk.model_validate_json(line[6:]).root
                      for line in r.iter_lines() if line.startswith("data: ")]
        assert len(chunks) == 3                       # 9 codes in chunks of 4
        total = sum(len(c) for c in chunks)
        assert 0 < total <= 2 * engine.model.output_length(9)  # every chunk loses the samples its trimming drops
        assert all(len(c) % 2 == 0 for c in chunks)   # PCM16
    finally:
        engine.shutdown()
