"""Command-line client and notebook client: the pure helpers, and both clients against a local control plane on CPU
(real gateway / task dispatcher / resource manager / sidecars / tiny executors)."""

import asyncio
import base64
import io
import json
import os
import threading
import time
import uuid
import wave

import pytest

from cornserve.cli.audio_streamer import PCMStreamPlayer
from cornserve.cli.log_streamer import LogStreamer
from cornserve.cli.main import Alias, extract_nested, load_payload, save_png

APP_SOURCE = '''
from collections.abc import AsyncIterator
from cornserve.app.base import AppConfig, AppRequest
from cornserve_tasklib import MLLMTask, Modality, OpenAIChatCompletionRequest, OpenAIChatCompletionChunk

class Request(AppRequest):
    prompt: str
    image_url: str

mllm = MLLMTask(model_id="cornserve-b200/tiny-vlm", modalities=[Modality.IMAGE])

class Config(AppConfig):
    tasks = {"mllm": mllm}

async def serve(request: Request) -> AsyncIterator[OpenAIChatCompletionChunk]:
    content = [{"type": "image_url", "image_url": {"url": request.image_url}}, {"type": "text", "text": request.prompt}]
    return await mllm(OpenAIChatCompletionRequest(model="cornserve-b200/tiny-vlm", ignore_eos=True, temperature=0.0, max_completion_tokens=6,
                                                  messages=[{"role": "user", "content": content}]))
'''


def test_payload_and_nested_lookup(tmp_path):
    assert load_payload('{"a": 1}') == {"a": 1}
    assert load_payload("a: 1\nb: [1, 2]") == {"a": 1, "b": [1, 2]}
    f = tmp_path / "req.yaml"
    f.write_text("prompt: hi")
    assert load_payload(str(f)) == {"prompt": "hi"}
    with pytest.raises(ValueError):
        load_payload("[1, 2]")
    chunk = {"choices": [{"delta": {"content": "x", "audio": {"data": "QUJD"}}}]}
    assert extract_nested(chunk, "choices.0.delta.content") == "x"
    assert extract_nested(chunk, "choices.0.delta.audio.data") == "QUJD"
    assert extract_nested(chunk, "choices.3.delta") is None and extract_nested(chunk, "nope.x") is None


def test_alias_store(tmp_path):
    a = Alias(tmp_path / "alias.json")
    a.set("app-123", "mllm")
    assert Alias(tmp_path / "alias.json").get("mllm") == "app-123" and a.reverse_get("app-123") == "mllm"
    assert a.resolve("mllm") == "app-123" and a.resolve("app-9") == "app-9"
    with pytest.raises(ValueError):
        a.set("app-1", "app-bad")
    a.remove("app-123")
    assert a.get("mllm") is None


def test_png_and_pcm_sinks(tmp_path):
    from cornserve.models.qwen_image import encode_png
    import numpy as np

    b64 = base64.b64encode(encode_png(np.zeros((4, 5, 3), dtype=np.uint8))).decode()
    out = save_png(b64, str(tmp_path / "x.png"))
    assert open(out, "rb").read(4) == b"\x89PNG"
    with pytest.raises(ValueError):
        save_png(base64.b64encode(b"not a png").decode(), None)
    p = PCMStreamPlayer(sample_rate=8000, play=False)
    p.feed(b"\x01\x00" * 100)
    p.feed(b"\x02\x00" * 60)
    p.close()
    with wave.open(io.BytesIO(p.wav_bytes())) as w:
        assert w.getframerate() == 8000 and w.getnframes() == 160


def test_log_streamer_follows_new_executor_logs(tmp_path):
    out = io.StringIO()
    s = LogStreamer(["encoder-x"], log_dir=str(tmp_path), out=out, poll_s=0.05).start()
    f = tmp_path / "te-eric-image-x-0_1.log"
    f.write_text("loading weights\n")
    time.sleep(0.3)
    with open(f, "a") as fh:
        fh.write("ready\n")
    time.sleep(0.3)
    s.stop()
    text = out.getvalue()
    assert "loading weights" in text and "ready" in text and "te-eric-image-x-0" in text


def test_tasklib_explorer_finds_tasks_and_descriptors(tmp_path):
    from cornserve.cli.tasklib_explorer import discover_tasklib

    (tmp_path / "mytasks.py").write_text('''
from cornserve.task.base import UnitTask, TaskInput, TaskOutput
from cornserve.task_executors.descriptor.base import TaskExecutionDescriptor

class EchoIn(TaskInput):
    text: str

class EchoOut(TaskOutput):
    text: str

class EchoTask(UnitTask[EchoIn, EchoOut]):
    model_id: str = "x"

class EchoDescriptor(TaskExecutionDescriptor[EchoTask, EchoIn, EchoOut]):
    pass
''')
    req = discover_tasklib(str(tmp_path))
    assert [t.task_class_name for t in req.task_definitions] == ["EchoTask"] and req.task_definitions[0].is_unit_task
    d = req.descriptor_definitions[0]
    assert d.descriptor_class_name == "EchoDescriptor" and d.task_class_name == "EchoTask" and d.is_default
    assert "class EchoTask" in base64.b64decode(d.source_b64).decode()


@pytest.mark.timeout(600)
def test_cli_and_notebook_client_against_local_cluster(tmp_path, monkeypatch, capsys):
    import socket

    s = socket.socket(); s.bind(("127.0.0.1", 0)); base = s.getsockname()[1]; s.close()
    env = {"CORNSERVE_DEVICE": "cpu", "SIDECAR_DEVICE": "cpu", "CORNSERVE_SIDECAR_BASE_PORT": str(base if base < 60000 else 31000),
           "SIDECAR_NAMESPACE": uuid.uuid4().hex[:8], "CORNSERVE_LOG_DIR": str(tmp_path / "logs"), "CORNSERVE_LOG_LEVEL": "WARNING",
           "CORNSERVE_SEED": "0", "OTEL_SDK_DISABLED": "true", "SIDECAR_SHM_SIZE": str(16 << 20), "CORNSERVE_STATE_DIR": str(tmp_path / "state")}
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    import importlib

    import cornserve.constants as c
    import cornserve.sidecar.constants as sc
    import cornserve.services.sidecar.launch as launch
    import cornserve.cli.main as cli
    import cornserve.cli.log_streamer as ls

    for m in (c, sc, launch, ls, cli):
        importlib.reload(m)
    from cornserve.services.local_cluster import LocalCluster
    from cornserve.services.process import free_port

    loop = asyncio.new_event_loop()
    t = threading.Thread(target=loop.run_forever, daemon=True)
    t.start()
    cluster = LocalCluster(num_gpus=2, cpu=True, gateway_port=free_port(), store_path=str(tmp_path / "store.sqlite"),
                           tm_manager_kwargs={"health_timeout_s": 240}, sidecar_slab_bytes=16 << 20)
    asyncio.run_coroutine_threadsafe(cluster.start(), loop).result(timeout=120)
    monkeypatch.setenv("CORNSERVE_GATEWAY_URL", cluster.url)
    try:
        app = tmp_path / "tinyapp.py"
        app.write_text(APP_SOURCE)
        assert cli.build_parser().parse_args(["list"]).fn(cli.build_parser().parse_args(["list"])) == 0
        args = cli.build_parser().parse_args(["register", str(app), "--alias", "tiny", "--no-logs"])
        assert args.fn(args) == 0
        out = capsys.readouterr().out
        assert "Successfully deployed" in out and "alias tiny" in out
        args = cli.build_parser().parse_args(["list"])
        assert args.fn(args) == 0 and "tiny" in capsys.readouterr().out
        req = json.dumps({"prompt": "what is this", "image_url": "synthetic:224x224:1"})
        args = cli.build_parser().parse_args(["invoke", "tiny", req, "--aggregate-keys", "choices.0.delta.content"])
        assert args.fn(args) == 0
        text = capsys.readouterr().out.strip()
        assert len(text) > 0

        # the notebook client shares the already deployed unit tasks and releases only its own reference
        from cornserve.frontend import CornserveClient
        from cornserve_tasklib import MLLMTask, Modality

        with CornserveClient(cluster.url) as client:
            assert client.is_online()
            task = MLLMTask(model_id="cornserve-b200/tiny-vlm", modalities=[Modality.IMAGE])
            r = client.deploy(task)
            assert r.status == 200, r.content
            assert client.teardown(task).status == 200
        args = cli.build_parser().parse_args(["invoke", "tiny", req, "--aggregate-keys", "choices.0.delta.content"])
        assert args.fn(args) == 0 and capsys.readouterr().out.strip() == text   # the app still works and is deterministic
        args = cli.build_parser().parse_args(["unregister", "tiny"])
        assert args.fn(args) == 0
        args = cli.build_parser().parse_args(["deploy_profiles", os.path.join(os.path.dirname(__file__), "..", "deploy_profiles"), "--dry-run"])
        assert args.fn(args) == 0
        # the comparison harness on the same cluster: deploy a backend shape, drive open-loop load, keep the result by config
        from benchmark.experiment import ExperimentConfig, Workload, run_experiment

        exp = ExperimentConfig("EV", "cornserve-b200/tiny-vlm", {"encoder": 1, "llm": 1},
                               Workload(input_len=8, output_len=4, num_prompts=4, num_warmups=1, request_rate=50.0,
                                        image_width=224, image_height=224))
        res = asyncio.run(run_experiment(exp, cluster.url, str(tmp_path / "bench")))
        assert res["result"]["completed"] == 4 and res["result"]["failed"] == 0, res["result"]
        assert res["result"]["ttft_ms"]["median"] > 0 and exp.result_path(tmp_path / "bench").is_file()
        assert asyncio.run(run_experiment(exp, cluster.url, str(tmp_path / "bench")))["key"] == res["key"]   # served from the file
    finally:
        asyncio.run_coroutine_threadsafe(cluster.stop(), loop).result(timeout=120)
        loop.call_soon_threadsafe(loop.stop)
        t.join(timeout=10)
