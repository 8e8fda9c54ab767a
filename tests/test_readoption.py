"""A restarted control plane finds its processes again.  The control plane of a live CPU deployment is killed with
SIGKILL (executors and sidecars run in their own sessions and survive); a new control plane over the same store takes
the sidecars and the executors over - same process ids, nothing started twice - and serves the re-registered app."""

import json
import os
import signal
import socket
import subprocess
import sys
import time
import urllib.request
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]

APP = '''
from collections.abc import AsyncIterator
from cornserve.app.base import AppConfig, AppRequest
from cornserve_tasklib import MLLMTask, Modality, OpenAIChatCompletionRequest, OpenAIChatCompletionChunk

class Request(AppRequest):
    prompt: str

mllm = MLLMTask(model_id="cornserve-b200/tiny-vlm", modalities=[Modality.IMAGE])

class Config(AppConfig):
    tasks = {"mllm": mllm}

async def serve(request: Request) -> AsyncIterator[OpenAIChatCompletionChunk]:
    content = [{"type": "image_url", "image_url": {"url": "synthetic:224x224:3"}}, {"type": "text", "text": request.prompt}]
    return await mllm(OpenAIChatCompletionRequest(model="cornserve-b200/tiny-vlm", ignore_eos=True, temperature=0.0,
                                                  max_completion_tokens=6, messages=[{"role": "user", "content": content}]))
'''


def _port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return int(s.getsockname()[1])


def _http(method: str, url: str, body: dict | None = None, timeout: float = 300) -> bytes:
    req = urllib.request.Request(url, data=json.dumps(body).encode() if body is not None else None, method=method,
                                 headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=timeout) as r:
        return r.read()


def _up(env: dict, port: int, log: Path) -> subprocess.Popen:
    proc = subprocess.Popen([sys.executable, "-m", "cornserve.cli.main", "up", "--cpu", "--num-gpus", "2", "--port", str(port)],
                            env=env, cwd=ROOT, stdout=open(log, "w"), stderr=subprocess.STDOUT, start_new_session=True)
    deadline = time.time() + 120
    while time.time() < deadline:
        assert proc.poll() is None, log.read_text()[-2000:]
        try:
            _http("GET", f"http://127.0.0.1:{port}/health", timeout=2)
            return proc
        except Exception:  # noqa: BLE001
            time.sleep(0.3)
    raise AssertionError("the control plane did not come up")


def _register_and_ask(port: int) -> tuple[str, list[dict]]:
    events = [json.loads(line[6:]) for line in _http("POST", f"http://127.0.0.1:{port}/app/register", {"source_code": APP}).decode().splitlines()
              if line.startswith("data: ")]
    assert events[-1]["event"]["type"] == "final", events
    app_id = events[0]["event"]["app_id"]
    chunks = [json.loads(line) for line in _http("POST", f"http://127.0.0.1:{port}/app/invoke/{app_id}",
                                                 {"request_data": {"prompt": "hello"}}).decode().splitlines() if line.strip()]
    assert chunks and all("error" not in c for c in chunks)
    return app_id, json.loads(_http("GET", f"http://127.0.0.1:{port}/cluster/executors"))


@pytest.mark.timeout(600)
def test_restarted_control_plane_adopts_running_executors_and_sidecars(tmp_path):
    import psutil

    env = dict(os.environ, CORNSERVE_DEVICE="cpu", SIDECAR_DEVICE="cpu", CORNSERVE_STORE_PATH=str(tmp_path / "store.sqlite"),
               CORNSERVE_LOG_DIR=str(tmp_path / "logs"), CORNSERVE_SIDECAR_BASE_PORT=str(_port()), SIDECAR_NAMESPACE=f"adopt{os.getpid()}",
               SIDECAR_SHM_SIZE=str(16 << 20), OTEL_SDK_DISABLED="true", CORNSERVE_LOG_LEVEL="INFO", CORNSERVE_SEED="0",
               PYTHONPATH=str(ROOT) + os.pathsep + os.environ.get("PYTHONPATH", ""))
    first = _up(env, _port_a := _port(), tmp_path / "first.log")
    survivors: list[int] = []
    second = None
    try:
        _, before = _register_and_ask(_port_a)
        assert len(before) == 2 and all(e["pid"] for e in before)
        survivors = [e["pid"] for e in before]
        sidecars = [p.pid for p in psutil.Process(first.pid).children(recursive=True) if "sidecar.server" in " ".join(p.cmdline())]
        assert len(sidecars) == 2
        survivors += sidecars
        os.kill(first.pid, signal.SIGKILL)           # the control plane alone; its children are in their own sessions
        first.wait(timeout=10)
        assert all(psutil.pid_exists(p) for p in survivors)
        second = _up(env, _port_b := _port(), tmp_path / "second.log")
        log = (tmp_path / "second.log").read_text()
        assert log.count("Adopted sidecar") == 2 and log.count("Adopted task executor") == 2, log[-3000:]
        adopted = json.loads(_http("GET", f"http://127.0.0.1:{_port_b}/cluster/executors"))
        assert sorted(e["pid"] for e in adopted) == sorted(e["pid"] for e in before)          # taken over, not restarted
        _, after = _register_and_ask(_port_b)                                                  # the app again: served by them
        assert sorted(e["pid"] for e in after) == sorted(e["pid"] for e in before)
    finally:
        for p in (first, second):
            if p is not None and p.poll() is None:
                os.killpg(p.pid, signal.SIGTERM)
                try:
                    p.wait(timeout=30)
                except subprocess.TimeoutExpired:
                    os.killpg(p.pid, signal.SIGKILL)
        time.sleep(0.5)
        for pid in survivors:                          # exactly the processes this test started
            try:
                os.killpg(pid, signal.SIGKILL)
            except (ProcessLookupError, PermissionError):
                pass
