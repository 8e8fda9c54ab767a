"""Prefill/decode disaggregation on GPUs with two real executor processes: the decode executor maps the prefill
executor's KV cache (CUDA IPC) and pulls the prompt's pages with the copy kernel: on one GPU, and across NVLink when
two GPUs are visible.  The generated text must equal what one executor produces alone."""

import json
import os
import subprocess
import sys
import time
import urllib.request

import pytest
import torch

from cornserve.services.process import free_port

pytestmark = pytest.mark.gpu

MODEL = "cornserve-b200/tiny-vlm"


def _post(url, body, timeout=120):
    req = urllib.request.Request(url, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=timeout) as r:
        return json.loads(r.read())


def _start(role, gpu, port, log):
    env = dict(os.environ, CORNSERVE_LOCAL_GPUS=str(gpu), CORNSERVE_SEED="0", OTEL_SDK_DISABLED="true", CORNSERVE_LOG_LEVEL="WARNING")
    cmd = [sys.executable, "-m", "cornserve.task_executors.llm.server", MODEL, "--port", str(port), "--num-kv-pages", "64",
           "--max-model-len", "2048", "--kv-transfer-config", json.dumps({"kv_connector": "P2PConnector", "kv_role": role})]
    return subprocess.Popen(cmd, env=env, stdout=log, stderr=subprocess.STDOUT)


def _wait_healthy(port, proc, deadline=240):
    t0 = time.monotonic()
    while time.monotonic() - t0 < deadline:
        if proc.poll() is not None:
            raise RuntimeError(f"executor exited with code {proc.returncode}")
        try:
            with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=2) as r:
                if r.status == 200:
                    return
        except Exception:
            time.sleep(0.5)
    raise RuntimeError("executor did not become healthy")


@pytest.mark.timeout(600)
@pytest.mark.parametrize("consumer_gpu", [0, 1])
def test_decode_executor_pulls_kv_pages_from_prefill_executor(tmp_path, consumer_gpu):
    if consumer_gpu >= torch.cuda.device_count():
        pytest.skip("needs a second GPU")
    pp, dp = free_port(), free_port()
    logs = [open(tmp_path / f"{n}.log", "w") for n in ("prefill", "decode")]
    procs = [_start("kv_producer", 0, pp, logs[0]), _start("kv_consumer", consumer_gpu, dp, logs[1])]
    try:
        _wait_healthy(pp, procs[0])
        _wait_healthy(dp, procs[1])
        for i, n_words in enumerate((5, 300)):   # one page, several pages
            body = {"model": MODEL, "messages": [{"role": "user", "content": " ".join(f"w{i}{j}" for j in range(n_words))}],
                    "max_completion_tokens": 12, "ignore_eos": True, "temperature": 0, "request_id": f"req{i}"}
            alone = _post(f"http://127.0.0.1:{dp}/v1/chat/completions", body)
            first = _post(f"http://127.0.0.1:{pp}/v1/chat/completions", body)
            params = first["kv_transfer_params"]
            assert first["usage"]["completion_tokens"] == 1 and len(params["pages"]) == -(-params["num_tokens"] // 128)
            rest = _post(f"http://127.0.0.1:{dp}/v1/chat/completions", {**body, "kv_transfer_params": params})
            assert rest["cornserve"]["kv_source"] == "mapped", rest
            assert rest["choices"][0]["message"]["content"] == alone["choices"][0]["message"]["content"]
            assert rest["usage"] == alone["usage"]
            # the decode executor already told the producer to free the pages
            assert _post(f"http://127.0.0.1:{pp}/kv/release", {"request_id": f"req{i}"}) == {"released": False}
    except Exception:
        for f in logs:
            f.flush()
        print((tmp_path / "prefill.log").read_text()[-3000:], (tmp_path / "decode.log").read_text()[-3000:])
        raise
    finally:
        for p in procs:
            p.terminate()
        for p in procs:
            try:
                p.wait(timeout=20)
            except subprocess.TimeoutExpired:
                p.kill()
        for f in logs:
            f.close()
