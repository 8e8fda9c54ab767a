"""The encoder executor with ``--model.tp-size 2`` as real processes (gloo ranks on the CPU): rank 0 serves HTTP and
runs the engine, rank 1 replays its batches (small part as an object, the pixel tensors by a tensor broadcast), and the
embeddings equal those of a one-rank executor that loaded the same checkpoint."""

import json
import os
import socket
import subprocess
import sys
import time
import urllib.request
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return int(s.getsockname()[1])


def _checkpoint(tmp: Path) -> Path:
    """A tiny Qwen2.5-VL checkpoint in the Hugging Face layout (vision tower under ``visual.``)."""
    sys.path.insert(0, str(ROOT / "tests"))
    from multigpu_fused import vit_weights
    from safetensors.torch import save_file

    from cornserve.models.qwen2_5_vl import Qwen25VisionConfig
    from cornserve.utils.hub import BUILTIN_CONFIGS

    cfg = dict(BUILTIN_CONFIGS["cornserve-b200/tiny-vlm"])
    d = tmp / "tiny-vlm"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(cfg))
    weights = vit_weights(Qwen25VisionConfig.from_hf(cfg))
    save_file({"visual." + k: v.float().contiguous() for k, v in weights.items()}, str(d / "model.safetensors"))
    return d


def _serve(tp: int, dump: Path, model: Path):
    port = _free_port()
    dump.mkdir()
    env = dict(os.environ, CORNSERVE_DEVICE="cpu", CORNSERVE_SEED="0", CORNSERVE_TEST_DUMP_TENSOR_DIR=str(dump),
               PYTHONPATH=str(ROOT) + os.pathsep + os.environ.get("PYTHONPATH", ""), OTEL_SDK_DISABLED="true")
    proc = subprocess.Popen([sys.executable, "-m", "cornserve.task_executors.eric.entrypoint", "--model.id", str(model),
                             "--model.tp-size", str(tp), "--server.port", str(port), "--server.max-batch-size", "4"],
                            env=env, cwd=ROOT)
    deadline = time.time() + 180
    while time.time() < deadline:
        if proc.poll() is not None:
            raise RuntimeError(f"the executor exited with {proc.returncode}")
        try:
            with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=2) as r:
                if r.status == 200:
                    return proc, port
        except Exception:  # noqa: BLE001
            time.sleep(0.5)
    proc.kill()
    raise RuntimeError("the executor did not become healthy")


def _embed(port: int, ids: list[str], model: Path) -> dict:
    body = {"data": [{"id": i, "modality": "image", "model_id": str(model), "url": f"synthetic:112x168:{k}",
                      "receiver_sidecar_ranks": None} for k, i in enumerate(ids)]}
    req = urllib.request.Request(f"http://127.0.0.1:{port}/embeddings", data=json.dumps(body).encode(),
                                 headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=120) as r:
        return json.loads(r.read())


def _get(port: int, path: str) -> dict:
    with urllib.request.urlopen(f"http://127.0.0.1:{port}{path}", timeout=10) as r:
        return json.loads(r.read())


@pytest.mark.timeout(600)
def test_tensor_parallel_encoder_executor_matches_single_rank(tmp_path):
    ids = ["a1", "b2", "c3"]
    outs = {}
    model = _checkpoint(tmp_path)
    for tp in (1, 2):
        proc, port = _serve(tp, tmp_path / f"dump{tp}", model)
        try:
            assert _embed(port, ids, model)["status"] == 0
            assert _embed(port, ["again"], model)["status"] == 0   # a second batch through the same broadcast path
            stats = _get(port, "/stats")
            assert stats["executor"] == "eric" and stats["tp_size"] == tp and stats["items"] == 4
            outs[tp] = {i: torch.load(tmp_path / f"dump{tp}" / f"{i}.pt") for i in ids}
        finally:
            proc.terminate()
            try:
                proc.wait(timeout=20)
            except subprocess.TimeoutExpired:
                proc.kill()
    for i in ids:
        assert outs[1][i].shape == outs[2][i].shape and outs[1][i].shape[1] == 256
        torch.testing.assert_close(outs[2][i], outs[1][i], rtol=1e-4, atol=1e-4)
