"""The LLM executor with ``--tensor-parallel-size 2`` as real processes (gloo ranks on the CPU): the leader serves HTTP,
the follower mirrors its engine steps, and the answers equal those of a one-rank executor on the same checkpoint."""

import json
import os
import socket
import subprocess
import sys
import time
import urllib.error
import urllib.request
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]

CONFIG = {"model_type": "qwen2", "architectures": ["Qwen2ForCausalLM"], "hidden_size": 64, "num_hidden_layers": 2,
          "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 128, "vocab_size": 512,
          "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "max_position_embeddings": 512, "tie_word_embeddings": False,
          "eos_token_id": 511, "torch_dtype": "float32"}


def _checkpoint(tmp: Path) -> Path:
    from safetensors.torch import save_file

    d = tmp / "tiny-llm"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(CONFIG))
    g = torch.Generator().manual_seed(0)
    H, dh, hq, hkv, inter, V = 64, 16, 4, 2, 128, 512
    r = lambda *s, std=0.08: torch.randn(*s, generator=g) * std  # noqa: E731
    w = {"model.embed_tokens.weight": r(V, H, std=0.5), "model.norm.weight": 1 + r(H), "lm_head.weight": r(V, H, std=0.3)}
    for i in range(2):
        p = f"model.layers.{i}."
        w.update({p + "input_layernorm.weight": 1 + r(H), p + "post_attention_layernorm.weight": 1 + r(H),
                  p + "self_attn.q_proj.weight": r(hq * dh, H), p + "self_attn.q_proj.bias": r(hq * dh),
                  p + "self_attn.k_proj.weight": r(hkv * dh, H), p + "self_attn.k_proj.bias": r(hkv * dh),
                  p + "self_attn.v_proj.weight": r(hkv * dh, H), p + "self_attn.v_proj.bias": r(hkv * dh),
                  p + "self_attn.o_proj.weight": r(H, hq * dh), p + "mlp.gate_proj.weight": r(inter, H),
                  p + "mlp.up_proj.weight": r(inter, H), p + "mlp.down_proj.weight": r(H, inter)})
    save_file({k: v.contiguous() for k, v in w.items()}, str(d / "model.safetensors"))
    return d


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return int(s.getsockname()[1])


def _serve(model_dir: Path, tp: int):
    port = _free_port()
    env = dict(os.environ, CORNSERVE_DEVICE="cpu", PYTHONPATH=str(ROOT) + os.pathsep + os.environ.get("PYTHONPATH", ""))
    proc = subprocess.Popen([sys.executable, "-m", "cornserve.task_executors.llm.server", str(model_dir), "--port", str(port),
                             "--tensor-parallel-size", str(tp), "--num-kv-pages", "16", "--max-model-len", "512",
                             "--max-num-batched-tokens", "64", "--decode-burst", "3"], env=env, cwd=ROOT)
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


def _chat(port: int, text: str, **extra) -> str:
    body = {"model": "tiny-llm", "messages": [{"role": "user", "content": text}], "max_completion_tokens": 12, "ignore_eos": True, "temperature": 0, **extra}
    req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/chat/completions", data=json.dumps(body).encode(),
                                 headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=120) as r:
        return json.loads(r.read())["choices"][0]["message"]["content"]


@pytest.mark.timeout(600)
def test_two_rank_executor_answers_like_one_rank(tmp_path):
    ckpt = _checkpoint(tmp_path)
    prompts = ["hello there", "a much longer question about tensor parallel serving of decoders", "x"]
    answers = {}
    for tp in (1, 2):
        proc, port = _serve(ckpt, tp)
        try:
            got = [_chat(port, p) for p in prompts]
            got.append(_chat(port, prompts[1], temperature=1.1, top_p=0.9, seed=7))
            got.append(_chat(port, prompts[1], temperature=1.1, top_p=0.9, seed=7))
            answers[tp] = got
        finally:
            proc.terminate()
            try:
                proc.wait(timeout=20)
            except subprocess.TimeoutExpired:
                proc.kill()
    assert answers[2][:3] == answers[1][:3]
    assert answers[2][3] == answers[2][4]          # a seeded sampled request repeats on the two-rank executor
    assert answers[2][3] == answers[1][3]          # and draws the same stream as on one rank


def _chat_full(port: int, text: str, **extra) -> dict:
    # sampled with a fixed seed: a random tiny model decodes greedily into one repeated token, which is poor text
    body = {"model": "tiny-llm", "messages": [{"role": "user", "content": text}], "max_completion_tokens": 48, "ignore_eos": True,
            "temperature": 1.5, "seed": 11, **extra}
    req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/chat/completions", data=json.dumps(body).encode(),
                                 headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=120) as r:
        return json.loads(r.read())


@pytest.mark.timeout(600)
@pytest.mark.parametrize("tp", [1, 2])
def test_stop_strings_cut_the_answer_and_free_the_sequence(tmp_path, tp):
    """A ``stop`` string ends the answer before its first occurrence with reason ``stop``; the sequence leaves the engine
    on every rank (the follower of a two-rank executor included: the next requests still answer alike)."""
    ckpt = _checkpoint(tmp_path)
    proc, port = _serve(ckpt, tp)
    try:
        full = _chat_full(port, "tell me something")["choices"][0]
        text = full["message"]["content"]
        assert full["finish_reason"] == "length" and len(text) >= 6
        stop = text[len(text) // 2: len(text) // 2 + 2]
        cut = _chat_full(port, "tell me something", stop=[stop, "\x00never"])["choices"][0]
        assert cut["finish_reason"] == "stop" and cut["message"]["content"] == text[: text.find(stop)]
        again = _chat_full(port, "tell me something")["choices"][0]
        assert again["message"]["content"] == text                    # the engine (all ranks) is in step after the abort
        pen = _chat_full(port, "tell me something", frequency_penalty=1.5, presence_penalty=2.0)["choices"][0]
        assert pen["finish_reason"] == "length"
        # n choices: choice 0 draws the request's own stream (the answer above), the others draw their own
        many = _chat_full(port, "tell me something", n=3)
        assert [c["index"] for c in many["choices"]] == [0, 1, 2] and many["choices"][0]["message"]["content"] == text
        assert len({c["message"]["content"] for c in many["choices"]}) == 3
        assert many["usage"]["completion_tokens"] == 3 * 48
        # log probabilities: one entry per generated token, the chosen token's value and the most likely ones in order
        lp = _chat_full(port, "tell me something", logprobs=True, top_logprobs=4, temperature=0)["choices"][0]
        entries = lp["logprobs"]["content"]
        assert len(entries) == 48
        for e in entries:
            tops = [t["logprob"] for t in e["top_logprobs"]]
            assert len(tops) == 4 and tops == sorted(tops, reverse=True) and e["logprob"] <= 0
            assert abs(e["logprob"] - tops[0]) < 1e-5 and e["token"] == e["top_logprobs"][0]["token"]   # greedy picks the top one
        with urllib.request.urlopen(f"http://127.0.0.1:{port}/stats", timeout=10) as r:
            st = json.loads(r.read())
        assert st["running"] == 0 and st["waiting"] == 0 and st["kv_pages_free"] == st["kv_pages"] - 1
    finally:
        proc.terminate()
        try:
            proc.wait(timeout=20)
        except subprocess.TimeoutExpired:
            proc.kill()


def test_untied_lm_head_of_a_checkpoint_is_loaded(tmp_path, monkeypatch):
    """``lm_head.weight`` sits at the top level of the checkpoint, beside ``model.*``; it must reach the model."""
    from safetensors import safe_open

    from cornserve.task_executors.llm.server import build_engine, parse_args

    monkeypatch.setenv("CORNSERVE_DEVICE", "cpu")
    ckpt = _checkpoint(tmp_path)
    eng, _ = build_engine(parse_args([str(ckpt), "--num-kv-pages", "16", "--max-model-len", "512"]))
    with safe_open(str(ckpt / "model.safetensors"), framework="pt") as f:
        want = f.get_tensor("lm_head.weight")
        emb = f.get_tensor("model.embed_tokens.weight")
    assert torch.allclose(eng.model.lm_head.weight.float(), want.float(), atol=1e-2)
    assert torch.allclose(eng.model.embed_tokens.weight.float(), emb.float(), atol=1e-2)


@pytest.mark.timeout(300)
def test_leader_turns_unhealthy_when_a_follower_rank_exits(tmp_path):
    """Host-side failure: the follower process is ended between requests; the leader's next step fails on the control
    channel, the request gets an error instead of hanging, and ``/health`` reports 503 so that the executor is replaced."""
    import psutil

    ckpt = _checkpoint(tmp_path)
    proc, port = _serve(ckpt, 2)
    try:
        assert _chat(port, "before")                      # both ranks work
        followers = [c for c in psutil.Process(proc.pid).children(recursive=True) if "--tp-rank" in " ".join(c.cmdline())]
        assert len(followers) == 1
        followers[0].kill()
        gone = time.time() + 20     # the leader is its parent, so it lingers as a zombie until the leader reaps it
        while time.time() < gone and followers[0].is_running() and followers[0].status() != psutil.STATUS_ZOMBIE:
            time.sleep(0.1)
        try:
            answer = _chat(port, "after")
        except Exception as e:  # noqa: BLE001  (an HTTP error status is as good as an error body)
            answer = f"error: {e}"
        assert "error" in answer.lower() or answer == ""
        deadline, status = time.time() + 30, 200
        while time.time() < deadline and status == 200:
            try:
                with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=2) as r:
                    status = r.status
            except urllib.error.HTTPError as e:
                status = e.code
            time.sleep(0.3)
        assert status == 503
    finally:
        proc.terminate()
        try:
            proc.wait(timeout=20)
        except subprocess.TimeoutExpired:
            proc.kill()
