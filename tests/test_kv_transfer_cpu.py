"""Prefill/decode disaggregation between two executor processes on the CPU: the decode executor cannot map the
producer's cache, so it fetches the pages over HTTP, frees them at the producer and continues the generation."""

import numpy as np
import pytest
import torch

import test_kv_transfer_gpu as flow
from cornserve.services.process import free_port


@pytest.mark.timeout(600)
def test_decode_executor_fetches_kv_pages_over_the_network(tmp_path, monkeypatch):
    monkeypatch.setenv("CORNSERVE_DEVICE", "cpu")
    pp, dp = free_port(), free_port()
    logs = [open(tmp_path / f"{n}.log", "w") for n in ("prefill", "decode")]
    procs = [flow._start("kv_producer", 0, pp, logs[0]), flow._start("kv_consumer", 0, dp, logs[1])]
    try:
        flow._wait_healthy(pp, procs[0])
        flow._wait_healthy(dp, procs[1])
        body = {"model": flow.MODEL, "messages": [{"role": "user", "content": " ".join(f"w{j}" for j in range(150))}],
                "max_completion_tokens": 8, "ignore_eos": True, "temperature": 0, "request_id": "r0"}
        alone = flow._post(f"http://127.0.0.1:{dp}/v1/chat/completions", body)
        first = flow._post(f"http://127.0.0.1:{pp}/v1/chat/completions", body)
        rest = flow._post(f"http://127.0.0.1:{dp}/v1/chat/completions", {**body, "kv_transfer_params": first["kv_transfer_params"]})
        assert rest["cornserve"]["kv_source"] == "network"
        assert rest["choices"][0]["message"]["content"] == alone["choices"][0]["message"]["content"]
        assert flow._post(f"http://127.0.0.1:{pp}/kv/release", {"request_id": "r0"}) == {"released": False}
    finally:
        for p in procs:
            p.terminate()
        for p in procs:
            p.wait(timeout=20)
        for f in logs:
            f.close()


def test_engine_level_transfer_and_page_accounting():
    """Two engines in one process: held pages are described, pulled (both source kinds), and returned to the pool."""
    from cornserve.task_executors.llm.engine import EngineConfig, LLMEngine, PrefilledKV, SamplingParams, Sequence
    from cornserve.models.qwen_llm import LLMConfig, QwenLLM

    cfg = LLMConfig(hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                    intermediate_size=256, vocab_size=512, eos_token_id=511)
    torch.manual_seed(0)
    model = QwenLLM(cfg, device="cpu").float().eval()
    eng = lambda: LLMEngine(model, EngineConfig(num_pages=16, max_batched_tokens=256, decode_burst=2, max_model_len=512))  # noqa: E731
    prompts = [np.arange(3 + i, 150 + 40 * i, dtype=np.int32) for i in range(2)]
    mono = eng().generate([Sequence(f"s{i}", p, SamplingParams(6, True)) for i, p in enumerate(prompts)])
    P, D = eng(), eng()
    free0 = P.blocks.num_free
    P.generate([Sequence(f"s{i}", p, SamplingParams(1, True), hold_kv=True) for i, p in enumerate(prompts)])
    assert set(P.held) == {"s0", "s1"} and P.blocks.num_free < free0
    seqs = []
    for i in range(2):
        kp = P.kv_transfer_params(f"s{i}")
        src = dict(src_cache=P.kv_backing) if i == 0 else dict(raw=P.read_pages(kp["pages"]))
        seqs.append(Sequence(f"s{i}", np.zeros(kp["num_tokens"], np.int32), SamplingParams(6, True),
                             prefilled=PrefilledKV(kp["first_token"], kp["next_pos"], kp["pages"], **src)))
    assert D.generate(seqs) == mono
    assert P.release_held("s0") and P.release_held("s1") and not P.release_held("s0")
    assert P.blocks.num_free == free0 and D.blocks.num_free == free0
    # pages nobody fetched are freed after the hold time
    P.generate([Sequence("s9", prompts[0], SamplingParams(1, True), hold_kv=True)])
    assert P.expire_held(3600) == [] and P.expire_held(0.0) == ["s9"] and P.blocks.num_free == free0


def test_transfer_with_foreign_geometry_is_refused_before_the_engine_sees_it():
    """KV-transfer parameters come from the network: a cache shape, dtype or page list that does not fit this
    executor's cache must be a client error, never an exception inside an engine step."""
    import types

    import pytest

    from cornserve.task_executors.llm.server import LLMServer

    srv = LLMServer.__new__(LLMServer)
    srv.engine = types.SimpleNamespace(kv_geometry=lambda: {"shape": [2, 16, 2, 1, 128, 32], "dtype": "float32"})
    good = {"shape": [2, 64, 2, 1, 128, 32], "dtype": "float32", "pages": [3, 4], "first_token": 1, "next_pos": 9,
            "num_tokens": 200, "request_id": "r"}
    srv._check_transfer(good)   # another pool size is fine
    for bad in ({"shape": [4, 64, 2, 1, 128, 32]}, {"shape": [2, 64, 2, 2, 128, 32]}, {"dtype": "bfloat16"},
                {"pages": [3, 64]}, {"pages": []}, {"pages": "3"}):
        with pytest.raises(ValueError):
            srv._check_transfer({**good, **bad})
    with pytest.raises(ValueError):
        srv._check_transfer({k: v for k, v in good.items() if k != "first_token"})


def test_ipc_description_is_plain_data_and_type_checked():
    import json

    import pytest

    from cornserve.utils.cuda_ipc import import_tensor

    desc = {"tensor_size": [4, 4], "tensor_stride": [4, 1], "tensor_offset": 0, "storage_cls": "UntypedStorage",
            "dtype": "float32", "storage_device": 0, "storage_handle": "", "storage_size_bytes": 64,
            "storage_offset_bytes": 0, "ref_counter_handle": "", "ref_counter_offset": 0, "event_handle": "",
            "event_sync_required": False}
    json.dumps(desc)
    for bad in ({"dtype": "os.system"}, {"storage_cls": "Popen"}, {"tensor_size": [4, 5]}, {"tensor_stride": [4]},
                {"tensor_offset": -1}):
        with pytest.raises((ValueError, TypeError)):
            import_tensor({**desc, **bad})
    with pytest.raises(TypeError):
        import_tensor("gASV...")
