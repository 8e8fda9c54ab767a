"""CPU plumbing configuration end to end with *real* executors: gateway -> task dispatcher -> Eric (tiny
Qwen2.5-VL-style vision tower) -> sidecar -> LLM executor (tiny decoder), fp32, TP=1, no GPU.  Four requests,
each one synthetic 224x224 image plus a text prompt, 16 greedy output tokens.  The streamed text must equal
what the in-process monolithic pipeline produces with the same (seeded) random weights."""

import asyncio
import json
import os
import socket
import uuid

import aiohttp
import numpy as np
import pytest
import torch
import uvicorn

APP_SOURCE = '''
from collections.abc import AsyncIterator
from cornserve.app.base import AppConfig, AppRequest
from cornserve_tasklib import MLLMTask, Modality, OpenAIChatCompletionRequest, OpenAIChatCompletionChunk

class Request(AppRequest):
    prompt: str
    image_url: str
    max_completion_tokens: int = 16

mllm = MLLMTask(model_id="cornserve-b200/tiny-vlm", modalities=[Modality.IMAGE])

class Config(AppConfig):
    tasks = {"mllm": mllm}

async def serve(request: Request) -> AsyncIterator[OpenAIChatCompletionChunk]:
    content = [{"type": "image_url", "image_url": {"url": request.image_url}}, {"type": "text", "text": request.prompt}]
    return await mllm(OpenAIChatCompletionRequest(model="cornserve-b200/tiny-vlm", ignore_eos=True, temperature=0.0,
                                                  max_completion_tokens=request.max_completion_tokens,
                                                  messages=[{"role": "user", "content": content}]))
'''


def _port_block(n):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p if p + n < 65000 else 30000


def _expected_text(prompt: str, image_url: str, n_tokens: int, device: str = "cpu") -> str:
    """The same request through the in-process pipeline with identically seeded weights."""
    from cornserve.task_executors.eric.processor import load_image
    from cornserve.task_executors.llm.engine import EngineConfig
    from cornserve.task_executors.llm.tokenizer import load_tokenizer
    from cornserve.models.qwen2_5_vl import Qwen25VisionConfig, Qwen25VisionTransformer
    from cornserve.models.qwen_llm import LLMConfig, QwenLLM
    from cornserve.pipelines import MLLMPipeline
    from cornserve.task_executors.llm.engine import SamplingParams, Sequence, MMItem
    from cornserve.utils.hub import load_config

    cfg = load_config("cornserve-b200/tiny-vlm")
    torch.manual_seed(0)
    vision = Qwen25VisionTransformer(Qwen25VisionConfig.from_hf(cfg), device=device).eval()
    torch.manual_seed(0)
    llm = QwenLLM(LLMConfig.from_hf(cfg), device=device).eval()
    if device == "cpu":
        vision, llm = vision.float(), llm.float()
    pipe = MLLMPipeline(vision, llm, EngineConfig(num_pages=16, decode_burst=4, max_model_len=2048, use_cuda_graph=device != "cpu"))
    tok = load_tokenizer("cornserve-b200/tiny-vlm", cfg, llm.cfg.vocab_size)
    (emb, grid), = pipe.encode_images([torch.from_numpy(load_image(image_url))])
    ids, marks = tok.render_chat([{"role": "user", "content": [{"type": "image_url", "image_url": {"url": image_url}},
                                                               {"type": "text", "text": prompt}]}])
    (pos, _), = marks
    full = ids[:pos] + [ids[pos]] * emb.shape[0] + ids[pos + 1:]
    seq = Sequence("x", np.asarray(full, dtype=np.int32), SamplingParams(n_tokens, True), mm_items=[MMItem(emb, pos, grid)])
    return tok.decode(pipe.engine.generate([seq])["x"])


DISAGG_APP_SOURCE = APP_SOURCE.replace("import MLLMTask,", "import DisaggregatedMLLMTask,").replace(
    "mllm = MLLMTask(", "mllm = DisaggregatedMLLMTask(")


@pytest.mark.timeout(600)
def test_cpu_plumbing_with_real_executors(tmp_path, monkeypatch):
    texts = _serve_app(tmp_path, monkeypatch, APP_SOURCE, num_gpus=2)
    for i in (0, 3):
        assert texts[i] == _expected_text(f"describe picture {i}", f"synthetic:224x224:{i}", 16)


@pytest.mark.timeout(600)
def test_cpu_disaggregated_prefill_and_decode_executors(tmp_path, monkeypatch):
    """Encoder -> prefill executor -> decode executor: the prefill executor answers after one token and forwards where
    its KV pages are; the decode executor fetches them (over HTTP here: CPU engines have no GPU cache to map), frees
    them at the producer and streams the rest.  The text must equal the monolithic pipeline's."""
    texts = _serve_app(tmp_path, monkeypatch, DISAGG_APP_SOURCE, num_gpus=3)
    for i in (0, 3):
        assert texts[i] == _expected_text(f"describe picture {i}", f"synthetic:224x224:{i}", 16)


@pytest.mark.gpu
@pytest.mark.timeout(900)
@pytest.mark.parametrize("app", ["mllm", "disaggregated"])
def test_gpu_plumbing_across_gpus(tmp_path, monkeypatch, app):
    """The same deployments with every executor on its own B200: encoder rows travel through the sidecars' GPU slabs
    (mapped by the consumer and read in place over NVLink), and the decode executor pulls KV pages from the prefill
    executor's cache with the copy kernel.  bf16 on the GPU: every request must stream, repeating a request must
    repeat its text, and a request that runs alone must produce the text of the in-process pipeline."""
    need = 2 if app == "mllm" else 3
    if torch.cuda.device_count() < need:
        pytest.skip(f"needs {need} GPUs")
    texts = _serve_app(tmp_path, monkeypatch, APP_SOURCE if app == "mllm" else DISAGG_APP_SOURCE, num_gpus=need, device="cuda")
    assert len(texts) == 5
    # request 1 once more, alone in its batch like the in-process pipeline runs it (same seeds, same kernels)
    assert texts[4] == _expected_text("describe picture 1", "synthetic:224x224:1", 16, device="cuda")


def _text_of(chunks):
    return "".join((ch["choices"][0]["delta"].get("content") or "") for ch in chunks if ch.get("choices"))


def _serve_app(tmp_path, monkeypatch, app_source, num_gpus, device="cpu", collect=_text_of, request_of=None,
               extra_env=None):
    base = _port_block(16)
    ns = uuid.uuid4().hex[:8]
    monkeypatch.delenv("CORNSERVE_DEVICE", raising=False)
    monkeypatch.delenv("SIDECAR_DEVICE", raising=False)
    env = {
        **({"CORNSERVE_DEVICE": "cpu", "SIDECAR_DEVICE": "cpu"} if device == "cpu" else {}),
        "CORNSERVE_SIDECAR_BASE_PORT": str(base),
        "SIDECAR_NAMESPACE": ns, "CORNSERVE_STORE_PATH": str(tmp_path / "store.sqlite"),
        "CORNSERVE_LOG_DIR": str(tmp_path / "logs"), "CORNSERVE_LOG_LEVEL": "WARNING", "CORNSERVE_SEED": "0",
        "OTEL_SDK_DISABLED": "true", "SIDECAR_SHM_SIZE": str(16 << 20),
    }
    for k, v in {**env, **(extra_env or {})}.items():
        monkeypatch.setenv(k, v)
    import importlib

    import cornserve.constants as c
    import cornserve.sidecar.constants as sc
    import cornserve.services.sidecar.launch as launch

    for m in (c, sc, launch):
        importlib.reload(m)

    import cornserve_tasklib  # noqa: F401
    from cornserve.services.gateway.router import create_app
    from cornserve.services.process import free_port
    from cornserve.services.resource_manager.grpc import start_server as start_rm
    from cornserve.services.resource_manager.manager import ResourceManager
    from cornserve.services.store import LocalStore
    from cornserve.services.task_dispatcher.app import create_app as create_td_app, start_grpc as start_td_grpc
    from cornserve.services.task_dispatcher.dispatcher import TaskDispatcher
    from cornserve.services.task_registry.registry import TaskRegistry

    async def serve(app, port):
        server = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="warning"))
        task = asyncio.create_task(server.serve())
        while not server.started:
            await asyncio.sleep(0.02)
        return server, task

    async def run():
        store = LocalStore(str(tmp_path / "store.sqlite"))
        registry = TaskRegistry(store)
        dispatcher = TaskDispatcher(registry)
        td_grpc_addr = f"127.0.0.1:{free_port()}"
        td_grpc = await start_td_grpc(dispatcher, td_grpc_addr)
        td_port = free_port()
        td_server, td_task = await serve(create_td_app(dispatcher), td_port)
        rm = await ResourceManager.init(num_gpus=num_gpus, sidecar_slab_bytes=16 << 20, sidecar_device="cpu" if device == "cpu" else None, registry=registry,
                                        dispatcher_urls=[td_grpc_addr], tm_manager_kwargs={"health_timeout_s": 240})
        rm_addr = f"127.0.0.1:{free_port()}"
        rm_server = await start_rm(rm, rm_addr)
        gw_port = free_port()
        gw_server, gw_task = await serve(create_app(rm_addr, f"http://127.0.0.1:{td_port}", [td_grpc_addr], registry), gw_port)
        url = f"http://127.0.0.1:{gw_port}"
        try:
            async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=500)) as http:
                async with http.post(f"{url}/app/register", json={"source_code": app_source}) as resp:
                    events = [json.loads(l.decode()[6:]) async for l in resp.content if l.startswith(b"data: ")]
                assert events[-1]["event"]["type"] == "final", events
                app_id = events[0]["event"]["app_id"]

                async def ask(i):
                    data = request_of(i) if request_of else {"prompt": f"describe picture {i}", "image_url": f"synthetic:224x224:{i}"}
                    req = {"request_data": data}
                    async with http.post(f"{url}/app/invoke/{app_id}", json=req) as resp:
                        assert resp.status == 200, await resp.text()
                        chunks = [json.loads(l) async for l in resp.content if l.strip()]
                    assert all("error" not in ch for ch in chunks), chunks
                    return collect(chunks)

                texts = await asyncio.gather(*(ask(i) for i in range(4)))
                if device == "cpu":
                    assert await ask(1) == texts[1]  # deterministic, whatever the batch it ran in
                else:
                    alone = await ask(1)
                    assert alone == await ask(1)  # bf16 kernels pick tile shapes by batch size: compare like with like
                    texts = [*texts, alone]
                assert (await http.post(f"{url}/app/unregister/{app_id}")).status == 200
            return texts
        finally:
            gw_server.should_exit = True
            td_server.should_exit = True
            await asyncio.gather(gw_task, td_task, return_exceptions=True)
            await rm_server.stop(0.5)
            await td_grpc.stop(0.5)
            await rm.shutdown()
            await dispatcher.shutdown()
            await registry.shutdown()
            store.close()

    return asyncio.run(run())
