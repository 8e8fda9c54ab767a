"""Control plane end to end in one process: gateway (HTTP) -> task dispatcher (HTTP + gRPC) -> resource
manager (gRPC) -> task managers (gRPC) -> fake executors (HTTP).  Nothing here needs a GPU; executors
are tiny aiohttp apps started through the task managers' spawn hook."""

import asyncio
import json
import os

import aiohttp
import pytest
import uvicorn
from aiohttp import web

import cornserve_tasklib  # noqa: F401
from cornserve.services.process import free_port
from cornserve.services.resource import CannotColocateError, NotEnoughGPUsError, Resource
from cornserve.services.resource_manager.grpc import start_server as start_rm
from cornserve.services.resource_manager.manager import ResourceManager
from cornserve.services.store import LocalStore
from cornserve.services.task_dispatcher.app import create_app as create_td_app
from cornserve.services.task_dispatcher.app import start_grpc as start_td_grpc
from cornserve.services.task_dispatcher.dispatcher import TaskDispatcher
from cornserve.services.task_manager.manager import plan_executors
from cornserve.services.task_registry.registry import TaskRegistry

APP_SOURCE = '''
from collections.abc import AsyncIterator
from cornserve.app.base import AppConfig, AppRequest, AppResponse
from cornserve_tasklib import MLLMTask, Modality, OpenAIChatCompletionRequest, OpenAIChatCompletionChunk

class Request(AppRequest):
    prompt: str
    image_urls: list[str] = []

mllm = MLLMTask(model_id="tiny/vlm", modalities=[Modality.IMAGE])

class Config(AppConfig):
    tasks = {"mllm": mllm}

async def serve(request: Request) -> AsyncIterator[OpenAIChatCompletionChunk]:
    content = [{"type": "text", "text": request.prompt}]
    content += [{"type": "image_url", "image_url": {"url": u}} for u in request.image_urls]
    req = OpenAIChatCompletionRequest(model="tiny/vlm", messages=[{"role": "user", "content": content}])
    return await mllm(req)
'''


class FakeExecutors:
    """Spawn hook for task managers: every "executor" is an aiohttp app in this process."""

    def __init__(self):
        self.runners = {}
        self.requests = []
        self.fail_health = set()

    async def spawn(self, executor_id, gpus, port, launch_args):
        app = web.Application()

        async def health(_):
            return web.Response(status=503 if executor_id in self.fail_health else 200)

        async def embeddings(req):
            self.requests.append((executor_id, "embeddings", await req.json()))
            return web.json_response({"status": 0, "error_message": None})

        async def chat(req):
            body = await req.json()
            self.requests.append((executor_id, "chat", body))
            resp = web.StreamResponse(headers={"Content-Type": "text/event-stream"})
            await resp.prepare(req)
            for i, word in enumerate(["hello", " world"]):
                chunk = {"id": "c", "object": "chat.completion.chunk", "created": 0, "model": body["model"],
                         "choices": [{"index": 0, "delta": {"content": word}, "finish_reason": None if i == 0 else "stop"}]}
                await resp.write(f"data: {json.dumps(chunk)}\n\n".encode())
            await resp.write(b"data: [DONE]\n\n")
            return resp

        app.add_routes([web.get("/health", health), web.post("/embeddings", embeddings),
                        web.post("/v1/chat/completions", chat)])
        runner = web.AppRunner(app)
        await runner.setup()
        await web.TCPSite(runner, "127.0.0.1", port).start()
        self.runners[executor_id] = (runner, [g.global_rank for g in gpus], launch_args)
        return f"http://127.0.0.1:{port}", None

    async def close(self):
        for runner, _, _ in self.runners.values():
            await runner.cleanup()


async def _serve_uvicorn(app, port):
    server = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="warning", lifespan="on"))
    task = asyncio.create_task(server.serve())
    while not server.started:
        await asyncio.sleep(0.02)
    return server, task


def test_resource_allocation_policies():
    from cornserve.services.resource import GPU

    r = Resource([GPU(f"n{i // 4}", i, i % 4) for i in range(8)])
    a = r.allocate(2, "a")
    assert {g.node for g in a} == {"n0"} or {g.node for g in a} == {"n1"}
    b = r.allocate(2, "b", node_selection_policy="spread")
    assert {g.node for g in b} != {g.node for g in a}  # spread prefers the emptier node
    c = r.allocate(1, "c", node_selection_policy="pack")
    c += r.allocate(1, "c", node_selection_policy="spread")
    assert {g.node for g in c} == {"n0", "n1"}  # one free GPU left on each node
    with pytest.raises(CannotColocateError):
        r.allocate(2, "d")
    d = r.allocate(2, "d", must_colocate=False)
    assert len(d) == 2 and r.num_free() == 0
    with pytest.raises(NotEnoughGPUsError):
        r.allocate(1, "e")
    r.release(c)
    assert r.num_free() == 2 and "n0" in r.render()


def test_plan_executors_packs_largest_first():
    from cornserve.services.resource import GPU

    gpus = [GPU("n", i, i) for i in range(7)]
    groups, left = plan_executors(gpus, [1, 2, 4])
    assert [len(g) for g in groups] == [4, 2, 1] and not left
    groups, left = plan_executors(gpus[:3], [2])
    assert [len(g) for g in groups] == [2] and len(left) == 1


def test_gateway_to_executors_round_trip(tmp_path):
    async def run():
        store = LocalStore(str(tmp_path / "store.sqlite"))
        registry = TaskRegistry(store)
        fakes = FakeExecutors()
        # dispatcher
        dispatcher = TaskDispatcher(registry)
        td_grpc_addr = f"127.0.0.1:{free_port()}"
        td_grpc = await start_td_grpc(dispatcher, td_grpc_addr)
        td_port = free_port()
        td_server, td_task = await _serve_uvicorn(create_td_app(dispatcher), td_port)
        # resource manager with in-process task managers and fake executors
        rm = ResourceManager(Resource.single_node(4), registry, dispatcher_urls=[td_grpc_addr],
                             tm_manager_kwargs={"spawn_fn": fakes.spawn, "health_timeout_s": 10})
        rm_addr = f"127.0.0.1:{free_port()}"
        rm_server = await start_rm(rm, rm_addr)
        # gateway
        from cornserve.services.gateway.router import create_app

        gw_app = create_app(rm_addr, f"http://127.0.0.1:{td_port}", [td_grpc_addr], registry, resource_manager_local=rm)
        gw_port = free_port()
        gw_server, gw_task = await _serve_uvicorn(gw_app, gw_port)
        base = f"http://127.0.0.1:{gw_port}"
        try:
            async with aiohttp.ClientSession() as http:
                # register: SSE with an initial and a final event
                async with http.post(f"{base}/app/register", json={"source_code": APP_SOURCE}) as resp:
                    events = [json.loads(l[6:]) async for l in _sse(resp)]
                assert [e["event"]["type"] for e in events] == ["initial", "final"], events
                app_id = events[0]["event"]["app_id"]
                assert sorted(events[0]["event"]["task_names"]) == ["encoder-image-vlm", "llm-vlm"]
                assert len(fakes.runners) == 2 and rm.resource.num_free() == 2
                tasks = await (await http.get(f"{base}/tasks/list")).json()
                assert {t[2] for t in tasks} == {"ready"} and len(tasks) == 2
                assert (await (await http.get(f"{base}/app/list")).json())[app_id] == "ready"

                # invoke: NDJSON stream of chunks produced by the fake LLM, relayed through two hops
                req = {"request_data": {"prompt": "hi", "image_urls": ["http://img/a.png", "http://img/b.png"]}}
                async with http.post(f"{base}/app/invoke/{app_id}", json=req) as resp:
                    assert resp.status == 200, await resp.text()
                    chunks = [json.loads(l) async for l in resp.content if l.strip()]
                assert "".join(c["choices"][0]["delta"]["content"] for c in chunks) == "hello world"
                enc = [r for r in fakes.requests if r[1] == "embeddings"]
                chat = [r for r in fakes.requests if r[1] == "chat"]
                assert len(enc) == 2 and len(chat) == 1
                llm_ranks = next(r for eid, (_, r, _) in fakes.runners.items() if eid == chat[0][0])
                ids = []
                for _, _, body in enc:
                    (item,) = body["data"]
                    assert item["receiver_sidecar_ranks"] == [llm_ranks] and item["modality"] == "image"
                    ids.append(item["id"])
                parts = [p for p in chat[0][2]["messages"][0]["content"] if p["type"] == "image_url"]
                assert [p["image_url"]["url"] for p in parts] == [
                    f"data:image/uuid;data_id={ids[0]};url=http://img/a.png,",
                    f"data:image/uuid;data_id={ids[1]};url=http://img/b.png,"]
                assert chat[0][2]["stream"] is True and "cornserve_embeddings" not in chat[0][2]

                # scaling the LLM task by one GPU adds a second executor; routing alternates between them
                llm_id = next(t[1] for t in tasks if t[1].startswith("llmunittask"))
                r = await http.post(f"{base}/task/scale", json={"task_id": llm_id, "num_gpus": 1})
                assert r.status == 200, await r.text()
                assert len(fakes.runners) == 3 and rm.resource.num_free() == 1
                for _ in range(2):
                    async with http.post(f"{base}/app/invoke/{app_id}", json=req) as resp:
                        await resp.read()
                assert len({r[0] for r in fakes.requests if r[1] == "chat"}) == 2
                assert (await http.post(f"{base}/task/scale", json={"task_id": llm_id, "num_gpus": 0})).status == 400
                assert (await http.post(f"{base}/task/scale", json={"task_id": "nope", "num_gpus": 1})).status == 404

                # health: an executor that starts failing /health is reported, then replaced
                ok, _ = await rm.healthcheck()
                assert ok
                victim = chat[0][0]
                fakes.fail_health.add(victim)
                ok, statuses = await rm.healthcheck()
                assert not ok and statuses[llm_id] is False
                fakes.fail_health.clear()
                st = rm.task_managers[llm_id]
                assert await st.servicer.manager.respawn_unhealthy() == [victim]
                assert (await rm.healthcheck())[0]

                # unknown app / invalid source
                assert (await http.post(f"{base}/app/invoke/app-x", json=req)).status == 404
                async with http.post(f"{base}/app/register", json={"source_code": "x = 1"}) as resp:
                    events = [json.loads(l[6:]) async for l in _sse(resp)]
                assert events[-1]["event"]["type"] == "error"

                # unregister tears everything down and frees the GPUs
                assert (await http.post(f"{base}/app/unregister/{app_id}")).status == 200
                assert rm.resource.num_free() == 4 and not dispatcher.task_infos
                assert await registry.list_task_instances() == []
        finally:
            gw_server.should_exit = True
            td_server.should_exit = True
            await asyncio.gather(gw_task, td_task, return_exceptions=True)
            await rm_server.stop(0.5)
            await td_grpc.stop(0.5)
            await rm.shutdown()
            await dispatcher.shutdown()
            await fakes.close()
            await registry.shutdown()
            store.close()

    asyncio.run(run())


async def _sse(resp):
    async for raw in resp.content:
        line = raw.decode().strip()
        if line.startswith("data: "):
            yield line
