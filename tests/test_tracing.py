"""Trace context crosses every transport on its own: an HTTP client span parents the server span of the FastAPI app it
calls, and a gRPC client span parents the server span of the RPC, without any hand-written inject / extract."""

import asyncio
import socket

import pytest


def _port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return int(s.getsockname()[1])


@pytest.fixture()
def spans(monkeypatch):
    from opentelemetry import trace
    from opentelemetry.sdk.trace import TracerProvider
    from opentelemetry.sdk.trace.export import SimpleSpanProcessor
    from opentelemetry.sdk.trace.export.in_memory_span_exporter import InMemorySpanExporter

    monkeypatch.setenv("OTEL_SDK_DISABLED", "false")
    exporter = InMemorySpanExporter()
    provider = TracerProvider()
    provider.add_span_processor(SimpleSpanProcessor(exporter))
    # the global provider can be set once per process: install ours unless a test before did, then attach to that one
    current = trace.get_tracer_provider()
    if isinstance(current, TracerProvider):
        current.add_span_processor(SimpleSpanProcessor(exporter))
    else:
        trace.set_tracer_provider(provider)
    yield exporter
    exporter.clear()


def test_http_hops_carry_the_trace(spans):
    import aiohttp
    import uvicorn
    from fastapi import FastAPI

    from cornserve.tracing import aiohttp_trace_configs, get_tracer, instrument_fastapi

    app = FastAPI()
    instrument_fastapi(app, "test")

    @app.get("/ping/{x}")
    async def ping(x: int):
        return {"x": x}

    async def run():
        port = _port()
        server = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="warning"))
        task = asyncio.create_task(server.serve())
        while not server.started:
            await asyncio.sleep(0.02)
        with get_tracer("test").start_as_current_span("caller"):
            async with aiohttp.ClientSession(trace_configs=aiohttp_trace_configs()) as http:
                async with http.get(f"http://127.0.0.1:{port}/ping/3") as r:
                    assert (await r.json()) == {"x": 3}
        server.should_exit = True
        await task

    asyncio.run(run())
    by_name = {s.name: s for s in spans.get_finished_spans()}
    caller, client, server = by_name["caller"], by_name["GET /ping/3"], None
    for s in spans.get_finished_spans():
        if s.name == "GET /ping/3" and s.kind.name == "SERVER":
            server = s
        if s.name == "GET /ping/3" and s.kind.name == "CLIENT":
            client = s
    assert server is not None and client.kind.name == "CLIENT"
    assert client.parent.span_id == caller.context.span_id
    assert server.parent.span_id == client.context.span_id and server.context.trace_id == caller.context.trace_id
    assert server.attributes["http.status_code"] == 200


def test_grpc_hops_carry_the_trace(spans):
    import grpc

    from cornserve.services.pb import common_pb2, task_dispatcher_pb2_grpc
    from cornserve.tracing import get_tracer, grpc_client_interceptors, grpc_server_interceptors

    class Servicer(task_dispatcher_pb2_grpc.TaskDispatcherServicer):
        async def SyncTaskRegistry(self, request, context):
            return common_pb2.SyncTaskRegistryResponse(status=common_pb2.STATUS_OK)

    async def run():
        server = grpc.aio.server(interceptors=grpc_server_interceptors())
        task_dispatcher_pb2_grpc.add_TaskDispatcherServicer_to_server(Servicer(), server)
        port = server.add_insecure_port("127.0.0.1:0")
        await server.start()
        with get_tracer("test").start_as_current_span("rpc-caller"):
            async with grpc.aio.insecure_channel(f"127.0.0.1:{port}", interceptors=grpc_client_interceptors()) as ch:
                resp = await task_dispatcher_pb2_grpc.TaskDispatcherStub(ch).SyncTaskRegistry(common_pb2.SyncTaskRegistryRequest())
                assert resp.status == common_pb2.STATUS_OK
        await server.stop(0.2)

    asyncio.run(run())
    done = spans.get_finished_spans()
    caller = next(s for s in done if s.name == "rpc-caller")
    client = next(s for s in done if s.kind.name == "CLIENT" and "SyncTaskRegistry" in s.name)
    server = next(s for s in done if s.kind.name == "SERVER" and "SyncTaskRegistry" in s.name)
    assert client.parent.span_id == caller.context.span_id
    assert server.parent.span_id == client.context.span_id and server.context.trace_id == caller.context.trace_id
