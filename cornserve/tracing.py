"""OpenTelemetry set-up (reference: python/cornserve/tracing.py:14-21).  ``configure_otel`` installs a
tracer provider exporting to ``OTEL_EXPORTER_OTLP_ENDPOINT`` when the exporter package is present and
``OTEL_SDK_DISABLED`` is not set; otherwise the API's no-op tracer is used.  ``inject``/``extract``
carry the W3C trace context across process hops (ZMQ messages, RPC metadata)."""

from __future__ import annotations

import os
from typing import Any

from opentelemetry import propagate, trace

_configured = False


def configure_otel(service_name: str) -> None:
    global _configured
    if _configured or os.environ.get("OTEL_SDK_DISABLED", "").lower() == "true":
        return
    endpoint = os.environ.get("OTEL_EXPORTER_OTLP_ENDPOINT")
    if not endpoint:
        return
    try:
        from opentelemetry.exporter.otlp.proto.grpc.trace_exporter import OTLPSpanExporter
        from opentelemetry.sdk.resources import Resource
        from opentelemetry.sdk.trace import TracerProvider
        from opentelemetry.sdk.trace.export import BatchSpanProcessor
    except Exception:
        return
    provider = TracerProvider(resource=Resource.create({"service.name": service_name}))
    provider.add_span_processor(BatchSpanProcessor(OTLPSpanExporter(endpoint=endpoint)))
    trace.set_tracer_provider(provider)
    _configured = True


def get_tracer(name: str):
    return trace.get_tracer(name)


def inject() -> dict[str, str]:
    """Current trace context as a W3C carrier dict."""
    carrier: dict[str, str] = {}
    propagate.inject(carrier)
    return carrier


def extract(carrier: dict[str, str] | None) -> Any:
    return propagate.extract(carrier or {})


# ----------------------------------------------------------------------------------------------------------------------
# Automatic instrumentation of the transports (reference: FastAPIInstrumentor / AioHttpClientInstrumentor /
# GrpcAio{Client,Server}Instrumentor calls in python/cornserve/services/gateway/entrypoint.py:11-44,
# task_dispatcher/entrypoint.py:39-45, services/sidecar/server.py:450-453).  The opentelemetry-instrumentation-*
# packages are used when they are installed; otherwise the equivalents below do the same job with the API alone: one
# server span per HTTP request / RPC whose parent is the caller's span (W3C ``traceparent``), one client span per
# outgoing HTTP request / RPC that carries the context in its headers / metadata.  With the SDK disabled all of it is
# a few no-op calls.
# ----------------------------------------------------------------------------------------------------------------------
def _enabled() -> bool:
    return os.environ.get("OTEL_SDK_DISABLED", "").lower() != "true"


def instrument_fastapi(app, service_name: str = "") -> None:
    """Server spans ``"<METHOD> <path>"`` for every HTTP request of a FastAPI / Starlette app."""
    if getattr(app.state, "_cornserve_traced", False):
        return
    app.state._cornserve_traced = True
    try:
        from opentelemetry.instrumentation.fastapi import FastAPIInstrumentor

        FastAPIInstrumentor.instrument_app(app)
        return
    except Exception:  # noqa: BLE001  (package not installed)
        pass
    tracer = trace.get_tracer(service_name or "cornserve.http")

    class _Trace:
        def __init__(self, inner):
            self.inner = inner

        async def __call__(self, scope, receive, send):
            if scope["type"] != "http" or not _enabled():
                await self.inner(scope, receive, send)
                return
            headers = {k.decode("latin-1"): v.decode("latin-1") for k, v in scope.get("headers", [])}
            ctx = propagate.extract(headers)
            with tracer.start_as_current_span(f"{scope['method']} {scope['path']}", context=ctx,
                                              kind=trace.SpanKind.SERVER) as span:
                span.set_attribute("http.method", scope["method"])
                span.set_attribute("http.target", scope["path"])

                async def traced_send(message):
                    if message["type"] == "http.response.start":
                        span.set_attribute("http.status_code", int(message["status"]))
                    await send(message)

                await self.inner(scope, receive, traced_send)

    app.add_middleware(_Trace)


def aiohttp_trace_configs() -> list:
    """``trace_configs=`` for ``aiohttp.ClientSession``: a client span per request, context injected into the headers."""
    import aiohttp

    tracer = trace.get_tracer("cornserve.http.client")
    cfg = aiohttp.TraceConfig()

    async def on_start(session, ctx, params):
        if not _enabled():
            return
        span = tracer.start_span(f"{params.method} {params.url.path}", kind=trace.SpanKind.CLIENT)
        span.set_attribute("http.method", params.method)
        span.set_attribute("http.url", str(params.url))
        ctx.span = span
        carrier: dict[str, str] = {}
        propagate.inject(carrier, context=trace.set_span_in_context(span))
        for k, v in carrier.items():
            params.headers[k] = v

    async def on_end(session, ctx, params):
        span = getattr(ctx, "span", None)
        if span is not None:
            span.set_attribute("http.status_code", params.response.status)
            span.end()

    async def on_exception(session, ctx, params):
        span = getattr(ctx, "span", None)
        if span is not None:
            span.record_exception(params.exception)
            span.end()

    cfg.on_request_start.append(on_start)
    cfg.on_request_end.append(on_end)
    cfg.on_request_exception.append(on_exception)
    return [cfg]


def grpc_client_interceptors() -> list:
    """Interceptors for ``grpc.aio.insecure_channel``: a client span per unary RPC, context sent as metadata."""
    import grpc

    tracer = trace.get_tracer("cornserve.grpc.client")

    class _Client(grpc.aio.UnaryUnaryClientInterceptor):
        async def intercept_unary_unary(self, continuation, details, request):
            if not _enabled():
                return await continuation(details, request)
            method = details.method.decode() if isinstance(details.method, bytes) else details.method
            with tracer.start_as_current_span(method.lstrip("/"), kind=trace.SpanKind.CLIENT) as span:
                span.set_attribute("rpc.system", "grpc")
                carrier: dict[str, str] = {}
                propagate.inject(carrier)
                md = list(details.metadata or []) + list(carrier.items())
                new = grpc.aio.ClientCallDetails(details.method, details.timeout, grpc.aio.Metadata(*md), details.credentials,
                                                 details.wait_for_ready)
                return await continuation(new, request)

    return [_Client()]


def grpc_server_interceptors() -> list:
    """Interceptors for ``grpc.aio.server``: a server span per unary RPC, parented by the caller's metadata."""
    import grpc

    tracer = trace.get_tracer("cornserve.grpc.server")

    class _Server(grpc.aio.ServerInterceptor):
        async def intercept_service(self, continuation, details):
            handler = await continuation(details)
            if handler is None or not _enabled() or handler.unary_unary is None:
                return handler
            inner = handler.unary_unary
            carrier = {k: v for k, v in (details.invocation_metadata or []) if isinstance(v, str)}
            method = details.method.lstrip("/")

            async def traced(request, context):
                with tracer.start_as_current_span(method, context=propagate.extract(carrier), kind=trace.SpanKind.SERVER) as span:
                    span.set_attribute("rpc.system", "grpc")
                    return await inner(request, context)

            return grpc.unary_unary_rpc_method_handler(traced, request_deserializer=handler.request_deserializer,
                                                       response_serializer=handler.response_serializer)

    return [_Server()]
