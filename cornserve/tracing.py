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
