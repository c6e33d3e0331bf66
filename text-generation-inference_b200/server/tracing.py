"""Span tracing of the shard: W3C trace context in, OTLP/HTTP JSON (or log lines) out.

Role of ``server/text_generation_server/tracing.py:16-63`` in the reference (OTLP span exporter, a
gRPC server interceptor that continues the caller's trace, spans around ``generate_token`` /
``filter`` / ``concatenate``).  The OpenTelemetry SDK is not a dependency here: a span is a small
record, the exporter is a background thread that posts batches in the OTLP/HTTP JSON encoding
(``/v1/traces``), and without an endpoint finished spans are written to the log at DEBUG level.

    setup_tracing("tgi.server", "http://collector:4318")
    with tracer().span("generate_token", attributes={"batch": 3}):
        ...
"""
from __future__ import annotations

import contextvars
import functools
import json
import logging
import os
import queue
import secrets
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import grpc

log = logging.getLogger("tgi_b200.tracing")

_current: contextvars.ContextVar = contextvars.ContextVar("tgi_b200_span", default=None)


@dataclass
class SpanContext:
    trace_id: str            # 32 hex digits
    span_id: str             # 16 hex digits
    sampled: bool = True

    def traceparent(self) -> str:
        return f"00-{self.trace_id}-{self.span_id}-{'01' if self.sampled else '00'}"


def parse_traceparent(value: Optional[str]) -> Optional[SpanContext]:
    """``00-<32 hex>-<16 hex>-<2 hex>`` -> context, or ``None`` when malformed / all-zero."""
    if not value:
        return None
    parts = value.strip().split("-")
    if len(parts) != 4 or len(parts[1]) != 32 or len(parts[2]) != 16 or len(parts[3]) != 2:
        return None
    try:
        int(parts[1], 16), int(parts[2], 16)
        flags = int(parts[3], 16)
    except ValueError:
        return None
    if parts[0] == "ff" or set(parts[1]) == {"0"} or set(parts[2]) == {"0"}:
        return None
    return SpanContext(parts[1].lower(), parts[2].lower(), bool(flags & 1))


@dataclass
class Span:
    name: str
    context: SpanContext
    parent_id: Optional[str]
    start_ns: int
    end_ns: int = 0
    attributes: Dict[str, Any] = field(default_factory=dict)
    error: Optional[str] = None

    def set_attribute(self, key: str, value: Any) -> None:
        self.attributes[key] = value


def _otlp_value(v: Any) -> Dict[str, Any]:
    if isinstance(v, bool):
        return {"boolValue": v}
    if isinstance(v, int):
        return {"intValue": str(v)}
    if isinstance(v, float):
        return {"doubleValue": v}
    return {"stringValue": str(v)}


def encode_otlp(spans: List[Span], service_name: str) -> Dict[str, Any]:
    """OTLP/HTTP JSON body (``ExportTraceServiceRequest``) for a batch of finished spans."""
    return {"resourceSpans": [{
        "resource": {"attributes": [{"key": "service.name", "value": {"stringValue": service_name}}]},
        "scopeSpans": [{"scope": {"name": "tgi_b200"}, "spans": [{
            "traceId": s.context.trace_id, "spanId": s.context.span_id,
            **({"parentSpanId": s.parent_id} if s.parent_id else {}),
            "name": s.name, "kind": 2, "startTimeUnixNano": str(s.start_ns), "endTimeUnixNano": str(s.end_ns),
            "attributes": [{"key": k, "value": _otlp_value(v)} for k, v in s.attributes.items()],
            "status": {"code": 2, "message": s.error} if s.error else {"code": 1},
        } for s in spans]}],
    }]}


class Tracer:
    def __init__(self, service_name: str = "tgi_b200.server", endpoint: Optional[str] = None,
                 flush_interval_s: float = 2.0, max_batch: int = 256):
        self.service_name = service_name
        self.endpoint = endpoint.rstrip("/") + "/v1/traces" if endpoint else None
        self.finished: "queue.Queue[Span]" = queue.Queue(maxsize=8192)
        self.flush_interval_s, self.max_batch = flush_interval_s, max_batch
        self.exported = 0
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        if self.endpoint:
            self._thread = threading.Thread(target=self._export_loop, name="otlp-export", daemon=True)
            self._thread.start()

    # ---- span life cycle -----------------------------------------------------------------------
    def start_span(self, name: str, parent: Optional[SpanContext] = None, attributes: Optional[Dict] = None) -> Span:
        if parent is None:
            cur = _current.get()
            parent = cur.context if cur is not None else None
        trace_id = parent.trace_id if parent else secrets.token_hex(16)
        ctx = SpanContext(trace_id, secrets.token_hex(8), parent.sampled if parent else True)
        return Span(name, ctx, parent.span_id if parent else None, time.time_ns(), attributes=dict(attributes or {}))

    def end_span(self, span: Span) -> None:
        span.end_ns = time.time_ns()
        if not span.context.sampled:
            return
        if self.endpoint is None:
            log.debug("span %s trace=%s span=%s parent=%s %.3f ms %s", span.name, span.context.trace_id,
                      span.context.span_id, span.parent_id, (span.end_ns - span.start_ns) / 1e6, span.attributes)
            return
        try:
            self.finished.put_nowait(span)
        except queue.Full:      # never block the serving loop on telemetry
            pass

    def span(self, name: str, parent: Optional[SpanContext] = None, attributes: Optional[Dict] = None):
        return _SpanScope(self, name, parent, attributes)

    # ---- export --------------------------------------------------------------------------------
    def _drain(self) -> List[Span]:
        out: List[Span] = []
        while len(out) < self.max_batch:
            try:
                out.append(self.finished.get_nowait())
            except queue.Empty:
                break
        return out

    def flush(self) -> int:
        batch = self._drain()
        if not batch or self.endpoint is None:
            return 0
        try:
            import requests

            requests.post(self.endpoint, data=json.dumps(encode_otlp(batch, self.service_name)),
                          headers={"content-type": "application/json"}, timeout=5)
            self.exported += len(batch)
        except Exception as err:  # noqa: BLE001 - telemetry must never take the shard down
            log.debug("OTLP export failed: %s", err)
        return len(batch)

    def _export_loop(self):
        while not self._stop.wait(self.flush_interval_s):
            while self.flush():
                pass
        self.flush()

    def shutdown(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=10)


class _SpanScope:
    def __init__(self, tracer: Tracer, name, parent, attributes):
        self.tracer, self.name, self.parent, self.attributes = tracer, name, parent, attributes
        self.span: Optional[Span] = None
        self._token = None

    def __enter__(self) -> Span:
        self.span = self.tracer.start_span(self.name, self.parent, self.attributes)
        self._token = _current.set(self.span)
        return self.span

    def __exit__(self, exc_type, exc, tb):
        if exc is not None:
            self.span.error = f"{exc_type.__name__}: {exc}"
        _current.reset(self._token)
        self.tracer.end_span(self.span)
        return False


_TRACER = Tracer()


def tracer() -> Tracer:
    return _TRACER


def setup_tracing(service_name: str, endpoint: Optional[str]) -> Tracer:
    """Install the process-wide tracer; ``endpoint`` is the collector's OTLP/HTTP base URL."""
    global _TRACER
    _TRACER.shutdown()
    _TRACER = Tracer(service_name or os.environ.get("OTEL_SERVICE_NAME", "tgi_b200.server"), endpoint)
    return _TRACER


def traced(name: Optional[str] = None):
    """Decorator: run the function inside a span named ``name`` (default: the function's name)."""

    def wrap(fn):
        label = name or fn.__qualname__

        @functools.wraps(fn)
        def inner(*args, **kwargs):
            with _TRACER.span(label):
                return fn(*args, **kwargs)

        return inner

    return wrap


class TracingInterceptor(grpc.aio.ServerInterceptor):
    """Continues the caller's trace: reads ``traceparent`` from the call metadata and runs the handler
    inside a server span named after the method."""

    async def intercept_service(self, continuation, handler_call_details):
        handler = await continuation(handler_call_details)
        if handler is None or handler.unary_unary is None:
            return handler
        meta = dict(handler_call_details.invocation_metadata or ())
        parent = parse_traceparent(meta.get("traceparent"))
        method = handler_call_details.method
        inner = handler.unary_unary

        async def with_span(request, context):
            with _TRACER.span(method, parent=parent, attributes={"rpc.system": "grpc", "rpc.method": method}):
                return await inner(request, context)

        return grpc.unary_unary_rpc_method_handler(
            with_span, request_deserializer=handler.request_deserializer,
            response_serializer=handler.response_serializer)
