"""Tracing: W3C trace-context parsing, span nesting, OTLP/HTTP JSON export to a local collector."""
import json
import threading
from http.server import BaseHTTPRequestHandler, HTTPServer

from tgi_b200.server.tracing import SpanContext, Tracer, encode_otlp, parse_traceparent


def test_traceparent_parsing():
    ctx = parse_traceparent("00-4bf92f3577b34da6a3ce929d0e0e4736-00f067aa0ba902b7-01")
    assert ctx == SpanContext("4bf92f3577b34da6a3ce929d0e0e4736", "00f067aa0ba902b7", True)
    assert ctx.traceparent() == "00-4bf92f3577b34da6a3ce929d0e0e4736-00f067aa0ba902b7-01"
    assert parse_traceparent("00-4bf92f3577b34da6a3ce929d0e0e4736-00f067aa0ba902b7-00").sampled is False
    for bad in (None, "", "garbage", "00-" + "0" * 32 + "-00f067aa0ba902b7-01", "00-abc-def-01",
                "ff-4bf92f3577b34da6a3ce929d0e0e4736-00f067aa0ba902b7-01"):
        assert parse_traceparent(bad) is None


def test_nested_spans_share_the_trace_and_export_as_otlp():
    received = []

    class Collector(BaseHTTPRequestHandler):
        def do_POST(self):
            body = self.rfile.read(int(self.headers["content-length"]))
            received.append((self.path, json.loads(body)))
            self.send_response(200)
            self.end_headers()

        def log_message(self, *a):
            pass

    srv = HTTPServer(("127.0.0.1", 0), Collector)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    try:
        t = Tracer("unit-test", f"http://127.0.0.1:{srv.server_port}", flush_interval_s=60)
        parent = parse_traceparent("00-4bf92f3577b34da6a3ce929d0e0e4736-00f067aa0ba902b7-01")
        with t.span("Prefill", parent=parent, attributes={"batch_size": 3}) as outer:
            with t.span("generate_token") as inner:
                inner.set_attribute("tokens", 7)
        try:
            with t.span("boom"):
                raise ValueError("x")
        except ValueError:
            pass
        assert inner.context.trace_id == outer.context.trace_id == parent.trace_id
        assert inner.parent_id == outer.context.span_id and outer.parent_id == parent.span_id
        assert t.flush() == 3
        t.shutdown()
    finally:
        srv.shutdown()
    path, body = received[0]
    assert path == "/v1/traces"
    spans = body["resourceSpans"][0]["scopeSpans"][0]["spans"]
    assert [s["name"] for s in spans] == ["generate_token", "Prefill", "boom"]
    assert spans[2]["status"]["code"] == 2 and "ValueError" in spans[2]["status"]["message"]
    assert {"key": "tokens", "value": {"intValue": "7"}} in spans[0]["attributes"]
    assert body["resourceSpans"][0]["resource"]["attributes"][0]["value"]["stringValue"] == "unit-test"
    assert encode_otlp([], "x")["resourceSpans"][0]["scopeSpans"][0]["spans"] == []
