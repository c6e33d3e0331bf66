"""The framed unix-socket transport of the shard (the one the C++ router speaks): a handler that raises
``RuntimeError`` answers with an error frame and then ends the serve loop, other exceptions only
answer with an error frame, and a frame that carries a ``traceparent`` runs inside the caller's trace."""
import asyncio
import struct

from tgi_b200.proto import generate_v3 as pb
from tgi_b200.server import server as srv
from tgi_b200.server.tracing import tracer


class _StubService:
    def __init__(self):
        self.seen_parent = None

    async def Health(self, request, context):
        from tgi_b200.server import tracing

        cur = tracing._current.get()
        self.seen_parent = (cur.context.trace_id, cur.parent_id) if cur is not None else None
        return pb.HealthResponse()

    async def Prefill(self, request, context):
        raise RuntimeError("kernel status 5: a device-side wait ran out")

    async def Decode(self, request, context):
        raise ValueError("Batch ID 7 not found in cache.")


async def _call(reader, writer, method, payload=b"", traceparent=None):
    m = srv.FRAMED_METHODS.index(method)
    head = bytes([m | (0x80 if traceparent else 0)]) + struct.pack("<I", len(payload))
    writer.write(head + (traceparent.encode() if traceparent else b"") + payload)
    await writer.drain()
    rh = await reader.readexactly(5)
    n = struct.unpack("<I", rh[1:5])[0]
    return rh[0], (await reader.readexactly(n)) if n else b""


def test_runtime_error_sends_the_error_frame_then_stops_the_shard(tmp_path):
    async def run():
        stopped = asyncio.Event()
        service = _StubService()
        path = str(tmp_path / "shard-0.raw")
        server = await srv.serve_framed(service, path, shutdown_callback=stopped.set)
        reader, writer = await asyncio.open_unix_connection(path)
        # a non-fatal error keeps the connection and the shard alive
        status, body = await _call(reader, writer, "Decode", pb.DecodeRequest().SerializeToString())
        assert status == 1 and b"not found" in body and not stopped.is_set()
        # trace context in the frame header
        tp = "00-4bf92f3577b34da6a3ce929d0e0e4736-00f067aa0ba902b7-01"
        status, _ = await _call(reader, writer, "Health", b"", traceparent=tp)
        assert status == 0
        assert service.seen_parent == ("4bf92f3577b34da6a3ce929d0e0e4736", "00f067aa0ba902b7")
        status, _ = await _call(reader, writer, "Health")
        assert status == 0 and service.seen_parent is None
        # a RuntimeError is fatal: error frame first, then the shutdown callback
        status, body = await _call(reader, writer, "Prefill", pb.PrefillRequest().SerializeToString())
        assert status == 1 and b"device-side wait ran out" in body
        await asyncio.wait_for(stopped.wait(), timeout=5)
        assert (await reader.read(1)) == b""       # the shard closed the connection
        writer.close()
        server.close()
        await server.wait_closed()

    assert tracer() is not None
    asyncio.run(run())
