"""Shard gRPC server: ``generate.v3.TextGenerationService`` over a unix domain socket.

Reference: ``server/text_generation_server/server.py`` (servicer ``:56-226``, ``serve`` ``:229-325``).
The service is registered through grpcio's generic handlers with the run-time protobuf classes of
``proto/generate_v3.py`` (no generated stubs).  Every shard receives the same RPCs; each answers
only with the generations of the requests it owns (``request.id % world_size == rank``).
"""
from __future__ import annotations

import asyncio
import logging
import os
import signal
import time
from pathlib import Path
from typing import List, Optional

import grpc
import torch

from ..proto import generate_v3 as pb
from .cache import Cache
from .interceptor import ExceptionInterceptor
from .tracing import TracingInterceptor, tracer

log = logging.getLogger("tgi_b200.server")


class SignalHandler:
    KEEP_PROCESSING = True

    def __init__(self):
        signal.signal(signal.SIGINT, self.exit_gracefully)
        signal.signal(signal.SIGTERM, self.exit_gracefully)

    def set_keep_processing(self, value: bool):
        self.KEEP_PROCESSING = value

    def exit_gracefully(self, signum, frame):
        log.info("Exiting gracefully: signal %s", signum)
        self.set_keep_processing(False)


class TextGenerationService:
    """The eight RPCs; methods are ``async`` and run on the server's event loop."""

    def __init__(self, model, cache: Cache, server_urls: List[str]):
        self.model = model
        self.cache = cache
        self.server_urls = server_urls
        if model.device.type == "cuda":
            torch.cuda.set_device(model.device)

    def _check_kernels(self):
        if self.model.device.type == "cuda":
            from ..ops import cuda as K

            code = K.check_status(self.model.device)
            if code != 0:
                raise RuntimeError(f"a device-side wait timed out (status {code}); the step's results are invalid")

    async def Info(self, request, context):
        return self.model.info

    async def Health(self, request, context):
        if self.model.device.type == "cuda":
            torch.zeros((2, 2), device=self.model.device)
        return pb.HealthResponse()

    async def ServiceDiscovery(self, request, context):
        return pb.ServiceDiscoveryResponse(urls=self.server_urls)

    async def ClearCache(self, request, context):
        if request.HasField("id"):
            self.cache.delete(request.id)
        else:
            self.cache.clear()
        return pb.ClearCacheResponse()

    async def FilterBatch(self, request, context):
        batch = self.cache.pop(request.batch_id)
        if batch is None:
            raise ValueError(f"Batch ID {request.batch_id} not found in cache.")
        with tracer().span("filter"):
            filtered = batch.filter(list(request.request_ids))
        self.cache.set(filtered)
        return pb.FilterBatchResponse(batch=filtered.to_pb())

    async def Warmup(self, request, context):
        batch = self.model.batch_type.from_pb(request.batch, self.model.tokenizer, self.model.dtype,
                                              self.model.device)
        batch.max_prefill_tokens = request.max_prefill_tokens or None
        self.model.max_prefill_tokens = request.max_prefill_tokens or None
        max_input = request.max_input_tokens if request.HasField("max_input_tokens") else None
        max_total = request.max_total_tokens if request.HasField("max_total_tokens") else None
        supported, max_input, max_total = self.model.warmup(batch, max_input, max_total)
        self._check_kernels()
        resp = pb.WarmupResponse(max_input_tokens=int(max_input), max_total_tokens=int(max_total))
        if supported is not None:
            resp.max_supported_total_tokens = int(supported)
        return resp

    async def Prefill(self, request, context):
        start = time.time_ns()
        batch = self.model.batch_type.from_pb(request.batch, self.model.tokenizer, self.model.dtype,
                                              self.model.device, getattr(self.model, "speculate", 0))
        concat_ns = None
        if self.model.support_chunking and request.HasField("cached_batch"):
            cached = self.cache.pop(request.cached_batch.id)
            if cached is None:
                raise ValueError(f"Batch ID {request.cached_batch.id} not found in cache.")
            t = time.time_ns()
            with tracer().span("concatenate"):
                batch = self.model.batch_type.concatenate([cached, batch])
            concat_ns = time.time_ns() - t
        with tracer().span("generate_token", attributes={"batch_size": len(batch)}):
            generations, next_batch, timings = self.model.generate_token(batch)
        self._check_kernels()
        self.cache.set(next_batch)
        resp = pb.PrefillResponse(generations=[g.to_pb() for g in generations], forward_ns=timings[0],
                                  decode_ns=timings[1], total_ns=time.time_ns() - start)
        if next_batch is not None:
            resp.batch.CopyFrom(next_batch.to_pb())
        if concat_ns is not None:
            resp.concat_ns = concat_ns
        return resp

    async def Decode(self, request, context):
        start = time.time_ns()
        if len(request.batches) == 0:
            raise ValueError("Must provide at least one batch")
        batches = []
        for b in request.batches:
            batch = self.cache.pop(b.id)
            if batch is None:
                raise ValueError(f"Batch ID {b.id} not found in cache.")
            batches.append(batch)
        if len(batches) == 0:
            raise ValueError("All batches are empty")
        concat_ns = None
        if len(batches) > 1:
            t = time.time_ns()
            with tracer().span("concatenate"):
                batch = self.model.batch_type.concatenate(batches)
            concat_ns = time.time_ns() - t
        else:
            batch = batches[0]
        with tracer().span("generate_token", attributes={"batch_size": len(batch)}):
            generations, next_batch, timings = self.model.generate_token(batch)
        self._check_kernels()
        self.cache.set(next_batch)
        resp = pb.DecodeResponse(generations=[g.to_pb() for g in generations], forward_ns=timings[0],
                                 decode_ns=timings[1], total_ns=time.time_ns() - start)
        if next_batch is not None:
            resp.batch.CopyFrom(next_batch.to_pb())
        if concat_ns is not None:
            resp.concat_ns = concat_ns
        return resp


FRAMED_METHODS = ["Info", "ServiceDiscovery", "ClearCache", "FilterBatch", "Warmup", "Prefill", "Decode", "Health"]


async def serve_framed(service: TextGenerationService, path: str, shutdown_callback=None):
    """Second transport for the same service: length-prefixed protobuf frames over a unix socket.

    The C++ router has no HTTP/2 stack, so it speaks this framing instead of gRPC; the messages are
    the same ``generate.v3`` protobufs.  Request frame: ``u8 method index (FRAMED_METHODS), u32 LE
    length, payload``; when bit 7 of the method byte is set, the 55 characters of a W3C ``traceparent``
    precede the payload (not counted in the length) and the handler runs in a span that continues the
    caller's trace, as the gRPC transport does from call metadata.  Response frame: ``u8 status (0 ok /
    1 error), u32 LE length, payload`` where the payload of an error is its UTF-8 message.

    A ``RuntimeError`` of a handler (a CUDA error, a device-side wait that ran out) is fatal for the
    shard as on the gRPC transport (``server/text_generation_server/interceptor.py:11-40`` in the
    reference): the error frame is sent, then ``shutdown_callback`` ends the serve loop so that the
    launcher tears the deployment down instead of letting one rank go on with stale flag epochs.
    """
    import struct

    from .tracing import parse_traceparent

    async def handle(reader: asyncio.StreamReader, writer: asyncio.StreamWriter):
        try:
            while True:
                try:
                    head = await reader.readexactly(5)
                except asyncio.IncompleteReadError:
                    break
                method, length = head[0], struct.unpack("<I", head[1:5])[0]
                parent = None
                if method & 0x80:
                    method &= 0x7F
                    parent = parse_traceparent((await reader.readexactly(55)).decode("ascii", "replace"))
                payload = await reader.readexactly(length) if length else b""
                fatal = False
                try:
                    name = FRAMED_METHODS[method]
                    req_cls = pb.message_class(pb.METHODS[name][0])
                    if parent is not None:
                        with tracer().span(name, parent=parent, attributes={"rpc.system": "framed", "rpc.method": name}):
                            resp = await getattr(service, name)(req_cls.FromString(payload), None)
                    else:
                        resp = await getattr(service, name)(req_cls.FromString(payload), None)
                    body, status = resp.SerializeToString(), 0
                except Exception as err:  # noqa: BLE001
                    log.exception("framed rpc %s failed", method)
                    fatal = isinstance(err, RuntimeError)
                    if torch.cuda.is_available():
                        torch.cuda.empty_cache()
                    body, status = f"{type(err).__name__}: {err}".encode(), 1
                writer.write(bytes([status]) + struct.pack("<I", len(body)) + body)
                await writer.drain()
                if fatal and shutdown_callback is not None:
                    shutdown_callback()
                    break
        finally:
            writer.close()

    if os.path.exists(path):
        os.unlink(path)
    return await asyncio.start_unix_server(handle, path=path)


def generic_handler(service: TextGenerationService) -> grpc.GenericRpcHandler:
    handlers = {}
    for rpc, (req, resp) in pb.METHODS.items():
        handlers[rpc] = grpc.unary_unary_rpc_method_handler(
            getattr(service, rpc),
            request_deserializer=pb.message_class(req).FromString,
            response_serializer=lambda m: m.SerializeToString(),
        )
    return grpc.method_handlers_generic_handler(f"{pb.PACKAGE}.{pb.SERVICE}", handlers)


def serve(model_id: str, lora_adapters=None, revision: Optional[str] = None, sharded: bool = False,
          quantize: Optional[str] = None, speculate: Optional[int] = None, dtype: Optional[str] = None,
          kv_cache_dtype: Optional[str] = None, trust_remote_code: bool = False,
          uds_path: Path = Path("/tmp/text-generation-server"), max_input_tokens: Optional[int] = None,
          model_factory=None):
    """Load the shard's model and serve until SIGINT/SIGTERM."""

    async def serve_inner():
        signal_handler = SignalHandler()
        world = int(os.environ.get("WORLD_SIZE", "1"))
        rank = int(os.environ.get("RANK", "0"))
        unix_socket_template = "unix://{}-{}"
        if sharded:
            server_urls = [unix_socket_template.format(uds_path, r) for r in range(world)]
            local_url = server_urls[rank]
        else:
            local_url = unix_socket_template.format(uds_path, 0)
            server_urls = [local_url]
        if model_factory is not None:
            model = model_factory()
        else:
            from ..models import get_model_with_lora_adapters

            model = get_model_with_lora_adapters(
                model_id, lora_adapters, revision=revision, sharded=sharded, quantize=quantize, speculate=speculate,
                dtype=dtype, kv_cache_dtype=kv_cache_dtype, trust_remote_code=trust_remote_code,
                max_input_tokens=max_input_tokens)
        server = grpc.aio.server(
            interceptors=[ExceptionInterceptor(lambda: signal_handler.set_keep_processing(False)), TracingInterceptor()],
            options=[("grpc.max_receive_message_length", (1 << 31) - 1),
                     ("grpc.max_send_message_length", (1 << 31) - 1)],
        )
        service = TextGenerationService(model, Cache(), server_urls)
        server.add_generic_rpc_handlers((generic_handler(service),))
        server.add_insecure_port(local_url)
        await server.start()
        framed = await serve_framed(service, local_url[len("unix://"):] + ".raw",
                                    shutdown_callback=lambda: signal_handler.set_keep_processing(False))
        log.info("Server started at %s", local_url)
        while signal_handler.KEEP_PROCESSING:
            await asyncio.sleep(0.5)
        framed.close()
        await server.stop(grace=2)

    asyncio.run(serve_inner())
