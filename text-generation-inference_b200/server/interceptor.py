"""Turns exceptions of RPC handlers into gRPC INTERNAL errors.

Reference behaviour (``server/text_generation_server/interceptor.py:11-40``): log, free cached
allocator blocks, answer INTERNAL; a ``RuntimeError`` (CUDA errors surface as such) is considered
fatal for the shard and triggers the shutdown callback so the launcher restarts the deployment.
A kernel wait time-out reported by the device status word is raised as ``RuntimeError`` too.
"""
from __future__ import annotations

import logging
from typing import Callable, Optional

import grpc
import torch

log = logging.getLogger("tgi_b200.server")


class ExceptionInterceptor(grpc.aio.ServerInterceptor):
    def __init__(self, shutdown_callback: Optional[Callable[[], None]] = None):
        self.shutdown_callback = shutdown_callback

    async def intercept_service(self, continuation, handler_call_details):
        handler = await continuation(handler_call_details)
        if handler is None or handler.unary_unary is None:
            return handler
        inner = handler.unary_unary
        method = handler_call_details.method

        async def guarded(request, context):
            try:
                return await inner(request, context)
            except Exception as err:  # noqa: BLE001
                log.exception("Method %s encountered an error.", method)
                if isinstance(err, RuntimeError) and self.shutdown_callback is not None:
                    self.shutdown_callback()
                if torch.cuda.is_available():
                    torch.cuda.empty_cache()
                await context.abort(grpc.StatusCode.INTERNAL, f"{method}: {err}")

        return grpc.unary_unary_rpc_method_handler(
            guarded, request_deserializer=handler.request_deserializer,
            response_serializer=handler.response_serializer)
