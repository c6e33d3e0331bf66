"""Blocking gRPC client of one shard or of all shards (used by the benchmark tool and the tests).

Mirrors the reference's Rust clients (``backends/v3/src/client/grpc_client.rs``,
``sharded_client.rs``): ``ShardedClient`` discovers the shard urls from shard 0, sends every RPC to
all shards, concatenates their generations and keeps the slowest shard's timings.
"""
from __future__ import annotations

from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional

import grpc

from ..proto import generate_v3 as pb


class ShardClient:
    def __init__(self, url: str):
        self.channel = grpc.insecure_channel(url, options=[("grpc.max_receive_message_length", (1 << 31) - 1),
                                                          ("grpc.max_send_message_length", (1 << 31) - 1)])
        self._calls = {}
        for rpc, (req, resp) in pb.METHODS.items():
            self._calls[rpc] = self.channel.unary_unary(
                pb.full_method(rpc), request_serializer=lambda m: m.SerializeToString(),
                response_deserializer=pb.message_class(resp).FromString)

    def call(self, rpc: str, request, timeout: Optional[float] = None):
        return self._calls[rpc](request, timeout=timeout)

    def close(self):
        self.channel.close()


class ShardedClient:
    def __init__(self, clients: List[ShardClient]):
        self.clients = clients
        self.pool = ThreadPoolExecutor(max_workers=max(1, len(clients)))

    @classmethod
    def connect_uds(cls, path: str) -> "ShardedClient":
        first = ShardClient(f"unix://{path}")
        urls = list(first.call("ServiceDiscovery", pb.ServiceDiscoveryRequest()).urls)
        first.close()
        return cls([ShardClient(u) for u in urls])

    def _all(self, rpc, request):
        return list(self.pool.map(lambda c: c.call(rpc, request), self.clients))

    def info(self):
        return self._all("Info", pb.InfoRequest())[0]

    def health(self):
        return self._all("Health", pb.HealthRequest())[0]

    def clear_cache(self, batch_id: Optional[int] = None):
        req = pb.ClearCacheRequest()
        if batch_id is not None:
            req.id = batch_id
        self._all("ClearCache", req)

    def filter_batch(self, batch_id: int, request_ids: List[int]):
        return self._all("FilterBatch", pb.FilterBatchRequest(batch_id=batch_id, request_ids=request_ids))[0].batch

    def warmup(self, request):
        rs = self._all("Warmup", request)
        supported = [r.max_supported_total_tokens for r in rs if r.HasField("max_supported_total_tokens")]
        return (min(supported) if supported else None, min(r.max_input_tokens for r in rs),
                min(r.max_total_tokens for r in rs))

    def _merge(self, rs):
        gens = [g for r in rs for g in r.generations]
        slow = max(rs, key=lambda r: r.total_ns)
        return gens, (slow.batch if slow.HasField("batch") else None), slow

    def prefill(self, batch, cached_batch=None):
        req = pb.PrefillRequest(batch=batch)
        if cached_batch is not None:
            req.cached_batch.CopyFrom(cached_batch)
        return self._merge(self._all("Prefill", req))

    def decode(self, batches):
        return self._merge(self._all("Decode", pb.DecodeRequest(batches=batches)))

    def close(self):
        for c in self.clients:
            c.close()
