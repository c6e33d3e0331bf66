"""B200-native LLM serving engine with the API surface of text-generation-inference.

Layout
------
proto/     proto3 ``generate.v3`` schema (built at run time, no protoc) and codecs
utils/     weights/sharding, quantization loaders, sampling, stopping, watermark, grammar, hub
ops/       hand-written sm_100a CUDA kernels (``csrc/``) and their Python bindings / CPU oracles
parallel/  process-group bootstrap, NVLink peer-memory heap, fused compute+collective ops
models/    decoder implementations, batch state, model runner, registry
server/    shard gRPC servicer, batch cache, interceptor, CLI
router/    C++ launcher / HTTP front / scheduler / prefix cache (built as ``tgi-b200-router``)
client/    Python HTTP client
"""
__version__ = "0.1.0"
