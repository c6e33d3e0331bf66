"""``generate.v3`` protobuf schema, built at import time without ``protoc``.

The router<->shard contract of the reference is ``proto/v3/generate.proto``
(service ``generate.v3.TextGenerationService``; messages at
``proto/v3/generate.proto:25-289``).  Neither ``protoc`` nor ``grpc_tools`` is
available where this package is built, so the schema is declared below as a
compact table and turned into a ``FileDescriptorProto``; message classes come
from the protobuf runtime's message factory.  Field names and numbers are the
wire contract and must not change.

Usage::

    from tgi_b200.proto import generate_v3 as pb
    req = pb.Request(id=1, inputs="hi")
    pb.Request.FromString(req.SerializeToString())
"""
from __future__ import annotations

from google.protobuf import descriptor_pb2, descriptor_pool, message_factory

_F = descriptor_pb2.FieldDescriptorProto

PACKAGE = "generate.v3"
SERVICE = "TextGenerationService"

_SCALAR = {
    "bool": _F.TYPE_BOOL,
    "string": _F.TYPE_STRING,
    "bytes": _F.TYPE_BYTES,
    "uint32": _F.TYPE_UINT32,
    "uint64": _F.TYPE_UINT64,
    "float": _F.TYPE_FLOAT,
}

_ENUMS = {
    "GrammarType": [("GRAMMAR_TYPE_NONE", 0), ("GRAMMAR_TYPE_JSON", 1), ("GRAMMAR_TYPE_REGEX", 2)],
    "FinishReason": [
        ("FINISH_REASON_LENGTH", 0),
        ("FINISH_REASON_EOS_TOKEN", 1),
        ("FINISH_REASON_STOP_SEQUENCE", 2),
    ],
}

# (name, number, type, label) with label in {"", "repeated", "optional", "oneof:<name>"}
_MESSAGES = {
    "HealthRequest": [],
    "HealthResponse": [],
    "InfoRequest": [],
    "InfoResponse": [
        ("requires_padding", 1, "bool", ""),
        ("dtype", 2, "string", ""),
        ("device_type", 3, "string", ""),
        ("window_size", 4, "uint32", "optional"),
        ("speculate", 5, "uint32", ""),
        ("support_chunking", 6, "bool", ""),
        ("use_prefix_caching", 7, "bool", ""),
        ("attention_impl", 8, "string", ""),
        ("block_size", 9, "uint32", ""),
    ],
    "ServiceDiscoveryRequest": [],
    "ServiceDiscoveryResponse": [("urls", 1, "string", "repeated")],
    "ClearCacheRequest": [("id", 1, "uint64", "optional")],
    "ClearCacheResponse": [],
    "Image": [("data", 1, "bytes", ""), ("mimetype", 2, "string", "")],
    "InputChunk": [("text", 1, "string", "oneof:chunk"), ("image", 2, "Image", "oneof:chunk")],
    "Input": [("chunks", 1, "InputChunk", "repeated")],
    "NextTokenChooserParameters": [
        ("temperature", 1, "float", ""),
        ("top_k", 2, "uint32", ""),
        ("top_p", 3, "float", ""),
        ("typical_p", 4, "float", ""),
        ("do_sample", 5, "bool", ""),
        ("seed", 6, "uint64", ""),
        ("repetition_penalty", 7, "float", ""),
        ("frequency_penalty", 9, "float", ""),
        ("watermark", 8, "bool", ""),
        ("grammar", 10, "string", ""),
        ("grammar_type", 11, "GrammarType", ""),
    ],
    "StoppingCriteriaParameters": [
        ("max_new_tokens", 1, "uint32", ""),
        ("stop_sequences", 2, "string", "repeated"),
        ("ignore_eos_token", 3, "bool", ""),
    ],
    "Request": [
        ("id", 1, "uint64", ""),
        ("input_chunks", 8, "Input", ""),
        ("inputs", 2, "string", ""),
        ("truncate", 3, "uint32", ""),
        ("parameters", 4, "NextTokenChooserParameters", ""),
        ("stopping_parameters", 5, "StoppingCriteriaParameters", ""),
        ("prefill_logprobs", 6, "bool", ""),
        ("top_n_tokens", 7, "uint32", ""),
        ("blocks", 9, "uint32", "repeated"),
        ("slots", 10, "uint32", "repeated"),
        ("adapter_id", 11, "string", "optional"),
        ("cache_len", 12, "uint32", ""),
        ("add_special_tokens", 13, "bool", ""),
        ("chunk_len", 14, "uint32", "optional"),
    ],
    "Batch": [
        ("id", 1, "uint64", ""),
        ("requests", 2, "Request", "repeated"),
        ("size", 3, "uint32", ""),
        ("max_tokens", 4, "uint32", ""),
        ("max_blocks", 5, "uint32", ""),
    ],
    "CachedBatch": [
        ("id", 1, "uint64", ""),
        ("request_ids", 2, "uint64", "repeated"),
        ("size", 3, "uint32", ""),
        ("max_tokens", 4, "uint32", ""),
        ("current_tokens", 5, "uint32", ""),
    ],
    "GeneratedText": [
        ("text", 1, "string", ""),
        ("generated_tokens", 2, "uint32", ""),
        ("finish_reason", 3, "FinishReason", ""),
        ("seed", 4, "uint64", "optional"),
    ],
    "Tokens": [
        ("ids", 1, "uint32", "repeated"),
        ("logprobs", 2, "float", "repeated"),
        ("texts", 3, "string", "repeated"),
        ("is_special", 4, "bool", "repeated"),
    ],
    "Generation": [
        ("request_id", 1, "uint64", ""),
        ("prefill_tokens", 2, "Tokens", ""),
        ("tokens", 3, "Tokens", ""),
        ("generated_text", 4, "GeneratedText", "optional"),
        ("top_tokens", 5, "Tokens", "repeated"),
    ],
    "FilterBatchRequest": [("batch_id", 1, "uint64", ""), ("request_ids", 2, "uint64", "repeated")],
    "FilterBatchResponse": [("batch", 1, "CachedBatch", "")],
    "PrefillRequest": [("batch", 1, "Batch", ""), ("cached_batch", 2, "CachedBatch", "")],
    "PrefillResponse": [
        ("generations", 1, "Generation", "repeated"),
        ("batch", 2, "CachedBatch", "optional"),
        ("forward_ns", 3, "uint64", ""),
        ("decode_ns", 4, "uint64", ""),
        ("total_ns", 5, "uint64", ""),
        ("concat_ns", 6, "uint64", "optional"),
    ],
    "DecodeRequest": [("batches", 1, "CachedBatch", "repeated")],
    "DecodeResponse": [
        ("generations", 1, "Generation", "repeated"),
        ("batch", 2, "CachedBatch", "optional"),
        ("forward_ns", 3, "uint64", ""),
        ("decode_ns", 4, "uint64", ""),
        ("total_ns", 5, "uint64", ""),
        ("concat_ns", 6, "uint64", "optional"),
    ],
    "WarmupRequest": [
        ("batch", 1, "Batch", ""),
        ("max_input_tokens", 2, "uint32", "optional"),
        ("max_prefill_tokens", 3, "uint32", ""),
        ("max_total_tokens", 4, "uint32", "optional"),
    ],
    "WarmupResponse": [
        ("max_supported_total_tokens", 1, "uint32", "optional"),
        ("max_input_tokens", 2, "uint32", ""),
        ("max_total_tokens", 3, "uint32", ""),
    ],
}

# rpc name -> (request message, response message)
METHODS = {
    "Info": ("InfoRequest", "InfoResponse"),
    "ServiceDiscovery": ("ServiceDiscoveryRequest", "ServiceDiscoveryResponse"),
    "ClearCache": ("ClearCacheRequest", "ClearCacheResponse"),
    "FilterBatch": ("FilterBatchRequest", "FilterBatchResponse"),
    "Warmup": ("WarmupRequest", "WarmupResponse"),
    "Prefill": ("PrefillRequest", "PrefillResponse"),
    "Decode": ("DecodeRequest", "DecodeResponse"),
    "Health": ("HealthRequest", "HealthResponse"),
}


def _build_file() -> descriptor_pb2.FileDescriptorProto:
    fdp = descriptor_pb2.FileDescriptorProto()
    fdp.name = "tgi_b200/generate_v3.proto"
    fdp.package = PACKAGE
    fdp.syntax = "proto3"
    for ename, values in _ENUMS.items():
        e = fdp.enum_type.add()
        e.name = ename
        for vname, num in values:
            v = e.value.add()
            v.name, v.number = vname, num
    for mname, fields in _MESSAGES.items():
        m = fdp.message_type.add()
        m.name = mname
        oneofs: dict[str, int] = {}
        # Real oneofs must be declared before the synthetic ones created for
        # proto3 ``optional`` fields.
        for fname, num, ftype, label in fields:
            if label.startswith("oneof:"):
                oname = label.split(":", 1)[1]
                if oname not in oneofs:
                    oneofs[oname] = len(m.oneof_decl)
                    m.oneof_decl.add().name = oname
        for fname, num, ftype, label in fields:
            f = m.field.add()
            f.name, f.number = fname, num
            f.label = _F.LABEL_REPEATED if label == "repeated" else _F.LABEL_OPTIONAL
            if ftype in _SCALAR:
                f.type = _SCALAR[ftype]
            elif ftype in _ENUMS:
                f.type = _F.TYPE_ENUM
                f.type_name = f".{PACKAGE}.{ftype}"
            else:
                f.type = _F.TYPE_MESSAGE
                f.type_name = f".{PACKAGE}.{ftype}"
            if label == "optional":
                f.proto3_optional = True
                f.oneof_index = len(m.oneof_decl)
                m.oneof_decl.add().name = "_" + fname
            elif label.startswith("oneof:"):
                f.oneof_index = oneofs[label.split(":", 1)[1]]
    svc = fdp.service.add()
    svc.name = SERVICE
    for rpc, (req, resp) in METHODS.items():
        meth = svc.method.add()
        meth.name = rpc
        meth.input_type = f".{PACKAGE}.{req}"
        meth.output_type = f".{PACKAGE}.{resp}"
    return fdp


FILE_DESCRIPTOR_PROTO = _build_file()
_pool = descriptor_pool.DescriptorPool()
_file_desc = _pool.Add(FILE_DESCRIPTOR_PROTO) or _pool.FindFileByName(FILE_DESCRIPTOR_PROTO.name)

_classes = {}
for _name in _MESSAGES:
    _classes[_name] = message_factory.GetMessageClass(_pool.FindMessageTypeByName(f"{PACKAGE}.{_name}"))
globals().update(_classes)

GrammarType = _pool.FindEnumTypeByName(f"{PACKAGE}.GrammarType")
FinishReason = _pool.FindEnumTypeByName(f"{PACKAGE}.FinishReason")

GRAMMAR_TYPE_NONE, GRAMMAR_TYPE_JSON, GRAMMAR_TYPE_REGEX = 0, 1, 2
FINISH_REASON_LENGTH, FINISH_REASON_EOS_TOKEN, FINISH_REASON_STOP_SEQUENCE = 0, 1, 2


def full_method(rpc: str) -> str:
    """gRPC path of an rpc, e.g. ``/generate.v3.TextGenerationService/Prefill``."""
    return f"/{PACKAGE}.{SERVICE}/{rpc}"


def message_class(name: str):
    return _classes[name]


__all__ = list(_MESSAGES) + [
    "METHODS",
    "PACKAGE",
    "SERVICE",
    "full_method",
    "message_class",
    "GrammarType",
    "FinishReason",
]
