"""Shard command line: ``serve``, ``download-weights`` and ``quantize``.

Same commands as the reference's typer app (``server/text_generation_server/cli.py:41-372``), built on
argparse:  ``python -m tgi_b200.server.cli serve MODEL_DIR [--sharded] [--quantize fp8] ...``
"""
from __future__ import annotations

import argparse
import json
import logging
import os
import sys
from pathlib import Path


class _JsonFormatter(logging.Formatter):
    def format(self, record):
        message = record.getMessage()
        if record.exc_info:      # keep the traceback with the record: the launcher re-emits one record per line
            message += "\n" + self.formatException(record.exc_info)
        return json.dumps({"timestamp": self.formatTime(record), "level": record.levelname,
                           "target": record.name, "message": message})


def _setup_logging(level: str, json_output: bool):
    h = logging.StreamHandler(sys.stdout)
    h.setFormatter(_JsonFormatter() if json_output else logging.Formatter("%(asctime)s %(levelname)s %(name)s: %(message)s"))
    logging.basicConfig(level=getattr(logging, level.upper(), logging.INFO), handlers=[h], force=True)


def _parse_lora(spec: str):
    from ..utils.adapter import parse_lora_adapters

    return parse_lora_adapters(spec)


def cmd_serve(a):
    _setup_logging(a.logger_level, a.json_output)
    if a.sharded:
        for var in ("RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT"):
            if os.environ.get(var) is None:
                raise SystemExit(f"{var} must be set when sharded is True")
    lora = _parse_lora(os.environ.get("LORA_ADAPTERS", "")) if os.environ.get("LORA_ADAPTERS") else []
    if os.environ.get("TGI_B200_PIN_CPU") == "1":
        from ..parallel.dist import pin_cpu_threads

        local_world = int(os.environ.get("LOCAL_WORLD_SIZE", os.environ.get("WORLD_SIZE", "1")))
        pin_cpu_threads(int(os.environ.get("LOCAL_RANK", os.environ.get("RANK", "0"))) % max(local_world, 1), local_world)
    if a.otlp_endpoint:
        from .tracing import setup_tracing

        setup_tracing(a.otlp_service_name, a.otlp_endpoint)
    from .server import serve

    dtype = None if a.dtype is None else a.dtype
    if dtype is not None and a.quantize not in (None, "fp8", "eetq"):
        raise SystemExit("Only 1 can be set between `dtype` and `quantize`, as they both decide how goes the final model.")
    serve(a.model_id, lora, a.revision, a.sharded, a.quantize, a.speculate, dtype, a.kv_cache_dtype,
          a.trust_remote_code, Path(a.uds_path), a.max_input_tokens)


def cmd_download(a):
    _setup_logging(a.logger_level, a.json_output)
    from ..utils import hub

    hub.download_weights(a.model_id, a.revision, a.extension, a.auto_convert, a.merge_lora)


def cmd_quantize(a):
    _setup_logging(a.logger_level, a.json_output)
    from ..utils.gptq_quantize import quantize

    quantize(a.model_id, a.output_dir, bits=a.bits, groupsize=a.groupsize, act_order=a.act_order,
             percdamp=a.percdamp, nsamples=a.nsamples, seed=a.seed)


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="text-generation-server")
    sub = p.add_subparsers(dest="cmd", required=True)

    def common(sp):
        sp.add_argument("--logger-level", default=os.environ.get("LOG_LEVEL", "INFO"))
        sp.add_argument("--json-output", action="store_true")

    s = sub.add_parser("serve")
    s.add_argument("model_id")
    s.add_argument("--revision")
    s.add_argument("--sharded", action="store_true")
    s.add_argument("--quantize", choices=["bitsandbytes", "bitsandbytes-nf4", "bitsandbytes-fp4", "gptq", "awq",
                                          "compressed-tensors", "eetq", "exl2", "fp8", "marlin"])
    s.add_argument("--speculate", type=int)
    s.add_argument("--dtype", choices=["float16", "bfloat16", "float32"])
    s.add_argument("--kv-cache-dtype", choices=["fp8_e4m3fn", "fp8_e5m2"])
    s.add_argument("--trust-remote-code", action="store_true")
    s.add_argument("--uds-path", default="/tmp/text-generation-server")
    s.add_argument("--max-input-tokens", type=int)
    s.add_argument("--otlp-endpoint")
    s.add_argument("--otlp-service-name", default="text-generation-inference.server")
    common(s)
    s.set_defaults(fn=cmd_serve)

    d = sub.add_parser("download-weights")
    d.add_argument("model_id")
    d.add_argument("--revision")
    d.add_argument("--extension", default=".safetensors")
    d.add_argument("--auto-convert", action=argparse.BooleanOptionalAction, default=True)
    d.add_argument("--merge-lora", action="store_true")
    common(d)
    d.set_defaults(fn=cmd_download)

    q = sub.add_parser("quantize")
    q.add_argument("model_id")
    q.add_argument("output_dir")
    q.add_argument("--bits", type=int, default=4)
    q.add_argument("--groupsize", type=int, default=128)
    q.add_argument("--act-order", action="store_true")
    q.add_argument("--percdamp", type=float, default=0.01)
    q.add_argument("--nsamples", type=int, default=128)
    q.add_argument("--seed", type=int, default=0)
    common(q)
    q.set_defaults(fn=cmd_quantize)
    return p


def main(argv=None):
    a = build_parser().parse_args(argv)
    a.fn(a)


if __name__ == "__main__":
    main()
