"""Model registry: ``config.json`` -> runner.

Role of the reference's ``models/__init__.py`` (``ModelType`` enum ``:217-417``, ``get_model``
``:425-1800``, ``get_model_with_lora_adapters`` ``:1802-1916``): resolve dtype / quantisation /
KV-cache dtype / speculation, pick a runner, load weights shard-wise, attach LoRA adapters.
"""
from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Dict, List, Optional

import torch

from ..parallel.dist import initialize_torch_distributed
from ..utils.quantization import get_loader
from ..utils.tokenizer import load_tokenizer
from ..utils.weights import Weights, weight_files
from .arch import ARCHS, ModelConfig

# model_type -> (display name, multimodal)
SUPPORTED: Dict[str, str] = {k: k for k in ARCHS}

_DTYPES = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32, None: None}


def resolve_dtype(dtype: Optional[str], device: torch.device, quantize: Optional[str]) -> torch.dtype:
    if dtype is not None:
        return _DTYPES[dtype]
    if device.type == "cpu":
        return torch.float32
    return torch.bfloat16


def resolve_kv_dtype(kv_cache_dtype: Optional[str], dtype: torch.dtype) -> torch.dtype:
    if kv_cache_dtype in (None, "", "auto"):
        return dtype
    if kv_cache_dtype in ("fp8_e4m3fn", "fp8", "fp8_e4m3"):
        return torch.float8_e4m3fn
    if kv_cache_dtype == "fp8_e5m2":
        return torch.float8_e5m2
    raise ValueError(f"unknown kv cache dtype {kv_cache_dtype}")


def eos_token_ids(model_path: Path, cfg: ModelConfig):
    ids = set()
    g = model_path / "generation_config.json"
    src = json.loads(g.read_text()) if g.exists() else {}
    for e in (src.get("eos_token_id"), cfg.get("eos_token_id")):
        if isinstance(e, int):
            ids.add(e)
        elif isinstance(e, (list, tuple)):
            ids.update(int(x) for x in e)
    return ids or None


def get_model(
    model_id: str,
    revision: Optional[str] = None,
    sharded: bool = False,
    quantize: Optional[str] = None,
    speculate: Optional[int] = None,
    dtype: Optional[str] = None,
    kv_cache_dtype: Optional[str] = None,
    trust_remote_code: bool = False,
    max_input_tokens: Optional[int] = None,
    device: Optional[torch.device] = None,
    max_prefill_tokens: Optional[int] = None,
):
    """Load the shard of ``model_id`` (a local directory) that belongs to this process."""
    from .flash_causal_lm import FlashCausalLM
    from .decoder import CausalDecoder

    process_group, rank, world = initialize_torch_distributed()
    if device is None:
        device = torch.device(f"cuda:{torch.cuda.current_device()}") if torch.cuda.is_available() else torch.device("cpu")
    path = Path(model_id)
    if not path.is_dir():
        from ..utils.hub import resolve_model_path

        path = resolve_model_path(model_id, revision)
    cfg = ModelConfig.from_path(path)
    model_type = cfg.model_type
    tdtype = resolve_dtype(dtype, device, quantize)
    loader = get_loader(quantize, path, cfg.to_dict())
    speculate = int(speculate or 0)
    tokenizer = load_tokenizer(str(path), revision, trust_remote_code, vocab_size=cfg.get("vocab_size", 259))
    if model_type == "idefics":
        from .idefics import load_idefics

        return load_idefics(path, cfg, process_group, rank, world, tdtype, device, tokenizer)
    if model_type == "mllama":
        from .mllama import load_mllama

        return load_mllama(path, cfg, loader, process_group, rank, world, tdtype, device, tokenizer, speculate,
                           kv_cache_dtype, max_prefill_tokens)
    if model_type in ("llava_next", "llava", "idefics2", "idefics3", "paligemma", "qwen2_vl", "qwen2_5_vl") or (
            model_type == "gemma3" and cfg.get("vision_config") is not None):
        from .vlm_causal_lm import load_vlm

        return load_vlm(path, cfg, loader, process_group, rank, world, tdtype, device, tokenizer, speculate,
                        kv_cache_dtype, max_prefill_tokens)
    if model_type not in ARCHS and os.environ.get("TGI_B200_TRANSFORMERS_BACKEND", "1") == "1":
        # unknown architecture whose transformers implementation goes through the attention interface: its
        # own modules run around the paged attention (continuous batching, prefix caching, chunking kept)
        from . import transformers_backend

        if transformers_backend.supports(cfg.to_dict()):
            return transformers_backend.load_transformers_flash(
                path, cfg, process_group, rank, world, tdtype, device, tokenizer, speculate, kv_cache_dtype,
                max_prefill_tokens)
    if model_type in ("bloom", "mpt", "opt", "t5", "mamba") or model_type not in ARCHS:
        from .padded import load_padded

        return load_padded(path, cfg, process_group, rank, world, tdtype, device, tokenizer)
    text_cfg = cfg.text_config()
    weights = Weights(weight_files(path), device, tdtype, process_group=process_group, loader=loader,
                      aliases=_aliases(model_type))
    prefix = ""
    if model_type in ("gpt2",) and weights.has_tensor("transformer.wte.weight"):
        prefix = "transformer"
    if model_type == "gpt2" and text_cfg.get("attention_head_type") == "multiquery":
        weights.derive = _santacoder_fused_qkv
    from ..parallel.peer import make_comm

    hidden = int(text_cfg.get("hidden_size", text_cfg.get("n_embd", text_cfg.get("d_model", 0))) or 0)
    comm = make_comm(process_group, rank, world, device, hidden, int(max_prefill_tokens or 4096)) if hidden else None
    model = CausalDecoder(text_cfg, weights, comm=comm, prefix=prefix,
                          max_positions=_max_positions(text_cfg, max_input_tokens))
    from .speculative import find_speculator, load_speculator

    spec_path = find_speculator(path)
    if spec_path is not None and (spec_path / "config.json").exists() and (
            spec_path != path or (path / "medusa_lm_head.safetensors").exists()):
        head, n_spec = load_speculator(spec_path, device, tdtype, process_group, model.head)
        model.speculator = head
        speculate = speculate or n_spec
    runner = FlashCausalLM(model, tokenizer, tdtype, device, rank, world, speculate,
                           resolve_kv_dtype(kv_cache_dtype, tdtype), max_prefill_tokens,
                           eos_token_ids(path, cfg))
    weights.close()
    return runner


def _max_positions(cfg: ModelConfig, max_input_tokens: Optional[int]) -> int:
    mp = int(cfg.get("max_position_embeddings", cfg.get("n_positions", 2048)))
    cap = int(os.environ.get("TGI_B200_MAX_POSITIONS", "0"))
    if cap:
        mp = min(mp, cap) if cap < mp else cap
    return mp


def _santacoder_fused_qkv(weights, name: str, probe: bool):
    """The first SantaCoder checkpoints (a ``gpt2`` config with ``attention_head_type: multiquery`` and custom
    modelling code) store the query projection and the shared key/value projection separately
    (``attn.q_attn`` [H, H], ``attn.kv_attn`` [H, 2 D], both in the transposed GPT-2 layout); the decoder wants one
    ``attn.c_attn``.  Reference: ``custom_modeling/flash_santacoder_modeling.py:60-130`` builds the same fused
    matrix at load."""
    for kind in ("weight", "bias"):
        tail = f"attn.c_attn.{kind}"
        if name.endswith(tail):
            stem = name[:-len(tail)]
            q, kv = f"{stem}attn.q_attn.{kind}", f"{stem}attn.kv_attn.{kind}"
            if not (weights.has_tensor(q) and weights.has_tensor(kv)):
                return None
            if probe:
                return True
            return torch.cat([weights.get_tensor(q, to_device=False), weights.get_tensor(kv, to_device=False)], dim=-1)
    return None


def _aliases(model_type: str):
    if model_type in ("llama", "mistral", "qwen2", "qwen3", "gemma", "gemma2", "phi3", "granite"):
        return {"lm_head.weight": ["model.embed_tokens.weight"]}
    if model_type == "gpt2":
        return {"lm_head.weight": ["wte.weight", "transformer.wte.weight"]}
    return {}


def get_model_with_lora_adapters(model_id: str, lora_adapters=None, **kwargs):
    model = get_model(model_id, **kwargs)
    if lora_adapters:
        from ..utils.adapter import load_and_attach_adapters

        load_and_attach_adapters(model, model_id, lora_adapters)
    return model
