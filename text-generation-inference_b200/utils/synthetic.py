"""Random-weight checkpoints of a given architecture (tests, smoke run, benchmarks).

``write_llama_checkpoint`` writes an HF-layout directory (``config.json`` + ``model.safetensors``)
with weights ``N(0, std)`` from a seed and norm weights 1.0 — small models for CPU tests.
``SyntheticWeights`` generates an *in-memory* checkpoint tensor by tensor directly on the GPU for
benchmark-size models that would take too long to write to disk; it returns a ``Weights``-like
object the decoder loads from (same names, same sharding entry points).
"""
from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Dict, Optional

import torch

from .weights import save_safetensors


def llama_config(hidden=256, layers=2, heads=4, kv_heads=2, intermediate=688, vocab=32000, eps=1e-5,
                 theta=10000.0, max_pos=4096, tie=False, model_type="llama", **extra) -> dict:
    cfg = dict(
        architectures=["LlamaForCausalLM"], model_type=model_type, hidden_size=hidden, num_hidden_layers=layers,
        num_attention_heads=heads, num_key_value_heads=kv_heads, intermediate_size=intermediate,
        vocab_size=vocab, rms_norm_eps=eps, rope_theta=theta, max_position_embeddings=max_pos,
        hidden_act="silu", tie_word_embeddings=tie, torch_dtype="float32", bos_token_id=1, eos_token_id=2,
    )
    cfg.update(extra)
    return cfg


def llama_state_dict(cfg: dict, seed: int = 0, std: float = 0.02, dtype=torch.float32,
                     device: str = "cpu") -> Dict[str, torch.Tensor]:
    """Random weights of a Llama / Mixtral shape as a CPU state dict; ``device`` is where the random numbers are
    drawn (a GPU draws a multi-billion-parameter checkpoint in seconds)."""
    g = torch.Generator(device=device).manual_seed(seed)
    H, L = cfg["hidden_size"], cfg["num_hidden_layers"]
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    D = cfg.get("head_dim") or H // nh
    I, V = cfg["intermediate_size"], cfg["vocab_size"]

    def rnd(*shape):
        return (torch.randn(*shape, generator=g, device=device) * std).to(dtype).cpu()

    sd = {"model.embed_tokens.weight": rnd(V, H), "model.norm.weight": torch.ones(H, dtype=dtype)}
    if not cfg.get("tie_word_embeddings"):
        sd["lm_head.weight"] = rnd(V, H)
    E = cfg.get("num_local_experts", 0)
    for i in range(L):
        p = f"model.layers.{i}"
        sd[f"{p}.input_layernorm.weight"] = torch.ones(H, dtype=dtype)
        sd[f"{p}.post_attention_layernorm.weight"] = torch.ones(H, dtype=dtype)
        sd[f"{p}.self_attn.q_proj.weight"] = rnd(nh * D, H)
        sd[f"{p}.self_attn.k_proj.weight"] = rnd(nkv * D, H)
        sd[f"{p}.self_attn.v_proj.weight"] = rnd(nkv * D, H)
        sd[f"{p}.self_attn.o_proj.weight"] = rnd(H, nh * D)
        if cfg.get("attention_bias") or cfg["model_type"] == "qwen2":
            sd[f"{p}.self_attn.q_proj.bias"] = rnd(nh * D)
            sd[f"{p}.self_attn.k_proj.bias"] = rnd(nkv * D)
            sd[f"{p}.self_attn.v_proj.bias"] = rnd(nkv * D)
        if E:
            sd[f"{p}.block_sparse_moe.gate.weight"] = rnd(E, H)
            for e in range(E):
                sd[f"{p}.block_sparse_moe.experts.{e}.w1.weight"] = rnd(I, H)
                sd[f"{p}.block_sparse_moe.experts.{e}.w3.weight"] = rnd(I, H)
                sd[f"{p}.block_sparse_moe.experts.{e}.w2.weight"] = rnd(H, I)
        else:
            sd[f"{p}.mlp.gate_proj.weight"] = rnd(I, H)
            sd[f"{p}.mlp.up_proj.weight"] = rnd(I, H)
            sd[f"{p}.mlp.down_proj.weight"] = rnd(H, I)
    return sd


def write_llama_checkpoint(path, cfg: Optional[dict] = None, seed: int = 0, std: float = 0.02,
                           dtype=torch.float32, device: str = "cpu") -> Path:
    cfg = cfg or llama_config()
    p = Path(path)
    p.mkdir(parents=True, exist_ok=True)
    (p / "config.json").write_text(json.dumps(cfg, indent=1))
    save_safetensors(llama_state_dict(cfg, seed, std, dtype, device), p / "model.safetensors", {"format": "pt"})
    return p


def reference_llama_forward(sd: Dict[str, torch.Tensor], cfg: dict, input_ids: torch.Tensor) -> torch.Tensor:
    """Plain dense PyTorch Llama forward (no paging, no fusion) over one sequence ``input_ids[T]``.

    Independent oracle for the engine's logits: returns ``[T, vocab]`` in fp32.
    """
    H, L = cfg["hidden_size"], cfg["num_hidden_layers"]
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    D = cfg.get("head_dim") or H // nh
    eps, theta = cfg["rms_norm_eps"], cfg["rope_theta"]
    T = input_ids.shape[0]
    x = sd["model.embed_tokens.weight"].float()[input_ids]
    pos = torch.arange(T, dtype=torch.float32)
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    ang = torch.outer(pos, inv)
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]

    def norm(v, w):
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * w.float()

    def rope(v):
        a, b = v[..., : D // 2], v[..., D // 2:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)

    mask = torch.full((T, T), float("-inf")).triu(1)
    for i in range(L):
        p = f"model.layers.{i}"
        h = norm(x, sd[f"{p}.input_layernorm.weight"])
        q = (h @ sd[f"{p}.self_attn.q_proj.weight"].float().t()).view(T, nh, D)
        k = (h @ sd[f"{p}.self_attn.k_proj.weight"].float().t()).view(T, nkv, D)
        v = (h @ sd[f"{p}.self_attn.v_proj.weight"].float().t()).view(T, nkv, D)
        q, k = rope(q), rope(k)
        k = k.repeat_interleave(nh // nkv, 1)
        v = v.repeat_interleave(nh // nkv, 1)
        att = torch.einsum("thd,shd->hts", q, k) / (D ** 0.5) + mask
        o = torch.einsum("hts,shd->thd", att.softmax(-1), v).reshape(T, nh * D)
        x = x + o @ sd[f"{p}.self_attn.o_proj.weight"].float().t()
        h = norm(x, sd[f"{p}.post_attention_layernorm.weight"])
        g = h @ sd[f"{p}.mlp.gate_proj.weight"].float().t()
        u = h @ sd[f"{p}.mlp.up_proj.weight"].float().t()
        x = x + (torch.nn.functional.silu(g) * u) @ sd[f"{p}.mlp.down_proj.weight"].float().t()
    x = norm(x, sd["model.norm.weight"])
    head = sd.get("lm_head.weight", sd["model.embed_tokens.weight"]).float()
    return x @ head.t()


# ---------------------------------------------------------------------------------------------
# benchmark-size models: weights generated on the device, shard by shard, never materialised whole
# ---------------------------------------------------------------------------------------------
class _GeneratedSlice:
    """Stands in for ``weights.TensorSlice``: produces (a slice of) a random tensor on demand.

    The values of rows ``[a, b)`` depend only on ``(name, dim, a)``, so a weight shard and the
    block scales computed from the same rows agree with each other.
    """

    def __init__(self, owner: "SyntheticWeights", name: str, shape, kind: str):
        self.owner, self.name, self.shape, self.kind = owner, name, tuple(shape), kind

    def get_shape(self):
        return self.shape

    def tensor(self):
        return self.slice_dim(0, 0, self.shape[0]) if self.shape else self.owner._make(self.name, self.kind, (), 0, 0)

    def slice_dim(self, dim: int, start: int, stop: int):
        shape = list(self.shape)
        shape[dim] = max(0, stop - start)
        return self.owner._make(self.name, self.kind, tuple(shape), dim, start)


class SyntheticWeights:
    """``Weights``-compatible provider of random Llama-architecture parameters created on the device.

    ``fp8_block=True`` serves every linear projection as e4m3 with ``weight_scale_inv`` per 128x128
    block, quantised from seeded ``N(0, std)`` bf16 values; embeddings, norms and the head stay bf16.
    """

    def __new__(cls, cfg: dict, device, dtype=torch.bfloat16, process_group=None, fp8_block: bool = False,
                std: float = 0.02, seed: int = 0):
        from .weights import Weights

        class _Impl(Weights):
            pass

        self = _Impl.__new__(_Impl)
        Weights.__init__(self, [], device, dtype, process_group=process_group)
        self.cfg, self.fp8_block, self.std, self.seed = cfg, fp8_block, std, seed
        H, L = cfg["hidden_size"], cfg["num_hidden_layers"]
        nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
        D = cfg.get("head_dim") or H // nh
        I, V = cfg["intermediate_size"], cfg["vocab_size"]
        E = cfg.get("num_local_experts", 0)
        shapes = {"model.embed_tokens.weight": ((V, H), "plain"), "model.norm.weight": ((H,), "ones"),
                  "lm_head.weight": ((V, H), "plain")}
        for i in range(L):
            p = f"model.layers.{i}"
            shapes[f"{p}.input_layernorm.weight"] = ((H,), "ones")
            shapes[f"{p}.post_attention_layernorm.weight"] = ((H,), "ones")
            lin = {f"{p}.self_attn.q_proj": (nh * D, H), f"{p}.self_attn.k_proj": (nkv * D, H),
                   f"{p}.self_attn.v_proj": (nkv * D, H), f"{p}.self_attn.o_proj": (H, nh * D)}
            if E:
                shapes[f"{p}.block_sparse_moe.gate.weight"] = ((E, H), "plain")
                for e in range(E):
                    lin[f"{p}.block_sparse_moe.experts.{e}.w1"] = (I, H)
                    lin[f"{p}.block_sparse_moe.experts.{e}.w3"] = (I, H)
                    lin[f"{p}.block_sparse_moe.experts.{e}.w2"] = (H, I)
            else:
                lin.update({f"{p}.mlp.gate_proj": (I, H), f"{p}.mlp.up_proj": (I, H), f"{p}.mlp.down_proj": (H, I)})
            for name, shp in lin.items():
                if fp8_block and not E:
                    shapes[f"{name}.weight"] = (shp, "fp8")
                    shapes[f"{name}.weight_scale_inv"] = (((shp[0] + 127) // 128, (shp[1] + 127) // 128), "scale")
                else:
                    shapes[f"{name}.weight"] = (shp, "plain")
        self._shapes = shapes
        self.routing = {k: 0 for k in shapes}

        def _slice(name, _self=self):
            h, real = _self.resolve(name)
            shp, kind = _self._shapes[real]
            return _GeneratedSlice(_self, real, shp, kind)

        def resolve(name, _self=self):
            if name in _self._shapes:
                return None, name
            raise KeyError(f"weight {name} does not exist")

        def _make(name, kind, shape, dim, start, _self=self):
            import zlib

            dev = _self.device
            if kind == "ones":
                return torch.ones(shape, dtype=_self.dtype, device=dev)
            base = name[: -len("_scale_inv")] if kind == "scale" else name
            row0 = start * (128 if kind == "scale" else 1)
            g = torch.Generator(device=dev)
            g.manual_seed((zlib.crc32(base.encode()) * 1000003 + dim * 7919 + row0 + _self.seed) & 0x7FFFFFFF)
            if kind == "plain":
                return (torch.randn(shape, generator=g, device=dev, dtype=torch.float32) * _self.std).to(_self.dtype)
            from ..ops import reference as ref

            if kind == "fp8":
                w = (torch.randn(shape, generator=g, device=dev, dtype=torch.float32) * _self.std).to(torch.bfloat16)
                if dim == 1 and shape[0] > 0:
                    pass
                q, _ = ref.fp8_quant_block_weight(w)
                return q
            # scale: regenerate the rows the scales belong to
            full_w = _self._shapes[base][0]
            wshape = list(full_w)
            wshape[dim] = shape[dim] * 128
            wshape[dim] = min(wshape[dim], full_w[dim] - row0)
            w = (torch.randn(tuple(wshape), generator=g, device=dev, dtype=torch.float32) * _self.std).to(torch.bfloat16)
            _, s = ref.fp8_quant_block_weight(w)
            return s

        self._slice = _slice
        self.resolve = resolve
        self._make = _make
        self.has_tensor = lambda name, _self=self: name in _self._shapes
        return self


def llama3_8b_config(**kw) -> dict:
    return llama_config(hidden=4096, layers=32, heads=32, kv_heads=8, intermediate=14336, vocab=128256,
                        theta=500000.0, max_pos=8192, **kw)


def llama3_70b_config(block_fp8: bool = True, **kw) -> dict:
    cfg = llama_config(hidden=8192, layers=80, heads=64, kv_heads=8, intermediate=28672, vocab=128256,
                       theta=500000.0, max_pos=8192, **kw)
    if block_fp8:
        cfg["quantization_config"] = {"quant_method": "fp8", "weight_block_size": [128, 128],
                                      "activation_scheme": "dynamic", "fmt": "e4m3"}
    return cfg


def mixtral_8x7b_config(**kw) -> dict:
    return llama_config(hidden=4096, layers=32, heads=32, kv_heads=8, intermediate=14336, vocab=32000,
                        theta=1000000.0, max_pos=32768, model_type="mixtral", num_local_experts=8,
                        num_experts_per_tok=2, **kw)
