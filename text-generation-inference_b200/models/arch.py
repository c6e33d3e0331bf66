"""Architecture descriptions: one generic decoder, many model families.

The reference has one modeling file per family under
``server/text_generation_server/models/custom_modeling/`` (llama ``flash_llama_modeling.py``,
mistral, mixtral, qwen2, gemma/gemma2/gemma3, phi/phi3, cohere, dbrx, gpt2, gptj, neox,
falcon ``flash_rw_modeling.py``, santacoder, starcoder2 ...), all variations of the same
pre-norm decoder.  Here a family is a *declaration* (``Arch``): tensor-name templates plus the
handful of switches in which the families differ; ``models/decoder.py`` interprets it.

``ModelConfig`` is a thin attribute view over ``config.json`` so that no model-specific config
class is needed.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field, replace
from pathlib import Path
from typing import Any, Dict, List, Optional


class ModelConfig:
    """Attribute access to ``config.json`` with ``get``-style defaults; unknown attributes are ``None``."""

    def __init__(self, data: Dict[str, Any]):
        object.__setattr__(self, "_d", dict(data))

    @classmethod
    def from_path(cls, path) -> "ModelConfig":
        p = Path(path)
        if p.is_dir():
            p = p / "config.json"
        return cls(json.loads(p.read_text()))

    def __getattr__(self, k):
        if k.startswith("__"):
            raise AttributeError(k)
        return self._d.get(k)

    def __setattr__(self, k, v):
        self._d[k] = v

    def get(self, k, default=None):
        v = self._d.get(k)
        return default if v is None else v

    def to_dict(self):
        return dict(self._d)

    def text_config(self) -> "ModelConfig":
        """Language-model part of a multimodal config."""
        t = self._d.get("text_config")
        if isinstance(t, dict):
            merged = dict(t)
            merged.setdefault("quantization_config", self._d.get("quantization_config"))
            return ModelConfig(merged)
        return self


@dataclass(frozen=True)
class Arch:
    # ---- tensor names ------------------------------------------------------------------------
    embed: str = "model.embed_tokens"
    pos_embed: Optional[str] = None          # learned absolute positions (gpt2, opt)
    pos_offset: int = 0                      # opt adds 2 to positions
    embed_norm: Optional[str] = None         # bloom word_embeddings_layernorm
    layer: str = "model.layers.{i}"
    norm1: str = "input_layernorm"
    norm2: Optional[str] = "post_attention_layernorm"
    post_attn_norm: Optional[str] = None     # gemma2/3: norm on the attention output
    post_mlp_norm: Optional[str] = None      # gemma2/3: norm on the MLP output
    final_norm: str = "model.norm"
    lm_head: str = "lm_head"
    q: str = "self_attn.q_proj"
    k: str = "self_attn.k_proj"
    v: str = "self_attn.v_proj"
    qkv: Optional[str] = None                # fused projection name, if the checkpoint fuses q,k,v
    qkv_layout: str = "blocked"              # "blocked" [q|k|v], "interleaved" per-head [q,k,v] (neox, bloom), "falcon"
    o: str = "self_attn.o_proj"
    q_norm: Optional[str] = None
    k_norm: Optional[str] = None
    gate: Optional[str] = "mlp.gate_proj"
    up: str = "mlp.up_proj"
    gate_up: Optional[str] = None            # fused gate+up name
    down: str = "mlp.down_proj"
    conv1d_weights: bool = False             # gpt2 stores linear weights transposed
    # ---- behaviour ---------------------------------------------------------------------------
    norm: str = "rms"                        # "rms" | "layer"
    norm_unit_offset: bool = False           # gemma: weight + 1
    norm_bias: bool = True                   # layer norm with bias
    qkv_bias: bool = False
    o_bias: bool = False
    mlp_bias: bool = False
    act: Optional[str] = None                # None: from config.hidden_act
    gated_mlp: bool = True
    parallel_residual: bool = False
    parallel_shared_norm: bool = True        # parallel blocks: one norm feeds attention and MLP
    rope: bool = True
    rope_neox: bool = True
    alibi: bool = False
    embed_scale_sqrt_hidden: bool = False    # gemma
    qk_norm_kind: str = "rms"                # "rms" per-head over head_dim | "layer" (cohere)
    # ---- mixture of experts ------------------------------------------------------------------
    moe: bool = False
    moe_router: str = "block_sparse_moe.gate"
    moe_expert: str = "block_sparse_moe.experts.{e}"
    moe_gate: str = "w1"
    moe_up: str = "w3"
    moe_down: str = "w2"
    moe_fused: bool = False                  # dbrx: experts stored stacked
    moe_shared: Optional[str] = None         # shared expert MLP prefix (qwen2_moe, deepseek)
    mla: bool = False                        # DeepSeek multi-head latent attention (models/deepseek.py)
    moe_shared_gate: Optional[str] = None
    moe_renormalize: bool = True


_LLAMA = Arch()

ARCHS: Dict[str, Arch] = {
    "llama": _LLAMA,
    "mistral": _LLAMA,
    "baichuan": replace(_LLAMA, qkv="self_attn.W_pack"),
    "granite": _LLAMA,
    "qwen2": replace(_LLAMA, qkv_bias=True),
    "qwen3": replace(_LLAMA, q_norm="self_attn.q_norm", k_norm="self_attn.k_norm"),
    "phi3": replace(_LLAMA, qkv="self_attn.qkv_proj", gate=None, gate_up="mlp.gate_up_proj"),
    "gemma": replace(_LLAMA, norm_unit_offset=True, embed_scale_sqrt_hidden=True),
    "gemma2": replace(_LLAMA, norm_unit_offset=True, embed_scale_sqrt_hidden=True,
                      norm2="pre_feedforward_layernorm", post_attn_norm="post_attention_layernorm",
                      post_mlp_norm="post_feedforward_layernorm"),
    "gemma3_text": replace(_LLAMA, norm_unit_offset=True, embed_scale_sqrt_hidden=True,
                           norm2="pre_feedforward_layernorm", post_attn_norm="post_attention_layernorm",
                           post_mlp_norm="post_feedforward_layernorm",
                           q_norm="self_attn.q_norm", k_norm="self_attn.k_norm"),
    "starcoder2": replace(_LLAMA, norm="layer", qkv_bias=True, o_bias=True, mlp_bias=True, gated_mlp=False,
                          gate=None, up="mlp.c_fc", down="mlp.c_proj"),
    "cohere": replace(_LLAMA, norm="layer", norm_bias=False, norm2=None, parallel_residual=True, rope_neox=False,
                      q_norm="self_attn.q_norm", k_norm="self_attn.k_norm", qk_norm_kind="layer"),
    "mixtral": replace(_LLAMA, moe=True),
    "phimoe": replace(_LLAMA, moe=True, norm="layer", qkv_bias=True, o_bias=True),
    "qwen2_moe": replace(_LLAMA, qkv_bias=True, moe=True, moe_router="mlp.gate", moe_expert="mlp.experts.{e}",
                         moe_gate="gate_proj", moe_up="up_proj", moe_down="down_proj",
                         moe_shared="mlp.shared_expert", moe_shared_gate="mlp.shared_expert_gate",
                         moe_renormalize=False),
    "qwen3_moe": replace(_LLAMA, q_norm="self_attn.q_norm", k_norm="self_attn.k_norm", moe=True,
                         moe_router="mlp.gate", moe_expert="mlp.experts.{e}", moe_gate="gate_proj",
                         moe_up="up_proj", moe_down="down_proj"),
    "gpt2": Arch(embed="wte", pos_embed="wpe", layer="h.{i}", norm1="ln_1", norm2="ln_2", final_norm="ln_f",
                 lm_head="lm_head", qkv="attn.c_attn", o="attn.c_proj", gate=None, up="mlp.c_fc",
                 down="mlp.c_proj", conv1d_weights=True, norm="layer", qkv_bias=True, o_bias=True,
                 mlp_bias=True, gated_mlp=False, rope=False),
    "gpt_bigcode": Arch(embed="transformer.wte", pos_embed="transformer.wpe", layer="transformer.h.{i}",
                        norm1="ln_1", norm2="ln_2", final_norm="transformer.ln_f", lm_head="lm_head",
                        qkv="attn.c_attn", o="attn.c_proj", gate=None, up="mlp.c_fc", down="mlp.c_proj",
                        norm="layer", qkv_bias=True, o_bias=True, mlp_bias=True, gated_mlp=False, rope=False),
    "gptj": Arch(embed="transformer.wte", layer="transformer.h.{i}", norm1="ln_1", norm2=None,
                 final_norm="transformer.ln_f", q="attn.q_proj", k="attn.k_proj", v="attn.v_proj",
                 o="attn.out_proj", gate=None, up="mlp.fc_in", down="mlp.fc_out", norm="layer",
                 mlp_bias=True, gated_mlp=False, parallel_residual=True, rope_neox=False),
    "gpt_neox": Arch(embed="gpt_neox.embed_in", layer="gpt_neox.layers.{i}", norm1="input_layernorm",
                     norm2="post_attention_layernorm", final_norm="gpt_neox.final_layer_norm",
                     lm_head="embed_out", qkv="attention.query_key_value", qkv_layout="interleaved",
                     o="attention.dense", gate=None, up="mlp.dense_h_to_4h", down="mlp.dense_4h_to_h",
                     norm="layer", qkv_bias=True, o_bias=True, mlp_bias=True, gated_mlp=False,
                     parallel_residual=True, parallel_shared_norm=False),
    "phi": Arch(layer="model.layers.{i}", norm1="input_layernorm", norm2=None, final_norm="model.final_layernorm",
                o="self_attn.dense", gate=None, up="mlp.fc1", down="mlp.fc2", norm="layer", qkv_bias=True,
                o_bias=True, mlp_bias=True, gated_mlp=False, parallel_residual=True),
    "falcon": Arch(embed="transformer.word_embeddings", layer="transformer.h.{i}", norm1="input_layernorm",
                   norm2=None, final_norm="transformer.ln_f", qkv="self_attention.query_key_value",
                   qkv_layout="falcon", o="self_attention.dense", gate=None, up="mlp.dense_h_to_4h",
                   down="mlp.dense_4h_to_h", norm="layer", gated_mlp=False, parallel_residual=True),
    "bloom": Arch(embed="word_embeddings", embed_norm="word_embeddings_layernorm", layer="h.{i}",
                  norm1="input_layernorm", norm2="post_attention_layernorm", final_norm="ln_f",
                  lm_head="lm_head", qkv="self_attention.query_key_value", qkv_layout="interleaved",
                  o="self_attention.dense", gate=None, up="mlp.dense_h_to_4h", down="mlp.dense_4h_to_h",
                  norm="layer", qkv_bias=True, o_bias=True, mlp_bias=True, gated_mlp=False, rope=False, alibi=True),
    "mpt": Arch(embed="transformer.wte", layer="transformer.blocks.{i}", norm1="norm_1", norm2="norm_2",
                final_norm="transformer.norm_f", qkv="attn.Wqkv", o="attn.out_proj", gate=None,
                up="ffn.up_proj", down="ffn.down_proj", norm="layer", norm_bias=False, gated_mlp=False,
                rope=False, alibi=True),
    "opt": Arch(embed="model.decoder.embed_tokens", pos_embed="model.decoder.embed_positions", pos_offset=2,
                layer="model.decoder.layers.{i}", norm1="self_attn_layer_norm", norm2="final_layer_norm",
                final_norm="model.decoder.final_layer_norm", o="self_attn.out_proj", gate=None, up="fc1",
                down="fc2", norm="layer", qkv_bias=True, o_bias=True, mlp_bias=True, gated_mlp=False, rope=False),
    "dbrx": Arch(embed="transformer.wte", layer="transformer.blocks.{i}", norm1="norm_attn_norm.norm_1",
                 norm2="norm_attn_norm.norm_2", final_norm="transformer.norm_f",
                 qkv="norm_attn_norm.attn.Wqkv", o="norm_attn_norm.attn.out_proj", norm="layer", norm_bias=False,
                 moe=True, moe_router="ffn.router.layer", moe_expert="ffn.experts.mlp", moe_fused=True,
                 moe_gate="w1", moe_up="v1", moe_down="w2"),
}
ARCHS["RefinedWeb"] = ARCHS["RefinedWebModel"] = ARCHS["falcon"]
ARCHS["deepseek_v2"] = ARCHS["deepseek_v3"] = replace(
    _LLAMA, rope_neox=False, mla=True, moe=True, moe_router="mlp.gate", moe_expert="mlp.experts.{e}",
    moe_gate="gate_proj", moe_up="up_proj", moe_down="down_proj", moe_shared="mlp.shared_experts")
ARCHS["gemma3"] = ARCHS["gemma3_text"]
ARCHS["phi-msft"] = ARCHS["phi"]
ARCHS["qwen2_vl_text"] = ARCHS["qwen2_5_vl_text"] = ARCHS["qwen2"]   # language models of Qwen2-VL / Qwen2.5-VL


def arch_for(model_type: str) -> Arch:
    if model_type not in ARCHS:
        raise NotImplementedError(f"model type {model_type} has no architecture description")
    return ARCHS[model_type]


@dataclass
class ModelDims:
    """Numbers derived from the config, after tensor-parallel division."""

    hidden: int
    num_layers: int
    num_heads: int          # per rank
    num_kv_heads: int       # per rank
    head_dim: int
    intermediate: int
    vocab: int
    eps: float
    rope_theta: float
    rot_dim: int
    max_positions: int
    act: str
    softmax_scale: float
    windows: List[int]      # per layer, -1 = full attention
    attn_softcap: float
    logit_softcap: float
    logit_scale: float
    embed_scale: float
    residual_scale: float
    num_experts: int = 0
    top_k: int = 0
    total_heads: int = 0
    total_kv_heads: int = 0
    attn_head_dim: int = 0      # head dimension seen by the attention kernels and the KV cache: head_dim padded to 64/128/256


def derive_dims(cfg: ModelConfig, arch: Arch, world: int) -> ModelDims:
    hidden = cfg.get("hidden_size", cfg.get("n_embd", cfg.get("d_model")))
    layers = cfg.get("num_hidden_layers", cfg.get("n_layer", cfg.get("n_layers")))
    heads = cfg.get("num_attention_heads", cfg.get("n_head", cfg.get("n_heads")))
    head_dim = cfg.get("head_dim", hidden // heads)
    kv = cfg.get("num_key_value_heads")
    if arch.mla:
        # latent attention is expanded to ordinary heads of a padded dimension (models/deepseek.py)
        head_dim, kv = 256, heads
    if kv is None and cfg.get("new_decoder_architecture") and cfg.get("num_kv_heads") is not None:
        kv = cfg.get("num_kv_heads")     # Falcon-40B style: grouped KV heads, `multi_query` is ignored
    if kv is None:
        if cfg.get("attention_head_type") == "multiquery":        # the first SantaCoder checkpoints
            kv = 1
        elif cfg.get("multi_query") or (cfg.model_type in ("falcon", "RefinedWebModel", "RefinedWeb")
                                      and cfg.get("multi_query", True) and not cfg.get("new_decoder_architecture")):
            kv = 1
        elif cfg.get("n_head_kv") is not None or cfg.get("num_kv_heads") is not None:
            kv = cfg.get("n_head_kv", cfg.get("num_kv_heads"))
        elif isinstance(cfg.get("attn_config"), dict) and cfg.attn_config.get("kv_n_heads"):
            kv = cfg.attn_config["kv_n_heads"]
        else:
            kv = heads
    if heads % world != 0:
        raise ValueError(f"`num_heads` must be divisible by `num_shards` (got `num_heads`: {heads} "
                         f"and `num_shards`: {world}")
    # MQA / few KV heads: replicate KV heads when there are fewer than ranks.
    kv_local = kv // world if kv >= world else 1
    if kv >= world and kv % world != 0:
        raise ValueError(f"`num_key_value_heads` ({kv}) must be divisible by `num_shards` ({world})")
    inter = cfg.get("intermediate_size", cfg.get("n_inner", cfg.get("ffn_hidden_size")))
    if inter is None:
        ffn = cfg.get("ffn_config") if isinstance(cfg.get("ffn_config"), dict) else {}
        inter = ffn.get("ffn_hidden_size", 4 * hidden)
    eps = cfg.get("rms_norm_eps", cfg.get("layer_norm_eps", cfg.get("layer_norm_epsilon", cfg.get("norm_epsilon", 1e-5))))
    act = arch.act or cfg.get("hidden_act", cfg.get("hidden_activation", cfg.get("activation_function", "gelu")))
    rope_params = cfg.get("rope_parameters") if isinstance(cfg.get("rope_parameters"), dict) else {}
    full = rope_params.get("full_attention") if isinstance(rope_params.get("full_attention"), dict) else {}
    attn_cfg = cfg.get("attn_config") if isinstance(cfg.get("attn_config"), dict) else {}
    theta = 10000.0
    for cand in (cfg.get("rope_theta"), rope_params.get("rope_theta"), full.get("rope_theta"), attn_cfg.get("rope_theta"),
                 cfg.get("rotary_emb_base")):
        if cand is not None:
            theta = float(cand)
            break
    partial = cfg.get("partial_rotary_factor", cfg.get("rotary_pct", 1.0))
    rot = cfg.get("rotary_dim")
    if arch.mla:
        rot = int(cfg.qk_rope_head_dim)
    if rot is None:
        rot = int(head_dim * partial)
    rot_dim = rot if arch.rope else 0
    max_pos = cfg.get("max_position_embeddings", cfg.get("n_positions", cfg.get("max_seq_len", 2048)))
    scalar = cfg.get("query_pre_attn_scalar")
    scale = (scalar ** -0.5) if scalar else head_dim ** -0.5
    if cfg.get("attention_multiplier"):
        scale = float(cfg.attention_multiplier)
    window = cfg.get("sliding_window")
    windows = [-1] * layers
    if window and cfg.get("use_sliding_window", True):
        if cfg.model_type == "gemma2":
            windows = [window if i % 2 == 0 else -1 for i in range(layers)]
        elif cfg.model_type in ("gemma3", "gemma3_text"):
            pat = cfg.get("sliding_window_pattern", 6)
            lt = cfg.get("layer_types")
            windows = [(window if (lt[i] == "sliding_attention" if lt else (i + 1) % pat != 0) else -1)
                       for i in range(layers)]
        elif cfg.model_type == "qwen2" and cfg.get("max_window_layers") is not None:
            windows = [window if i >= cfg.max_window_layers else -1 for i in range(layers)]
        else:
            windows = [window] * layers
    ne = cfg.get("num_local_experts", cfg.get("num_experts", cfg.get("n_routed_experts", 0))) or 0
    tk = cfg.get("num_experts_per_tok", cfg.get("moe_top_k", 0)) or 0
    if isinstance(cfg.get("ffn_config"), dict):
        ne = cfg.ffn_config.get("moe_num_experts", ne)
        tk = cfg.ffn_config.get("moe_top_k", tk)
    if arch.moe and cfg.get("moe_intermediate_size"):
        inter = cfg.moe_intermediate_size
    attn_dim = next((d for d in (64, 128, 256) if d >= head_dim), None)
    if attn_dim is None:
        raise ValueError(f"head dimension {head_dim} is larger than the attention kernels support (256)")
    return ModelDims(
        attn_head_dim=attn_dim,
        hidden=hidden, num_layers=layers, num_heads=heads // world, num_kv_heads=kv_local, head_dim=head_dim,
        intermediate=inter, vocab=cfg.get("vocab_size"), eps=float(eps), rope_theta=theta, rot_dim=rot_dim,
        max_positions=max_pos, act=act, softmax_scale=scale, windows=windows,
        attn_softcap=float(cfg.get("attn_logit_softcapping", 0.0) or 0.0),
        logit_softcap=float(cfg.get("final_logit_softcapping", 0.0) or 0.0),
        logit_scale=float(cfg.get("logit_scale", 1.0) or 1.0) / float(cfg.get("logits_scaling", 1.0) or 1.0),
        embed_scale=(math.sqrt(hidden) if arch.embed_scale_sqrt_hidden else float(cfg.get("embedding_multiplier", 1.0) or 1.0)),
        residual_scale=float(cfg.get("residual_multiplier", 1.0) or 1.0),
        num_experts=ne, top_k=tk, total_heads=heads, total_kv_heads=kv,
    )
