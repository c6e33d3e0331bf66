"""DeepSeek-V2 / V3 specifics: multi-head latent attention (MLA) and the routed-expert gate.

Reference: ``custom_modeling/flash_deepseek_v2_modeling.py`` / ``flash_deepseek_v3_modeling.py`` (MLA
expanded to padded multi-head attention ``:258-330``, group-limited routing and shared experts
``:473-489``).  Same approach here: the low-rank KV projection is expanded per head and the paged
attention kernels see ordinary heads of dimension 256:

    query head = [ q_rope (64) | q_nope (128) | 0 ... ]      key head = [ k_rope (64, shared by all heads) | k_nope (128) | 0 ... ]
    value head = [ v (128) | 0 ... ]

The rotary part is moved to the front so that the fused RoPE + KV-store kernel rotates the first
``qk_rope_head_dim`` elements of every query and key head; DeepSeek stores the rotary dimensions
interleaved, which is the kernel's non-NeoX mode.  A permutation applied to queries and keys alike
leaves the scores unchanged, and the zero padding contributes nothing.  The softmax scale is that of
the true head dimension (with the YaRN magnitude correction when the checkpoint asks for it).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from .. import ops
from .layers import FastLinear, TensorParallelColumnLinear, TensorParallelRowLinear, get_linear

MLA_HEAD_DIM = 256


def yarn_mscale(scale: float, mscale: float) -> float:
    return 1.0 if scale <= 1 else 0.1 * mscale * math.log(scale) + 1.0


def mla_softmax_scale(cfg) -> float:
    qk = int(cfg.qk_nope_head_dim) + int(cfg.qk_rope_head_dim)
    scale = qk ** -0.5
    rs = cfg.get("rope_scaling") or cfg.get("rope_parameters") or {}
    if isinstance(rs, dict) and rs.get("rope_type", rs.get("type", "default")) not in (None, "default"):
        m_all = rs.get("mscale_all_dim", 0)
        if m_all:
            m = yarn_mscale(float(rs.get("factor", 1.0)), float(m_all))
            scale = scale * m * m
    return scale


class MLAAttention:
    def __init__(self, arch, cfg, dims, prefix: str, weights, layer_idx: int, comm):
        pg = weights.process_group
        self.dims, self.layer_idx = dims, layer_idx
        self.nope, self.rope_dim, self.v_dim = int(cfg.qk_nope_head_dim), int(cfg.qk_rope_head_dim), int(cfg.v_head_dim)
        self.rank_kv = int(cfg.kv_lora_rank)
        assert self.nope + self.rope_dim <= MLA_HEAD_DIM and self.v_dim <= MLA_HEAD_DIM
        self.heads = dims.num_heads
        p = f"{prefix}.self_attn"
        self.q_a = self.q_a_norm = None
        if cfg.get("q_lora_rank"):
            self.q_a = FastLinear(weights.get_tensor(f"{p}.q_a_proj.weight"),
                                  weights.get_tensor(f"{p}.q_a_proj.bias") if weights.has_tensor(f"{p}.q_a_proj.bias") else None)
            self.q_a_norm = weights.get_tensor(f"{p}.q_a_layernorm.weight")
            self.q_b = TensorParallelColumnLinear.load(cfg, f"{p}.q_b_proj", weights, False)
        else:
            self.q_b = TensorParallelColumnLinear.load(cfg, f"{p}.q_proj", weights, False)
        self.kv_a = FastLinear(weights.get_tensor(f"{p}.kv_a_proj_with_mqa.weight"),
                               weights.get_tensor(f"{p}.kv_a_proj_with_mqa.bias")
                               if weights.has_tensor(f"{p}.kv_a_proj_with_mqa.bias") else None)
        self.kv_a_norm = weights.get_tensor(f"{p}.kv_a_layernorm.weight")
        self.kv_b = TensorParallelColumnLinear.load(cfg, f"{p}.kv_b_proj", weights, False)
        self.o = TensorParallelRowLinear.load(cfg, f"{p}.o_proj", weights, weights.has_tensor(f"{p}.o_proj.bias"), comm)
        self.eps = dims.eps
        self.scale = mla_softmax_scale(cfg)
        self.window = -1
        self.k_scale = self.v_scale = None
        self.qkv = None          # no fused qkv projection: the layer keeps its input un-quantised

    def _linear(self, lin, x):
        return lin(x)

    def __call__(self, x, x_scale, meta, rotary, kv, reduce: bool = True, out=None):
        assert x_scale is None
        T, Hl = x.shape[0], self.heads
        if self.q_a is not None:
            qa = self.q_a(x)
            qa, _ = ops.rms_norm(qa, None, self.q_a_norm, self.eps)
            q = self.q_b(qa)
        else:
            q = self.q_b(x)
        q = q.view(T, Hl, self.nope + self.rope_dim)
        ckv = self.kv_a(x)
        latent, k_pe = ckv[:, : self.rank_kv].contiguous(), ckv[:, self.rank_kv:]
        latent, _ = ops.rms_norm(latent, None, self.kv_a_norm, self.eps)
        kvb = self.kv_b(latent).view(T, Hl, self.nope + self.v_dim)
        D = MLA_HEAD_DIM
        fused = x.new_zeros(T, 3 * Hl, D)
        fused[:, :Hl, : self.rope_dim] = q[..., self.nope:]
        fused[:, :Hl, self.rope_dim: self.rope_dim + self.nope] = q[..., : self.nope]
        fused[:, Hl:2 * Hl, : self.rope_dim] = k_pe.unsqueeze(1)
        fused[:, Hl:2 * Hl, self.rope_dim: self.rope_dim + self.nope] = kvb[..., : self.nope]
        fused[:, 2 * Hl:, : self.v_dim] = kvb[..., self.nope:]
        k_cache, v_cache = kv
        qr = ops.rope_and_cache(fused.view(T, 3 * Hl * D), meta.positions, rotary.cos_sin, meta.slots, k_cache, v_cache,
                                Hl, Hl, D, self.rope_dim, False, self.k_scale, self.v_scale)
        attn = ops.paged_attention(qr, k_cache, v_cache, meta.block_tables, meta.cu_seqlens_q, meta.kv_lens, self.scale,
                                   -1, 0.0, None, None, meta.max_q, meta.max_kv)
        attn = attn.view(T, Hl, D)[:, :, : self.v_dim].reshape(T, Hl * self.v_dim)
        return self.o(attn, reduce=reduce, out=out)


class DeepseekRouter:
    """Expert selection of DeepSeek-V2 (softmax scores, optional group-limited greedy) and V3 (sigmoid
    scores, selection on bias-corrected scores with group limitation, weights from the raw scores)."""

    def __init__(self, cfg, weights, prefix: str):
        self.v3 = cfg.model_type == "deepseek_v3"
        self.top_k = int(cfg.num_experts_per_tok)
        self.n_group = int(cfg.get("n_group") or 1)
        self.topk_group = int(cfg.get("topk_group") or 1)
        self.scale = float(cfg.get("routed_scaling_factor") or 1.0)
        self.norm = bool(cfg.get("norm_topk_prob", False))
        self.method = cfg.get("topk_method", "noaux_tc" if self.v3 else "greedy")
        self.bias = None
        if weights.has_tensor(f"{prefix}.gate.e_score_correction_bias"):
            self.bias = weights.get_tensor(f"{prefix}.gate.e_score_correction_bias", to_dtype=False).float()

    def __call__(self, logits: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        x = logits.float()
        T, E = x.shape
        if self.v3:
            scores = torch.sigmoid(x)
            choice = scores + self.bias if self.bias is not None else scores
            if self.n_group > 1:
                g = choice.view(T, self.n_group, E // self.n_group)
                group_scores = g.topk(2, dim=-1)[0].sum(-1)
                keep = torch.zeros_like(group_scores).scatter_(1, group_scores.topk(self.topk_group, dim=-1)[1], 1.0)
                choice = choice.masked_fill(keep.unsqueeze(-1).expand_as(g).reshape(T, E) == 0, 0.0)
            idx = choice.topk(self.top_k, dim=-1)[1]
            w = scores.gather(1, idx)
            if self.norm:
                w = w / (w.sum(-1, keepdim=True) + 1e-20)
            return w * self.scale, idx
        scores = torch.softmax(x, dim=-1)
        if self.method == "group_limited_greedy" and self.n_group > 1:
            g = scores.view(T, self.n_group, E // self.n_group)
            group_scores = g.max(-1)[0]
            keep = torch.zeros_like(group_scores).scatter_(1, group_scores.topk(self.topk_group, dim=-1)[1], 1.0)
            masked = scores.masked_fill(keep.unsqueeze(-1).expand_as(g).reshape(T, E) == 0, 0.0)
            w, idx = masked.topk(self.top_k, dim=-1)
        else:
            w, idx = scores.topk(self.top_k, dim=-1)
        if self.top_k > 1 and self.norm:
            w = w / (w.sum(-1, keepdim=True) + 1e-20)
        return w * self.scale, idx


def is_moe_layer(cfg, idx: int) -> bool:
    if not cfg.get("n_routed_experts"):
        return False
    return idx >= int(cfg.get("first_k_dense_replace", 0) or 0) and idx % int(cfg.get("moe_layer_freq", 1) or 1) == 0
