"""Generic paged-KV decoder: every supported causal LM family runs through this file.

Reference structure being covered: ``custom_modeling/flash_llama_modeling.py`` (attention
``:137-267``, MLP ``:306-404``, layer ``:407-500``, model ``:503-614``, head ``:617-703``) and
its siblings for the other families.  The forward pass works on *ragged* batches (``T`` tokens,
no padding) and is a flat sequence of fused ops:

    embed -> L x [ add+norm(+quant) -> qkv GEMM -> RoPE+KV-store -> paged attention -> o GEMM(+reduce)
                   -> add+norm(+quant) -> gate_up GEMM -> act*mul(+quant) -> down GEMM(+reduce) ]
          -> add+norm -> gather last tokens -> lm_head

The residual stream is carried un-normalised and folded into the next norm kernel, logits are
computed only for the rows in ``lm_head_indices``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import torch

from .. import ops
from ..utils.rotary import RotaryTable
from .arch import Arch, ModelConfig, ModelDims, arch_for, derive_dims
from .layers import (
    FastLinear,
    Fp8Linear,
    TensorParallelColumnLinear,
    TensorParallelEmbedding,
    TensorParallelHead,
    TensorParallelRowLinear,
    get_linear,
)


@dataclass
class ForwardMeta:
    """Per-step device tensors describing the ragged batch (all int32)."""

    input_ids: torch.Tensor            # [T]
    positions: torch.Tensor            # [T]
    slots: torch.Tensor                # [T] KV slot of every token of the step
    block_tables: torch.Tensor         # [B, max_blocks]
    cu_seqlens_q: torch.Tensor         # [B+1]
    kv_lens: torch.Tensor              # [B] cached + current tokens
    max_q: int
    max_kv: int
    lm_head_indices: Optional[torch.Tensor] = None   # rows of the hidden state that need logits
    inputs_embeds: Optional[torch.Tensor] = None     # overrides the embedding lookup (VLM)
    adapter_data: Optional[object] = None            # LoRA batch metadata
    rope_cos_sin: Optional[torch.Tensor] = None      # [T, rot_dim] rotary rows of this step (multi-axis positions)
    rope_rows: Optional[torch.Tensor] = None         # [T] = arange(T): row of `rope_cos_sin` per token
    attn_horizon: Optional[torch.Tensor] = None      # [T] last KV position a row may see (image rows: end of their image)
    cross: Optional[object] = None                   # rows and image states for cross-attention layers (models/mllama.py)


class Norm:
    def __init__(self, kind: str, weight, bias, eps: float, unit_offset: bool):
        self.kind, self.weight, self.bias, self.eps, self.unit_offset = kind, weight, bias, eps, unit_offset

    @classmethod
    def load(cls, arch: Arch, prefix: str, weights, eps: float):
        w = weights.get_tensor(f"{prefix}.weight")
        b = None
        if arch.norm == "layer" and arch.norm_bias and weights.has_tensor(f"{prefix}.bias"):
            b = weights.get_tensor(f"{prefix}.bias")
        return cls(arch.norm, w, b, eps, arch.norm_unit_offset)

    def __call__(self, x, residual=None):
        if self.kind == "rms":
            return ops.rms_norm(x, residual, self.weight, self.eps, self.unit_offset)
        return ops.layer_norm(x, residual, self.weight, self.bias, self.eps)

    def quant(self, x, residual=None):
        """Fused add + RMSNorm + 1x128 fp8 quantisation -> ``(xq, scales, residual)``."""
        return ops.rms_norm_quant(x, residual, self.weight, self.eps, self.unit_offset)

    @property
    def can_quant(self):
        return self.kind == "rms" and self.weight.shape[0] % 128 == 0


def _maybe_T(w: torch.Tensor, arch: Arch) -> torch.Tensor:
    return w.t().contiguous() if arch.conv1d_weights else w


def _rows_for_rank(total_heads: int, total_kv: int, head_dim: int, layout: str, rank: int, world: int):
    """Row indices (into the checkpoint's fused qkv matrix) that form ``[q_r | k_r | v_r]`` for ``rank``."""
    D = head_dim
    hq, hkv = total_heads // world, (total_kv // world if total_kv >= world else 1)
    q_heads = range(rank * hq, (rank + 1) * hq)
    kv_heads = range(rank * hkv, (rank + 1) * hkv) if total_kv >= world else [rank * total_kv // world]
    ar = torch.arange(D)
    q_rows, k_rows, v_rows = [], [], []
    if layout == "blocked":
        for h in q_heads:
            q_rows.append(h * D + ar)
        for h in kv_heads:
            k_rows.append(total_heads * D + h * D + ar)
            v_rows.append((total_heads + total_kv) * D + h * D + ar)
    elif layout == "interleaved":  # [head, (q,k,v), D]; requires total_kv == total_heads
        for h in q_heads:
            q_rows.append((h * 3 + 0) * D + ar)
            k_rows.append((h * 3 + 1) * D + ar)
            v_rows.append((h * 3 + 2) * D + ar)
    elif layout == "falcon":  # [kv_group, (q x per_group, k, v), D]
        per = total_heads // total_kv
        for h in q_heads:
            g, j = divmod(h, per)
            q_rows.append((g * (per + 2) + j) * D + ar)
        for g in kv_heads:
            k_rows.append((g * (per + 2) + per) * D + ar)
            v_rows.append((g * (per + 2) + per + 1) * D + ar)
    else:
        raise ValueError(layout)
    return torch.cat(q_rows + k_rows + v_rows)


class Attention:
    def __init__(self, arch: Arch, cfg: ModelConfig, dims: ModelDims, prefix: str, weights, layer_idx: int, comm):
        self.arch, self.dims, self.layer_idx = arch, dims, layer_idx
        pg = weights.process_group
        D = dims.head_dim
        if arch.qkv is None:
            names = [f"{prefix}.{arch.q}", f"{prefix}.{arch.k}", f"{prefix}.{arch.v}"]
            if dims.total_kv_heads < pg.size():
                # fewer KV heads than ranks: shard q, replicate the owning KV head
                self.qkv = self._load_replicated_kv(cfg, names, weights, arch.qkv_bias)
            else:
                self.qkv = TensorParallelColumnLinear.load_multi(
                    cfg, names, weights, arch.qkv_bias and weights.has_tensor(f"{names[0]}.bias"))
        else:
            name = f"{prefix}.{arch.qkv}"
            simple = (arch.qkv_layout == "blocked" and not arch.conv1d_weights
                      and dims.total_kv_heads >= pg.size())
            if simple:
                self.qkv = TensorParallelColumnLinear.load_qkv(
                    cfg, name, weights, arch.qkv_bias and weights.has_tensor(f"{name}.bias"),
                    dims.total_heads * D, dims.total_kv_heads * D)
            else:
                layout = arch.qkv_layout
                w = _maybe_T(weights.get_tensor(f"{name}.weight"), arch)
                rows = _rows_for_rank(dims.total_heads, dims.total_kv_heads, D, layout, pg.rank(), pg.size()).to(w.device)
                b = None
                if arch.qkv_bias and weights.has_tensor(f"{name}.bias"):
                    b = weights.get_tensor(f"{name}.bias")[rows].contiguous()
                self.qkv = TensorParallelColumnLinear(FastLinear(w[rows].contiguous(), b))
        o_name = f"{prefix}.{arch.o}"
        o_bias = arch.o_bias and weights.has_tensor(f"{o_name}.bias")
        if arch.conv1d_weights:
            w = weights.get_sharded(f"{o_name}.weight", dim=0).t().contiguous()
            b = weights.get_tensor(f"{o_name}.bias") if o_bias and pg.rank() == 0 else None
            self.o = TensorParallelRowLinear(FastLinear(w, b), pg, comm)
        else:
            self.o = TensorParallelRowLinear.load(cfg, o_name, weights, o_bias, comm)
        self.q_norm = self.k_norm = None
        if arch.q_norm and weights.has_tensor(f"{prefix}.{arch.q_norm}.weight"):
            qn = weights.get_tensor(f"{prefix}.{arch.q_norm}.weight")
            kn = weights.get_tensor(f"{prefix}.{arch.k_norm}.weight")
            if arch.qk_norm_kind == "layer":  # cohere: per-head weights [heads, D], sharded over heads
                qn = qn.view(dims.total_heads, D)[pg.rank() * dims.num_heads:(pg.rank() + 1) * dims.num_heads]
                kn = kn.view(dims.total_kv_heads, D)[pg.rank() * dims.num_kv_heads:(pg.rank() + 1) * dims.num_kv_heads]
            self.q_norm, self.k_norm = qn.contiguous(), kn.contiguous()
        self.window = dims.windows[layer_idx]
        ac = cfg.get("attn_config")
        self.clip_qkv = float(ac.get("clip_qkv") or 0.0) if isinstance(ac, dict) else float(cfg.get("clip_qkv") or 0.0)
        self.k_scale = self.v_scale = None
        for kname, vname in ((f"{prefix}.self_attn.k_scale", f"{prefix}.self_attn.v_scale"),
                             (f"{prefix}.self_attn.kv_scale", f"{prefix}.self_attn.kv_scale")):
            if weights.has_tensor(kname):
                ks = weights.get_tensor(kname, to_dtype=False).float().reshape(-1)
                vs = weights.get_tensor(vname, to_dtype=False).float().reshape(-1)
                self.k_scale = ks.expand(dims.num_kv_heads).contiguous() if ks.numel() == 1 else ks
                self.v_scale = vs.expand(dims.num_kv_heads).contiguous() if vs.numel() == 1 else vs
                break
        self.alibi_slopes = None

    @staticmethod
    def _load_replicated_kv(cfg, names, weights, bias):
        pg = weights.process_group
        qw = weights.get_sharded(f"{names[0]}.weight", dim=0)
        parts_w, parts_b = [qw], []
        if bias:
            parts_b.append(weights.get_sharded(f"{names[0]}.bias", dim=0))
        for n in names[1:]:
            full = weights.get_tensor(f"{n}.weight")
            total_kv_rows = full.shape[0]
            # owner head for this rank
            heads_kv = cfg.get("num_key_value_heads", 1) or 1
            D = total_kv_rows // heads_kv
            h = pg.rank() * heads_kv // pg.size()
            parts_w.append(full[h * D:(h + 1) * D])
            if bias:
                parts_b.append(weights.get_tensor(f"{n}.bias")[h * D:(h + 1) * D])
        return TensorParallelColumnLinear(FastLinear(torch.cat(parts_w, 0).contiguous(),
                                                     torch.cat(parts_b, 0).contiguous() if bias else None))

    def _qk_norm(self, qkv: torch.Tensor) -> torch.Tensor:
        d = self.dims
        T = qkv.shape[0]
        if qkv.is_cuda and qkv.dtype == torch.bfloat16 and d.head_dim <= 256 and d.head_dim % 2 == 0:
            from ..ops import cuda as K

            return K.qk_norm(qkv, d.num_heads, d.num_kv_heads, d.head_dim, self.q_norm, self.k_norm, d.eps,
                             self.arch.qk_norm_kind == "rms" and self.arch.norm_unit_offset,
                             layer=self.arch.qk_norm_kind != "rms")
        nq, nk = d.num_heads * d.head_dim, d.num_kv_heads * d.head_dim
        q = qkv[:, :nq].reshape(T, d.num_heads, d.head_dim)
        k = qkv[:, nq:nq + nk].reshape(T, d.num_kv_heads, d.head_dim)
        if self.arch.qk_norm_kind == "rms":
            off = self.arch.norm_unit_offset
            q, _ = ops.ref.rms_norm(q, None, self.q_norm, d.eps, off)
            k, _ = ops.ref.rms_norm(k, None, self.k_norm, d.eps, off)
        else:
            qf, kf = q.float(), k.float()
            q = ((qf - qf.mean(-1, keepdim=True)) * torch.rsqrt(qf.var(-1, unbiased=False, keepdim=True) + d.eps)
                 * self.q_norm.float()).to(qkv.dtype)
            k = ((kf - kf.mean(-1, keepdim=True)) * torch.rsqrt(kf.var(-1, unbiased=False, keepdim=True) + d.eps)
                 * self.k_norm.float()).to(qkv.dtype)
        return torch.cat([q.reshape(T, nq), k.reshape(T, nk), qkv[:, nq + nk:]], dim=-1)

    def __call__(self, x, x_scale, meta: ForwardMeta, rotary: RotaryTable, kv, reduce: bool = True, out=None):
        d = self.dims
        qkv = self.qkv(x, x_scale)
        if self.clip_qkv:
            qkv = qkv.clamp(-self.clip_qkv, self.clip_qkv)     # DBRX
        if meta.adapter_data is not None:
            qkv = meta.adapter_data.apply_qkv(self.layer_idx, x, qkv)
        if self.q_norm is not None:
            qkv = self._qk_norm(qkv)
        k_cache, v_cache = kv
        D = d.head_dim
        Dp = d.attn_head_dim or D
        if Dp != D:
            # head dimensions the attention kernels have no instance for (80, 96, 160, ...) run zero-padded
            # to the next one; the rotary part stays at the front and the scale is that of the true dimension
            T_ = qkv.shape[0]
            qkv = torch.nn.functional.pad(qkv.view(T_, d.num_heads + 2 * d.num_kv_heads, D), (0, Dp - D)).view(T_, -1)
        rope_pos, rope_tab = meta.positions, rotary.cos_sin
        if meta.rope_cos_sin is not None and rotary.mrope_section:
            rope_pos, rope_tab = meta.rope_rows, meta.rope_cos_sin     # rows prepared per token (Qwen2-VL)
        q = ops.rope_and_cache(qkv, rope_pos, rope_tab, meta.slots, k_cache, v_cache,
                               d.num_heads, d.num_kv_heads, Dp, rotary.rot_dim, rotary.neox,
                               self.k_scale, self.v_scale)
        attn = ops.paged_attention(q, k_cache, v_cache, meta.block_tables, meta.cu_seqlens_q, meta.kv_lens,
                                   d.softmax_scale, self.window, d.attn_softcap,
                                   self.k_scale if k_cache.dtype == torch.float8_e4m3fn else None,
                                   self.v_scale if v_cache.dtype == torch.float8_e4m3fn else None,
                                   meta.max_q, meta.max_kv, horizon=meta.attn_horizon)
        if Dp != D:
            attn = attn.view(attn.shape[0], d.num_heads, Dp)[:, :, :D]
        attn = attn.reshape(attn.shape[0], d.num_heads * D)
        out = self.o(attn, reduce=reduce, out=out)
        if meta.adapter_data is not None:
            out = meta.adapter_data.apply_row(self.layer_idx, "o_proj", attn, out)
        return out


class DenseMLP:
    def __init__(self, arch: Arch, cfg, dims: ModelDims, prefix: str, weights, comm, layer_idx: int = 0,
                 names: Optional[Tuple[str, str, str]] = None):
        self.act = dims.act
        self.gated = arch.gated_mlp
        self.layer_idx = layer_idx
        pg = weights.process_group
        gate, up, down = names or (arch.gate, arch.up, arch.down)
        bias = arch.mlp_bias
        if arch.gate_up is not None and names is None:
            self.gate_up = TensorParallelColumnLinear.load_gate_up(cfg, f"{prefix}.{arch.gate_up}", weights, bias)
        elif self.gated:
            self.gate_up = TensorParallelColumnLinear.load_multi(
                cfg, [f"{prefix}.{gate}", f"{prefix}.{up}"], weights, bias)
        elif arch.conv1d_weights:
            w = weights.get_sharded(f"{prefix}.{up}.weight", dim=1).t().contiguous()
            b = weights.get_sharded(f"{prefix}.{up}.bias", dim=0) if bias else None
            self.gate_up = TensorParallelColumnLinear(FastLinear(w, b))
        else:
            self.gate_up = TensorParallelColumnLinear.load(
                cfg, f"{prefix}.{up}", weights, bias and weights.has_tensor(f"{prefix}.{up}.bias"))
        if arch.conv1d_weights:
            w = weights.get_sharded(f"{prefix}.{down}.weight", dim=0).t().contiguous()
            b = weights.get_tensor(f"{prefix}.{down}.bias") if bias and pg.rank() == 0 else None
            self.down = TensorParallelRowLinear(FastLinear(w, b), pg, comm)
        else:
            self.down = TensorParallelRowLinear.load(
                cfg, f"{prefix}.{down}", weights, bias and weights.has_tensor(f"{prefix}.{down}.bias"), comm)
        lin = self.down.linear
        self.down_quant = isinstance(lin, Fp8Linear) and lin.wants_quantized_input and self.gated

    def __call__(self, x, x_scale=None, reduce: bool = True, meta: Optional[ForwardMeta] = None, out=None):
        h = self.gate_up(x, x_scale)
        if meta is not None and meta.adapter_data is not None:
            h = meta.adapter_data.apply_gate_up(self.layer_idx, x, h)
        if self.gated:
            if self.down_quant and (meta is None or meta.adapter_data is None):
                hq, hs = ops.act_and_mul_quant(h, self.act)
                return self.down(hq, hs, reduce=reduce, out=out)
            a = ops.act_and_mul(h, self.act)
        else:
            a = ops.activation(h, self.act).to(h.dtype)
        out = self.down(a, reduce=reduce, out=out)
        if meta is not None and meta.adapter_data is not None:
            out = meta.adapter_data.apply_row(self.layer_idx, "down_proj", a, out)
        return out


def _expert_weight(weights, cfg, name: str, dim: Optional[int] = None) -> torch.Tensor:
    """One expert projection (``name`` without ``.weight``), whole (``dim=None``) or this rank's slice along ``dim``,
    in the serving dtype.  Experts of fp8 checkpoints — 128 x 128 ``weight_scale_inv`` blocks, or a per-tensor /
    per-channel ``weight_scale`` — are dequantised here: the grouped expert GEMM (``ops/csrc/moe_sm100.cu``) runs in
    bf16, where the reference keeps such experts in fp8 (``layers/moe/fp8.py:20-92``)."""
    from ..utils.weights import shard_bounds

    fp8 = getattr(torch, "float8_e4m3fn", None)
    if not weights.has_tensor(f"{name}.weight"):
        # packed integer experts (GPTQ / AWQ `qweight`, compressed-tensors `weight_packed`): dequantised through the
        # checkpoint's loader, like the fp8 ones (the reference serves them with a Marlin MoE kernel,
        # ``layers/moe/gptq_marlin.py``)
        qw = weights.weights_loader.get_weights(weights, name)
        w = qw.dequantize().to(weights.dtype) if hasattr(qw, "dequantize") else qw.weight.to(weights.dtype)
        if dim is not None:
            lo, hi = shard_bounds(w.shape[dim], weights.process_group.rank(), weights.process_group.size())
            w = w.narrow(dim, lo, hi - lo).contiguous()
        return w
    full = weights.get_tensor(f"{name}.weight", to_dtype=False)
    if fp8 is None or full.dtype != fp8:
        return weights.get_tensor(f"{name}.weight") if dim is None else weights.get_sharded(f"{name}.weight", dim=dim)
    N, K = full.shape
    if weights.has_tensor(f"{name}.weight_scale_inv"):
        q = cfg.get("quantization_config") or {}
        blk = list(q.get("weight_block_size") or [128, 128])
        s = weights.get_tensor(f"{name}.weight_scale_inv", to_dtype=False).float()
        s = s.repeat_interleave(blk[0], 0)[:N].repeat_interleave(blk[1], 1)[:, :K]
    else:
        s = weights.get_tensor(f"{name}.weight_scale", to_dtype=False).float()
        s = s.reshape(-1, 1) if s.numel() > 1 else s.reshape(1, 1)
    w = (full.float() * s.to(full.device)).to(weights.dtype)
    if dim is not None:
        lo, hi = shard_bounds(w.shape[dim], weights.process_group.rank(), weights.process_group.size())
        w = w.narrow(dim, lo, hi - lo).contiguous()
    return w


class SparseMoE:
    """Top-k routed experts.  Tensor-parallel mode slices every expert's intermediate dimension
    (what the reference does, ``layers/moe/unquantized.py:107-163``); expert-parallel mode
    (``parallel/expert.py``) places whole experts on ranks.  Either way a rank ends up with a partial
    ``[T, H]`` output that is summed over ranks by the layer's reduction."""

    def __init__(self, arch: Arch, cfg, dims: ModelDims, prefix: str, weights, comm):
        pg = weights.process_group
        self.pg, self.comm = pg, comm
        self.top_k, self.num_experts, self.act = dims.top_k, dims.num_experts, dims.act
        self.renorm = arch.moe_renormalize if cfg.get("norm_topk_prob") is None else bool(cfg.norm_topk_prob)
        self.router = FastLinear(weights.get_tensor(f"{prefix}.{arch.moe_router}.weight"))
        self.sparsemixer_eps = float(cfg.get("router_jitter_noise", 0.01)) if cfg.model_type == "phimoe" else None
        self.deepseek_router = None
        if arch.mla:
            from .deepseek import DeepseekRouter

            self.deepseek_router = DeepseekRouter(cfg, weights, f"{prefix}.mlp")
        E = dims.num_experts
        gu, dn = [], []
        from ..parallel.expert import ExpertParallel, local_expert_range, wants_expert_parallel

        self.expert_parallel = None
        if not arch.moe_fused and wants_expert_parallel(E, pg.size()):
            # whole experts on their owner rank (no slicing); see parallel/expert.py
            lo, hi = local_expert_range(E, pg.rank(), pg.size())
            for e in range(lo, hi):
                ep = f"{prefix}.{arch.moe_expert.format(e=e)}"
                gu.append(torch.cat([_expert_weight(weights, cfg, f"{ep}.{arch.moe_gate}"),
                                     _expert_weight(weights, cfg, f"{ep}.{arch.moe_up}")], dim=0))
                dn.append(_expert_weight(weights, cfg, f"{ep}.{arch.moe_down}"))
            self.w_gate_up = torch.stack(gu).contiguous()   # [E / world, 2I, H]
            self.w_down = torch.stack(dn).contiguous()       # [E / world, H, I]
            self.expert_parallel = ExpertParallel(self.w_gate_up, self.w_down, lo, self.act)
        elif arch.moe_fused:  # dbrx: [E*I, H] stacked
            ep = f"{prefix}.{arch.moe_expert}"
            I = dims.intermediate
            w1 = weights.get_tensor(f"{ep}.{arch.moe_gate}").view(E, I, dims.hidden)
            v1 = weights.get_tensor(f"{ep}.{arch.moe_up}").view(E, I, dims.hidden)
            w2 = weights.get_tensor(f"{ep}.{arch.moe_down}").view(E, I, dims.hidden)
            per = I // pg.size()
            sl = slice(pg.rank() * per, (pg.rank() + 1) * per)
            self.w_gate_up = torch.cat([w1[:, sl], v1[:, sl]], dim=1).contiguous()
            self.w_down = w2[:, sl].transpose(1, 2).contiguous()
        else:
            for e in range(E):
                ep = f"{prefix}.{arch.moe_expert.format(e=e)}"
                g = _expert_weight(weights, cfg, f"{ep}.{arch.moe_gate}", dim=0)
                u = _expert_weight(weights, cfg, f"{ep}.{arch.moe_up}", dim=0)
                gu.append(torch.cat([g, u], dim=0))
                dn.append(_expert_weight(weights, cfg, f"{ep}.{arch.moe_down}", dim=1))
            self.w_gate_up = torch.stack(gu).contiguous()   # [E, 2I/tp, H]
            self.w_down = torch.stack(dn).contiguous()       # [E, H, I/tp]
        self.shared = None
        self.shared_gate = None
        if arch.moe_shared and weights.has_tensor(f"{prefix}.{arch.moe_shared}.gate_proj.weight"):
            self.shared = DenseMLP(arch, cfg, dims, f"{prefix}.{arch.moe_shared}", weights, comm,
                                   names=("gate_proj", "up_proj", "down_proj"))
            if arch.moe_shared_gate and weights.has_tensor(f"{prefix}.{arch.moe_shared_gate}.weight"):
                self.shared_gate = FastLinear(weights.get_tensor(f"{prefix}.{arch.moe_shared_gate}.weight"))

    def __call__(self, x, x_scale=None, reduce: bool = True, meta=None, out=None):
        if out is not None:
            out.copy_(self(x, x_scale, reduce=False, meta=meta))
            return out
        logits = self.router(x)
        if self.deepseek_router is not None:
            w, idx = self.deepseek_router(logits)
        elif self.sparsemixer_eps is not None:
            w, idx = ops.moe_sparsemixer(logits, self.sparsemixer_eps)       # Phi-3.5-MoE routing
        else:
            w, idx = ops.moe_topk_softmax(logits, self.top_k, self.renorm)
        if self.expert_parallel is not None:
            out = self.expert_parallel(x, w, idx)
        else:
            # routed rows only: grouped kernels on CUDA (no host synchronisation, graph capturable), loop on CPU
            out = ops.moe_experts(x, self.w_gate_up, self.w_down, w, idx, self.act)
        if self.shared is not None:
            s = self.shared(x, reduce=False)
            if self.shared_gate is not None:
                s = s * torch.sigmoid(self.shared_gate(x).float()).to(s.dtype)
            out = out + s
        if reduce and self.pg.size() > 1:   # tensor-parallel slices and expert-parallel rows both sum over ranks
            out = self.comm.all_reduce(out) if self.comm is not None else _all_reduce(out, self.pg)
        return out


def _all_reduce(t, pg):
    from ..parallel import dist as pdist

    return pdist.all_reduce(t, pg)


class DecoderLayer:
    def __init__(self, arch: Arch, cfg, dims: ModelDims, prefix: str, weights, idx: int, comm):
        self.arch, self.dims = arch, dims
        if cfg.model_type in ("falcon", "RefinedWeb", "RefinedWebModel"):
            # the new decoder architecture names its norms ln_attn / ln_mlp and has no input_layernorm
            self.norm1, self.norm2 = self._falcon_norms(arch, cfg, prefix, weights, dims)
        else:
            self.norm1 = Norm.load(arch, f"{prefix}.{arch.norm1}", weights, dims.eps)
            self.norm2 = Norm.load(arch, f"{prefix}.{arch.norm2}", weights, dims.eps) if arch.norm2 else None
        self.post_attn = Norm.load(arch, f"{prefix}.{arch.post_attn_norm}", weights, dims.eps) if arch.post_attn_norm else None
        self.post_mlp = Norm.load(arch, f"{prefix}.{arch.post_mlp_norm}", weights, dims.eps) if arch.post_mlp_norm else None
        if arch.mla:
            from .deepseek import MLAAttention, is_moe_layer

            self.attn = MLAAttention(arch, cfg, dims, prefix, weights, idx, comm)
            is_moe = is_moe_layer(cfg, idx)      # the first layers of DeepSeek models are dense
        else:
            self.attn = Attention(arch, cfg, dims, prefix, weights, idx, comm)
            is_moe = arch.moe
        if is_moe and cfg.get("mlp_only_layers") and idx in cfg.mlp_only_layers:
            is_moe = False
        self.mlp = (SparseMoE(arch, cfg, dims, prefix, weights, comm) if is_moe
                    else DenseMLP(arch, cfg, dims, prefix, weights, comm, idx))
        self.pg, self.comm = weights.process_group, comm
        qlin = getattr(getattr(self.attn, "qkv", None), "linear", None)
        self.attn_in_quant = isinstance(qlin, Fp8Linear) and qlin.wants_quantized_input and self.norm1.can_quant
        glin = getattr(getattr(self.mlp, "gate_up", None), "linear", None)
        self.mlp_in_quant = (isinstance(glin, Fp8Linear) and glin.wants_quantized_input
                             and self.norm2 is not None and self.norm2.can_quant)

    @staticmethod
    def _falcon_norms(arch, cfg, prefix, weights, dims):
        if cfg.get("new_decoder_architecture") and (cfg.get("num_ln_in_parallel_attn") or 2) == 2 \
                and weights.has_tensor(f"{prefix}.ln_attn.weight"):
            return (Norm.load(arch, f"{prefix}.ln_attn", weights, dims.eps),
                    Norm.load(arch, f"{prefix}.ln_mlp", weights, dims.eps))
        return Norm.load(arch, f"{prefix}.input_layernorm", weights, dims.eps), None

    def __call__(self, h, residual, meta: ForwardMeta, rotary, kv):
        a = self.arch
        rs = self.dims.residual_scale
        if a.parallel_residual:
            normed, residual = self.norm1(h, residual)
            # attention and MLP partial sums of a parallel block share one reduction
            attn = self.attn(normed, None, meta, rotary, kv, reduce=False)
            if self.norm2 is not None:
                mlp_in, _ = self.norm2(residual, None)
            else:
                mlp_in = normed
            mlp = self.mlp(mlp_in, reduce=False, meta=meta)
            out = attn + mlp
            if self.pg.size() > 1:
                out = self.comm.all_reduce(out) if self.comm is not None else _all_reduce(out, self.pg)
            return out, residual
        if self.attn_in_quant and meta.adapter_data is None:
            xq, xs, residual = self.norm1.quant(h, residual)
            attn = self.attn(xq, xs, meta, rotary, kv)
        else:
            normed, residual = self.norm1(h, residual)
            attn = self.attn(normed, None, meta, rotary, kv)
        if self.post_attn is not None:
            attn, _ = self.post_attn(attn, None)
        if rs != 1.0:
            attn = attn * rs
        if self.mlp_in_quant and meta.adapter_data is None:
            xq, xs, residual = self.norm2.quant(attn, residual)
            mlp = self.mlp(xq, xs, meta=meta)
        else:
            normed, residual = self.norm2(attn, residual)
            mlp = self.mlp(normed, meta=meta)
        if self.post_mlp is not None:
            mlp, _ = self.post_mlp(mlp, None)
        if rs != 1.0:
            mlp = mlp * rs
        return mlp, residual

    @property
    def fusable_tp(self) -> bool:
        """True when the layer is a plain pre-norm block whose two reductions can each be fused with
        the residual add and the following RMSNorm."""
        a = self.arch
        return (not a.parallel_residual and a.norm == "rms" and self.norm2 is not None and self.post_attn is None
                and self.post_mlp is None and self.dims.residual_scale == 1.0)

    def fused_tp(self, x, meta: ForwardMeta, rotary, kv, next_norm: Norm, next_quant: bool, comm):
        """Tensor-parallel layer on peer memory.  ``x`` is this layer's *normalised* input (a tensor or
        ``(xq, scales)``); returns the normalised input of the next layer in the same form.  Both
        row-parallel GEMMs write their partial sums into the peer buffer, and one kernel per
        reduction sums them across ranks, adds the residual stream kept by the row's owner, applies
        the next RMSNorm (and quantises) and gathers the result on every rank."""
        T = meta.input_ids.shape[0]
        xq, xs = x if isinstance(x, tuple) else (x, None)
        # o_proj and down_proj store their partial rows straight into the row owners' peer memory
        # (GEMM epilogue = reduce-scatter transport); producers without such an epilogue use the
        # plain buffer and the reduction pulls instead.
        # Measured on B200: below a few hundred rows the scattered peer stores and the system-scope
        # fences of the pushing epilogue cost more than the pull they replace (decode step 34.5 ms
        # pulled vs 37.3 ms pushed at TP=2), so small batches pull and prefill-sized ones push.
        push = hasattr(comm, "push_target") and T >= comm.push_min_tokens
        dst = comm.push_target(T) if push else None
        self.attn(xq, xs, meta, rotary, kv, reduce=False, out=dst if dst is not None else comm.partial(T))
        n2 = self.norm2
        x2 = comm.reduce_norm(T, n2.weight, n2.eps, 1.0 if n2.unit_offset else 0.0, quant=self.mlp_in_quant,
                              source=dst)
        x2q, x2s = x2 if isinstance(x2, tuple) else (x2, None)
        dst = comm.push_target(T) if push and isinstance(self.mlp, DenseMLP) else None
        self.mlp(x2q, x2s, reduce=False, meta=meta, out=dst if dst is not None else comm.partial(T))
        return comm.reduce_norm(T, next_norm.weight, next_norm.eps, 1.0 if next_norm.unit_offset else 0.0,
                                quant=next_quant, source=dst)


class CausalDecoder:
    """Weights + forward of one causal LM shard."""

    def __init__(self, cfg: ModelConfig, weights, comm=None, prefix: str = "", max_positions: Optional[int] = None):
        self.cfg = cfg
        self.arch = arch_for(cfg.model_type)
        pg = weights.process_group
        self.pg = pg
        self.comm = comm
        self.speculator = None                   # Medusa / MLP speculator head (models/speculative.py)
        self._fusable: Optional[bool] = None
        self.dims = dims = derive_dims(cfg, self.arch, pg.size())
        self.dtype, self.device = weights.dtype, weights.device
        a = self.arch
        px = (prefix + ".") if prefix else ""
        self.prefix = px
        self.embed = TensorParallelEmbedding(px + a.embed, weights, comm=comm)
        self.pos_embed = weights.get_tensor(px + a.pos_embed + ".weight") if a.pos_embed else None
        self.embed_norm = Norm.load(a, px + a.embed_norm, weights, dims.eps) if a.embed_norm else None
        from ..utils.quantization import DefaultWeightsLoader, Fp8Loader

        self.layers: List[DecoderLayer] = []
        cross_layers = set(cfg.get("cross_attention_layers") or [])
        for i in range(dims.num_layers):
            if i in cross_layers:
                from .mllama import CrossAttentionLayer

                self.layers.append(CrossAttentionLayer(a, cfg, dims, px + a.layer.format(i=i), weights, i, comm))
                continue
            # ``--quantize fp8`` (conversion at load) keeps the first and last layer in the serving
            # dtype, as the reference does (``flash_llama_modeling.py:124-134, 549``).
            loader = weights.weights_loader
            if isinstance(loader, Fp8Loader) and loader.to_fp8 and i in (0, dims.num_layers - 1):
                with weights.use_loader(DefaultWeightsLoader()):
                    self.layers.append(DecoderLayer(a, cfg, dims, px + a.layer.format(i=i), weights, i, comm))
            else:
                self.layers.append(DecoderLayer(a, cfg, dims, px + a.layer.format(i=i), weights, i, comm))
        self.final_norm = Norm.load(a, px + a.final_norm, weights, dims.eps)
        head_name = px + a.lm_head if not a.lm_head.startswith("lm_head") or not prefix else a.lm_head
        candidates = [head_name, px + a.lm_head, a.lm_head, px + a.embed]
        if cfg.get("tie_word_embeddings") and not any(weights.has_tensor(f"{c}.weight") for c in candidates[:3]):
            candidates = [px + a.embed]
        with weights.use_loader(DefaultWeightsLoader()):
            for cand in candidates:
                if weights.has_tensor(f"{cand}.weight"):
                    self.head = TensorParallelHead.load(cfg, cand, weights)
                    break
            else:
                raise KeyError("no lm_head / tied embedding weight found")
        self.max_positions = int(max_positions or dims.max_positions)
        self.rotary = RotaryTable.from_config(cfg, dims.rot_dim, dims.rope_theta, self.max_positions,
                                              a.rope_neox).to(self.device)
        # Gemma-3: sliding-window layers rotate with their own (unscaled) base frequency
        self.rotary_local = None
        local_theta = cfg.get("rope_local_base_freq")
        rp = cfg.get("rope_parameters")
        if local_theta is None and isinstance(rp, dict) and isinstance(rp.get("sliding_attention"), dict):
            local_theta = rp["sliding_attention"].get("rope_theta")
        if local_theta and cfg.model_type in ("gemma3", "gemma3_text"):
            self.rotary_local = RotaryTable.from_config(None, dims.rot_dim, float(local_theta), self.max_positions,
                                                        a.rope_neox).to(self.device)
        if a.alibi:
            slopes = alibi_slopes(dims.total_heads)[pg.rank() * dims.num_heads:(pg.rank() + 1) * dims.num_heads]
            for l in self.layers:
                l.attn.alibi_slopes = slopes.to(self.device)
            raise NotImplementedError("ALiBi attention bias is served by the padded fallback runner")

    # ---------------------------------------------------------------------------------------
    def embed_tokens(self, input_ids: torch.Tensor, positions: Optional[torch.Tensor] = None) -> torch.Tensor:
        h = self.embed(input_ids)
        if self.dims.embed_scale != 1.0:
            h = (h.float() * self.dims.embed_scale).to(h.dtype)
        if self.pos_embed is not None and positions is not None:
            h = h + self.pos_embed[(positions + self.arch.pos_offset).long()]
        if self.embed_norm is not None:
            h, _ = self.embed_norm(h, None)
        return h

    def _rotary_for(self, layer_idx: int) -> RotaryTable:
        if self.rotary_local is not None and self.dims.windows[layer_idx] > 0:
            return self.rotary_local
        return self.rotary

    def _fused_tp_ok(self, meta: ForwardMeta) -> bool:
        comm = self.comm
        if comm is None or not hasattr(comm, "reduce_norm") or self.pg.size() == 1:
            return False
        if self._fusable is None:
            d = self.dims
            self._fusable = (all(l.fusable_tp for l in self.layers) and self.final_norm.kind == "rms"
                             and d.embed_scale == 1.0 and self.pos_embed is None and self.embed_norm is None
                             and comm.width == d.hidden and self.dtype == torch.bfloat16)
        return (self._fusable and meta.adapter_data is None and meta.inputs_embeds is None
                and meta.input_ids.shape[0] <= comm.max_tokens)

    def _forward_hidden_fused_tp(self, meta: ForwardMeta, kv_cache) -> torch.Tensor:
        comm = self.comm
        T = meta.input_ids.shape[0]
        # vocab-parallel embedding rows (zero for ids of other ranks) are the first partial sums
        comm.partial(T).copy_(self.embed.local_rows(meta.input_ids))
        l0 = self.layers[0]
        x = comm.reduce_norm(T, l0.norm1.weight, l0.norm1.eps, 1.0 if l0.norm1.unit_offset else 0.0,
                             quant=l0.attn_in_quant, first=True)
        last = len(self.layers) - 1
        for i, layer in enumerate(self.layers):
            nxt = self.layers[i + 1] if i < last else None
            x = layer.fused_tp(x, meta, self._rotary_for(i), kv_cache[i], nxt.norm1 if nxt else self.final_norm,
                               nxt.attn_in_quant if nxt else False, comm)
        return x

    def forward_hidden(self, meta: ForwardMeta, kv_cache) -> torch.Tensor:
        if self._fused_tp_ok(meta):
            return self._forward_hidden_fused_tp(meta, kv_cache)
        h = meta.inputs_embeds if meta.inputs_embeds is not None else self.embed_tokens(meta.input_ids, meta.positions)
        residual = None
        for i, layer in enumerate(self.layers):
            h, residual = layer(h, residual, meta, self._rotary_for(i), kv_cache[i])
        h, _ = self.final_norm(h, residual)
        return h

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        out = self.head(hidden)
        d = self.dims
        if d.logit_scale != 1.0:
            out = out * d.logit_scale
        if d.logit_softcap > 0:
            out = (torch.tanh(out.float() / d.logit_softcap) * d.logit_softcap).to(out.dtype)
        return out

    @property
    def supports_local_head(self) -> bool:
        """True when greedy sampling can run on the vocabulary shards without gathering the logits."""
        return (self.comm is not None and hasattr(self.comm, "argmax") and self.pg.size() > 1
                and self.head.should_gather and self.dims.logit_softcap == 0 and self.speculator is None
                and self.dtype == torch.bfloat16)

    def forward_local(self, meta: ForwardMeta, kv_cache) -> Tuple[torch.Tensor, int]:
        """``(logits of this rank's vocabulary shard [rows, V / tp], first vocabulary id of the shard)``."""
        h = self.forward_hidden(meta, kv_cache)
        if meta.lm_head_indices is not None:
            h = h[meta.lm_head_indices.long()]
        return self.head.local_logits(h)

    def gather_logits(self, local: torch.Tensor) -> torch.Tensor:
        """Full ``[rows, V]`` logits from the shards (the path for samplers that need the distribution)."""
        out = self.head.gather(local)
        if self.dims.logit_scale != 1.0:
            out = out * self.dims.logit_scale
        return out

    def forward(self, meta: ForwardMeta, kv_cache) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """Returns ``(logits[rows, V], speculative_logits or None)``."""
        h = self.forward_hidden(meta, kv_cache)
        if meta.lm_head_indices is not None:
            h = h[meta.lm_head_indices.long()]
        logits = self.logits(h)
        spec = self.speculator(h, logits) if self.speculator is not None else None
        return logits, spec


def alibi_slopes(n: int) -> torch.Tensor:
    def pow2(n):
        start = 2 ** (-(2 ** -(math.log2(n) - 3)))
        return [start * (start ** i) for i in range(n)]

    if math.log2(n).is_integer():
        return torch.tensor(pow2(n), dtype=torch.float32)
    c = 2 ** math.floor(math.log2(n))
    return torch.tensor(pow2(c) + pow2(2 * c)[0::2][: n - c], dtype=torch.float32)
