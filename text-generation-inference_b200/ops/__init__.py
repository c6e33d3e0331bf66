"""Op front end: routes every hot op to the sm_100a kernels (CUDA tensors) or the PyTorch oracle (CPU).

On a CUDA tensor the native kernel library is *required*: if it has not been
built, the call raises instead of silently running a PyTorch fallback.  Setting
``TGI_B200_OPS=torch`` selects the PyTorch implementations on the GPU as well;
that switch exists for A/B numerics checks and for the library-kernel baseline
path, never as a default.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import reference as ref

_FORCE_TORCH = os.environ.get("TGI_B200_OPS", "") == "torch"
_backend = None


def native():
    """The CUDA kernel backend module (loads the in-tree shared library on first use)."""
    global _backend
    if _backend is None:
        from . import cuda as _cuda_backend

        _cuda_backend.load()
        _backend = _cuda_backend
    return _backend


def use_native(t: torch.Tensor) -> bool:
    return t.is_cuda and not _FORCE_TORCH


def set_force_torch(flag: bool) -> None:
    global _FORCE_TORCH
    _FORCE_TORCH = flag


def rms_norm(x, residual, weight, eps, unit_offset=False):
    if use_native(x):
        return native().rms_norm(x, residual, weight, eps, unit_offset)
    return ref.rms_norm(x, residual, weight, eps, unit_offset)


def rms_norm_quant(x, residual, weight, eps, unit_offset=False):
    """Residual-add + RMSNorm + 1x128 e4m3 quantisation: returns ``(xq, scales, new_residual)``."""
    if use_native(x):
        return native().rms_norm_quant(x, residual, weight, eps, unit_offset)
    y, res = ref.rms_norm(x, residual, weight, eps, unit_offset)
    q, s = ref.fp8_quant_act(y)
    return q, s, res


def layer_norm(x, residual, weight, bias, eps):
    if use_native(x):
        return native().layer_norm(x, residual, weight, bias, eps)
    return ref.layer_norm(x, residual, weight, bias, eps)


def rope_and_cache(qkv, positions, cos_sin, slots, k_cache, v_cache, num_heads, num_kv_heads, head_dim,
                   rot_dim, neox=True, k_scale=None, v_scale=None):
    if use_native(qkv):
        return native().rope_and_cache(qkv, positions, cos_sin, slots, k_cache, v_cache, num_heads,
                                       num_kv_heads, head_dim, rot_dim, neox, k_scale, v_scale)
    return ref.rope_and_cache(qkv, positions, cos_sin, slots, k_cache, v_cache, num_heads, num_kv_heads,
                              head_dim, rot_dim, neox, k_scale, v_scale)


def paged_attention(q, k_cache, v_cache, block_tables, cu_seqlens_q, kv_lens, scale, window=-1, softcap=0.0,
                    k_scale=None, v_scale=None, max_q=None, max_kv=None, horizon=None):
    """``horizon`` (optional int32 ``[T]``): last KV position each query row may see when that is past its own
    position (image rows that attend to their whole image); ``None`` is plain causal attention."""
    if use_native(q):
        return native().paged_attention(q, k_cache, v_cache, block_tables, cu_seqlens_q, kv_lens, scale,
                                        window, softcap, k_scale, v_scale, max_q, max_kv, horizon=horizon)
    return ref.paged_attention(q, k_cache, v_cache, block_tables, cu_seqlens_q, kv_lens, scale, window,
                               softcap, k_scale, v_scale, horizon=horizon)


def act_and_mul(gate_up, act="silu"):
    if use_native(gate_up):
        return native().act_and_mul(gate_up, act)
    return ref.act_and_mul(gate_up, act)


def act_and_mul_quant(gate_up, act="silu"):
    """``act(gate) * up`` followed by 1x128 e4m3 quantisation: ``(q, scales)``."""
    if use_native(gate_up):
        return native().act_and_mul_quant(gate_up, act)
    return ref.fp8_quant_act(ref.act_and_mul(gate_up, act))


def activation(x, act):
    return ref.activation(x, act)


def _into(out, y):
    if out is None:
        return y
    if getattr(out, "is_peer_push", False):
        out = out.fallback      # no pushing kernel on this path: the reduction pulls from the plain buffer
    out.copy_(y.view_as(out))
    return out


def linear(x, weight, bias=None, out=None):
    """``x @ weight^T + bias``; ``out`` (bf16, contiguous) receives the result when given."""
    if use_native(x) and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16:
        return native().gemm_bf16(x, weight, bias, out=out)
    return _into(out, ref.linear(x, weight, bias))


def fp8_quant_act(x, group=128):
    if use_native(x):
        return native().fp8_quant_act(x, group)
    return ref.fp8_quant_act(x, group)


def gemm_fp8_block(xq, xs, wq, ws, out_dtype=torch.bfloat16, bias=None, out=None):
    if use_native(xq):
        return native().gemm_fp8_block(xq, xs, wq, ws, out_dtype, bias, out=out)
    return _into(out, ref.gemm_fp8_block(xq, xs, wq, ws, out_dtype, bias))


def embedding(ids, table):
    if use_native(table):
        return native().embedding(ids, table)
    return ref.embedding(ids, table)


def argmax_logprob(logits):
    if use_native(logits):
        return native().argmax_logprob(logits)
    return ref.argmax_logprob(logits)


def has_fused_sample(scores) -> bool:
    return use_native(scores)


def fused_sample(scores, temperature=None, top_k=None, top_p=None, do_sample=None, seeds=None, steps=None, typical_p=None):
    """One-kernel temperature / top-k / top-p / typical-p / sampling on CUDA tensors (see ``ops.cuda.fused_sample``)."""
    return native().fused_sample(scores, temperature, top_k, top_p, do_sample, seeds, steps, typical_p=typical_p)


def penalties(scores, history, repetition_penalty=None, frequency_penalty=None):
    """fp32 copy of CUDA ``scores[B, V]`` with repetition / frequency penalties of ``history[B, L]`` applied."""
    return native().penalties(scores, history, repetition_penalty, frequency_penalty)


def moe_topk_softmax(router_logits, top_k, renormalize=True):
    if use_native(router_logits) and router_logits.shape[-1] <= 256 and top_k <= 8:
        return native().moe_topk_softmax(router_logits, top_k, renormalize)
    return ref.moe_topk_softmax(router_logits, top_k, renormalize)


def moe_sparsemixer(router_logits, jitter_eps=0.01):
    return ref.moe_sparsemixer(router_logits, jitter_eps)


def moe_experts(x, w_gate_up, w_down, topk_weights, topk_ids, act="silu", first: int = 0):
    """Routed experts ``first .. first + E_local - 1`` (``first`` > 0: an expert-parallel rank's share)."""
    if use_native(x) and x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 \
            and (w_gate_up.shape[1] // 2) % 8 == 0 and w_gate_up.shape[0] <= 256 and topk_ids.shape[1] <= 8:
        return native().moe_experts(x, w_gate_up, w_down, topk_weights, topk_ids, act, first)
    return ref.moe_experts(x, w_gate_up, w_down, topk_weights, topk_ids, act, first)
