"""Local `moe` kernel module for the reference (hub: kernels-community/moe, built from vllm's fused_moe):
routing and fused expert GEMMs from the installed vllm wheel."""
import torch
from vllm.model_executor.layers.fused_moe import fused_experts as _fused_experts
from vllm.model_executor.layers.fused_moe import fused_topk as _fused_topk
try:
    from vllm.model_executor.layers.fused_moe import grouped_topk as _grouped_topk
except ImportError:  # pragma: no cover
    _grouped_topk = None


def fused_topk(hidden_states, gating_output, topk, renormalize):
    out = _fused_topk(hidden_states, gating_output, topk, renormalize)
    return out[0], out[1]


def grouped_topk(hidden_states, gating_output, topk, renormalize, num_expert_group=0, topk_group=0,
                 scoring_func="softmax", e_score_correction_bias=None):
    out = _grouped_topk(hidden_states, gating_output, topk, renormalize, num_expert_group, topk_group,
                        scoring_func=scoring_func, e_score_correction_bias=e_score_correction_bias)
    return out[0], out[1]


def fused_experts(hidden_states, w1, w2, topk_weights, topk_ids, inplace=False, **kwargs):
    return _fused_experts(hidden_states, w1, w2, topk_weights, topk_ids, inplace=inplace)


def fused_moe(hidden_states, w1, w2, gating_output, topk, renormalize=True, inplace=False, **kwargs):
    tw, ti = fused_topk(hidden_states, gating_output, topk, renormalize)
    return fused_experts(hidden_states, w1, w2, tw, ti, inplace=inplace)


def fused_marlin_moe(*a, **k):
    raise NotImplementedError("fused_marlin_moe is not provided by the installed vllm wheel")
