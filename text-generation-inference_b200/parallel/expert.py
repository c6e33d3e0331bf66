"""Expert parallelism for sparse mixture-of-experts layers.

The reference only tensor-parallelises experts: every rank holds a 1/tp slice of every expert and the
partial outputs are all-reduced (``layers/moe/unquantized.py:107-163``,
``flash_mixtral_modeling.py:343-351``).  With expert parallelism each rank holds whole experts
(expert ``e`` lives on rank ``e // (E / world)``), which gives every expert GEMM its full K and N.

Token exchange.  The attention block of the same layer is tensor parallel, and the fused reduction that
follows it (``parallel/peer.py``) leaves the normalised activations of *all* tokens on every rank.  So
the "dispatch" all-to-all degenerates: a rank already holds every token routed to its experts and only
has to select them.  The "combine" is a sum over ranks of rows that are non-zero on at most ``top_k``
ranks; it is done by the same peer-memory kernel that reduces dense layers, fused with the residual add
and the next RMSNorm, so an expert-parallel layer issues exactly one collective.

Two evaluation modes of the local experts:

* ``routed`` (default): the (token, slot) pairs of the local experts are grouped by expert on the device and one
  grouped GEMM launch per projection walks the per-expert row ranges (``ops/csrc/moe_sm100.cu``): no host
  synchronisation, fixed buffer shapes, CUDA-graph capturable, only routed rows are computed.
* ``dense`` (``TGI_B200_MOE_EVAL=dense``, steps of up to ``TGI_B200_MOE_DENSE_TOKENS`` tokens): every local expert
  runs on all ``T`` tokens and its output is scaled by the token's routing weight; kept as the comparison point.
"""
from __future__ import annotations

import os
from typing import List, Optional

import torch

from .. import ops


def local_expert_range(num_experts: int, rank: int, world: int):
    assert num_experts % world == 0, "expert parallelism needs the expert count to be divisible by the ranks"
    per = num_experts // world
    return rank * per, (rank + 1) * per


class ExpertParallel:
    """Evaluates the experts owned by this rank; ``__call__`` returns this rank's partial output ``[T, H]``."""

    def __init__(self, w_gate_up: torch.Tensor, w_down: torch.Tensor, first: int, act: str,
                 dense_max_tokens: Optional[int] = None):
        self.w_gate_up, self.w_down, self.first, self.act = w_gate_up, w_down, first, act
        self.n_local = w_gate_up.shape[0]
        self.dense_max_tokens = int(os.environ.get("TGI_B200_MOE_DENSE_TOKENS", "512")) \
            if dense_max_tokens is None else dense_max_tokens

    def __call__(self, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        mode = os.environ.get("TGI_B200_MOE_EVAL", "routed")
        if mode == "dense" and x.shape[0] <= self.dense_max_tokens:
            return dense_experts(x, self.w_gate_up, self.w_down, topk_weights, topk_ids, self.first, self.act)
        # routed: the (token, slot) pairs that point at a local expert are grouped by expert on the device
        return ops.moe_experts(x, self.w_gate_up, self.w_down, topk_weights, topk_ids, self.act, self.first)


def dense_experts(x, w_gate_up, w_down, topk_weights, topk_ids, first: int, act: str) -> torch.Tensor:
    """``sum_e route[t, e] * MLP_e(x[t])`` over the experts ``first .. first + E_local`` with fixed shapes."""
    T, H = x.shape
    E_local = w_gate_up.shape[0]
    route = torch.zeros(T, first + E_local + 1, dtype=torch.float32, device=x.device)
    # ids outside the local range land in columns that are never read (clamped to the last column)
    cols = torch.where((topk_ids >= first) & (topk_ids < first + E_local), topk_ids,
                       torch.full_like(topk_ids, first + E_local))
    route.scatter_add_(1, cols.long(), topk_weights.float())
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    for j in range(E_local):
        h = ops.linear(x, w_gate_up[j])
        a = ops.act_and_mul(h, act)
        y = ops.linear(a, w_down[j])
        out.addcmul_(y.float(), route[:, first + j:first + j + 1])
    return out.to(x.dtype)


def wants_expert_parallel(num_experts: int, world: int) -> bool:
    """Whole experts per rank (``TGI_B200_MOE_PARALLEL=ep``) or every expert sliced over the ranks (``tp``, what the
    reference does and the default).  Measured on B200 with the Mixtral-8x7B shape, 256 sequences, bf16: sliced
    experts 18.3k / 30.1k tok/s on 2 / 4 GPUs against 17.6k / 25.8k with whole experts, and 28.5k against 23.3k on 4
    GPUs when two experts draw most of the tokens: a rank's load follows the routing when it owns whole experts,
    while slices always split every expert's work evenly."""
    mode = os.environ.get("TGI_B200_MOE_PARALLEL", "tp")
    if world == 1 or mode == "tp":
        return False
    if num_experts % world != 0:
        if mode == "ep":
            raise ValueError(f"{num_experts} experts cannot be spread over {world} ranks")
        return False
    return mode == "ep"
