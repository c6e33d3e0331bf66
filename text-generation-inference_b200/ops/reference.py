"""Plain PyTorch fp32 implementations of every op in ``tgi_b200.ops``.

They serve two purposes: they are the CPU execution path (the engine runs on a
machine without a GPU, e.g. for the tiny-Llama correctness configuration), and
they are the numerical oracle the CUDA kernels are tested against.  They favour
clarity over speed.

Tensor conventions (ragged / unpadded batches):

* ``T`` tokens of the step, ``B`` sequences, ``Hq``/``Hkv`` query/KV heads, ``D`` head size.
* KV cache of one layer: ``k_cache``/``v_cache`` of shape ``[num_blocks, block_size, Hkv, D]``;
  slot ``s`` addresses ``cache.view(-1, Hkv, D)[s]``.
* ``block_tables[B, max_blocks]`` int32; ``cu_seqlens_q[B+1]`` int32 prefix sums of the
  number of query tokens per sequence; ``kv_lens[B]`` int32 = number of KV tokens each
  sequence attends to *including* the tokens of this step.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

FP8_MAX = 448.0
FP8 = torch.float8_e4m3fn


def rms_norm(x, residual, weight, eps: float, unit_offset: bool = False):
    if residual is not None:
        x = x + residual
    res = x
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    y = xf * torch.rsqrt(var + eps)
    w = weight.float()
    if unit_offset:
        w = w + 1.0
    return (y * w).to(x.dtype), res


def layer_norm(x, residual, weight, bias, eps: float):
    if residual is not None:
        x = x + residual
    res = x
    y = F.layer_norm(x.float(), (x.shape[-1],), weight.float(), None if bias is None else bias.float(), eps)
    return y.to(x.dtype), res


def rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rot_dim: int, neox: bool) -> torch.Tensor:
    """Apply rotary embedding on the first ``rot_dim`` features of ``x[T, H, D]``.

    ``cos``/``sin`` are ``[T, rot_dim/2]``.  NeoX style pairs feature ``i`` with
    ``i + rot_dim/2``; GPT-J style pairs ``2i`` with ``2i+1``.
    """
    xr = x[..., :rot_dim].float()
    c = cos.float().unsqueeze(1)
    s = sin.float().unsqueeze(1)
    if neox:
        x1, x2 = xr[..., : rot_dim // 2], xr[..., rot_dim // 2 :]
        out = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)
    else:
        x1, x2 = xr[..., 0::2], xr[..., 1::2]
        out = torch.stack([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).flatten(-2)
    res = x.clone()
    res[..., :rot_dim] = out.to(x.dtype)
    return res


def rope_and_cache(
    qkv: torch.Tensor,
    positions: torch.Tensor,
    cos_sin: torch.Tensor,
    slots: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    rot_dim: int,
    neox: bool = True,
    k_scale: Optional[torch.Tensor] = None,
    v_scale: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Rotate q and k inside ``qkv[T, (Hq+2Hkv)*D]``, scatter k, v into the paged cache; returns q ``[T,Hq,D]``.

    ``cos_sin[max_pos, rot_dim]`` holds ``cos`` in the first half of each row and ``sin`` in the second
    (``rot_dim == 0`` disables rotation).  For an fp8 cache the stored value is
    ``x / scale`` with a per-KV-head ``scale[Hkv]`` (``None`` means 1).
    """
    T = qkv.shape[0]
    q, k, v = qkv.split([num_heads * head_dim, num_kv_heads * head_dim, num_kv_heads * head_dim], dim=-1)
    q = q.reshape(T, num_heads, head_dim)
    k = k.reshape(T, num_kv_heads, head_dim)
    v = v.reshape(T, num_kv_heads, head_dim)
    if rot_dim > 0:
        cs = cos_sin[positions.long()]
        cos, sin = cs[:, : rot_dim // 2], cs[:, rot_dim // 2 :]
        q = rotate(q, cos, sin, rot_dim, neox)
        k = rotate(k, cos, sin, rot_dim, neox)
    kc = k_cache.view(-1, num_kv_heads, head_dim)
    vc = v_cache.view(-1, num_kv_heads, head_dim)
    idx = slots.long()
    if k_cache.dtype == FP8:
        ks = 1.0 if k_scale is None else k_scale.float().view(1, -1, 1)
        vs = 1.0 if v_scale is None else v_scale.float().view(1, -1, 1)
        # scatter through a byte view: indexed writes are not implemented for fp8 on every backend
        kc.view(torch.uint8)[idx] = (k.float() / ks).clamp(-FP8_MAX, FP8_MAX).to(FP8).view(torch.uint8)
        vc.view(torch.uint8)[idx] = (v.float() / vs).clamp(-FP8_MAX, FP8_MAX).to(FP8).view(torch.uint8)
    else:
        kc[idx] = k.to(k_cache.dtype)
        vc[idx] = v.to(v_cache.dtype)
    return q.contiguous()


def paged_attention(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_tables: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    kv_lens: torch.Tensor,
    scale: float,
    window: int = -1,
    softcap: float = 0.0,
    k_scale: Optional[torch.Tensor] = None,
    v_scale: Optional[torch.Tensor] = None,
    max_q: Optional[int] = None,
    max_kv: Optional[int] = None,
    horizon: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Causal attention of ragged queries over paged KV (covers prefill, chunked prefill and decode).
    ``horizon[t]`` (optional) replaces the causal limit of query row ``t`` by a later position.

    Query ``i`` (0-based inside its sequence's chunk of ``n`` queries) of a sequence with ``L`` KV
    tokens sits at absolute position ``L - n + i`` and attends to KV positions ``<=`` its own
    (and ``> pos - window`` when ``window > 0``).
    """
    T, Hq, D = q.shape
    nblk, bs, Hkv, _ = k_cache.shape
    group = Hq // Hkv
    out = torch.empty_like(q)
    cu = cu_seqlens_q.tolist()
    lens = kv_lens.tolist()
    kc = k_cache.view(-1, Hkv, D)
    vc = v_cache.view(-1, Hkv, D)
    for b in range(len(lens)):
        s, e = cu[b], cu[b + 1]
        n, L = e - s, lens[b]
        if n == 0:
            continue
        nb = (L + bs - 1) // bs
        blocks = block_tables[b, :nb].long()
        slot = (blocks.unsqueeze(1) * bs + torch.arange(bs, device=q.device).unsqueeze(0)).reshape(-1)[:L]
        if kc.dtype == FP8:
            k = kc.view(torch.uint8)[slot].view(FP8).float()
            v = vc.view(torch.uint8)[slot].view(FP8).float()
        else:
            k = kc[slot].float()
            v = vc[slot].float()
        if k_scale is not None:
            k = k * k_scale.float().view(1, -1, 1)
        if v_scale is not None:
            v = v * v_scale.float().view(1, -1, 1)
        k = k.repeat_interleave(group, dim=1)  # [L, Hq, D]
        v = v.repeat_interleave(group, dim=1)
        qq = q[s:e].float()
        scores = torch.einsum("nhd,lhd->hnl", qq, k) * scale
        if softcap > 0:
            scores = softcap * torch.tanh(scores / softcap)
        qpos = torch.arange(L - n, L, device=q.device).unsqueeze(1)
        kpos = torch.arange(L, device=q.device).unsqueeze(0)
        limit = qpos if horizon is None else torch.maximum(qpos, horizon[s:e].long().clamp(max=L - 1).unsqueeze(1))
        mask = kpos <= limit
        if window > 0:
            mask &= kpos > qpos - window
        scores = scores.masked_fill(~mask.unsqueeze(0), float("-inf"))
        p = torch.softmax(scores, dim=-1)
        out[s:e] = torch.einsum("hnl,lhd->nhd", p, v).to(q.dtype)
    return out


def act_and_mul(gate_up: torch.Tensor, act: str = "silu") -> torch.Tensor:
    g, u = gate_up.float().chunk(2, dim=-1)
    return (activation(g, act) * u).to(gate_up.dtype)


def activation(x: torch.Tensor, act: str) -> torch.Tensor:
    if act in ("silu", "swish"):
        return F.silu(x)
    if act in ("gelu", "gelu_python"):
        return F.gelu(x)
    if act in ("gelu_new", "gelu_fast", "gelu_pytorch_tanh", "gelu_tanh"):
        return F.gelu(x, approximate="tanh")
    if act == "relu":
        return F.relu(x)
    if act == "quick_gelu":
        return x * torch.sigmoid(1.702 * x)
    raise ValueError(f"unknown activation {act}")


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    return F.linear(x, weight, bias)


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    return F.embedding(ids.long(), table)


# ---- block-scaled fp8 -------------------------------------------------------------------------
def fp8_quant_block_weight(w: torch.Tensor, block: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """Quantise ``w[N,K]`` to e4m3 with one fp32 scale per ``block x block`` tile.

    Returns ``(wq[N,K] e4m3, scale[ceil(N/block), ceil(K/block)])`` with ``w ~= wq * scale``.
    """
    N, K = w.shape
    nb, kb = (N + block - 1) // block, (K + block - 1) // block
    wp = torch.zeros(nb * block, kb * block, dtype=torch.float32, device=w.device)
    wp[:N, :K] = w.float()
    tiles = wp.view(nb, block, kb, block)
    amax = tiles.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    scale = amax / FP8_MAX
    q = (tiles / scale.view(nb, 1, kb, 1)).clamp(-FP8_MAX, FP8_MAX).view(nb * block, kb * block)[:N, :K]
    return q.to(FP8).contiguous(), scale.contiguous()


POW2_ACT_SCALES = False      # activation block scales rounded up to powers of two


def fp8_quant_act(x: torch.Tensor, group: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """Dynamic per-token, per-``group``-columns quantisation: ``x[T,K] ~= xq * scale[T, K/group]``."""
    T, K = x.shape
    assert K % group == 0
    xg = x.float().view(T, K // group, group)
    amax = xg.abs().amax(dim=-1).clamp_min(1e-12)
    scale = amax / FP8_MAX
    if POW2_ACT_SCALES:      # what the kernels do while the block-scaled MMA is in use (ops.cuda.set_fp8_mx)
        mant, expo = torch.frexp(scale)
        scale = torch.where(mant == 0.5, scale, torch.ldexp(torch.ones_like(scale), expo))
    q = (xg / scale.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).view(T, K)
    return q.to(FP8), scale.contiguous()


def fp8_dequant_block_weight(wq: torch.Tensor, scale: torch.Tensor, block: int = 128) -> torch.Tensor:
    N, K = wq.shape
    s = scale.repeat_interleave(block, 0)[:N].repeat_interleave(block, 1)[:, :K]
    return wq.float() * s


def gemm_fp8_block(
    xq: torch.Tensor,
    xs: torch.Tensor,
    wq: torch.Tensor,
    ws: torch.Tensor,
    out_dtype: torch.dtype = torch.bfloat16,
    bias: Optional[torch.Tensor] = None,
    block: int = 128,
) -> torch.Tensor:
    """``out[T,N] = (xq*xs) @ (wq*ws)^T`` with 1x128 activation and 128x128 weight scales."""
    x = xq.float() * xs.repeat_interleave(block, dim=1)[:, : xq.shape[1]]
    w = fp8_dequant_block_weight(wq, ws, block)
    out = x @ w.t()
    if bias is not None:
        out = out + bias.float()
    return out.to(out_dtype)


def fp8_quant_per_tensor(x: torch.Tensor, scale: Optional[torch.Tensor] = None, scale_ub: Optional[float] = None):
    """Per-tensor e4m3 quantisation; dynamic when ``scale`` is None."""
    if scale is None:
        amax = x.abs().max().float()
        if scale_ub is not None:
            amax = amax.clamp(max=scale_ub)
        scale = (amax / FP8_MAX).clamp_min(1e-12)
    q = (x.float() / scale).clamp(-FP8_MAX, FP8_MAX).to(FP8)
    return q, scale.reshape(()).float()


# ---- sampling ---------------------------------------------------------------------------------
def argmax_logprob(logits: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Greedy token and its log-probability for each row of ``logits[B,V]``."""
    lp = torch.log_softmax(logits.float(), dim=-1)
    ids = lp.argmax(dim=-1)
    return ids, lp.gather(1, ids.unsqueeze(1)).squeeze(1)


# ---- MoE --------------------------------------------------------------------------------------
def moe_topk_softmax(router_logits: torch.Tensor, top_k: int, renormalize: bool = True):
    probs = torch.softmax(router_logits.float(), dim=-1)
    w, idx = torch.topk(probs, top_k, dim=-1)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    return w, idx


def moe_sparsemixer(router_logits: torch.Tensor, jitter_eps: float = 0.01) -> Tuple[torch.Tensor, torch.Tensor]:
    """Top-2 routing of Phi-3.5-MoE ("sparsemixer", inference form): each of the two picks is the arg-max of
    the remaining logits, and its weight is the softmax over the logits that lie within a relative
    band ``2 * jitter_eps`` of that maximum."""
    s = router_logits.float()
    neg = float("-inf")
    m1, i1 = s.max(-1, keepdim=True)
    mask1 = ((m1 - s) / s.abs().clamp(min=m1)) > 2 * jitter_eps
    g1 = torch.softmax(s.masked_fill(mask1, neg), -1).gather(-1, i1)
    s2 = s.scatter(-1, i1, neg)
    m2, i2 = s2.max(-1, keepdim=True)
    mask2 = ((m2 - s) / s.abs().clamp(min=m2)) > 2 * jitter_eps
    g2 = torch.softmax(s2.masked_fill(mask2, neg), -1).gather(-1, i2)
    return torch.cat([g1, g2], -1), torch.cat([i1, i2], -1)


def moe_experts(
    x: torch.Tensor,
    w_gate_up: torch.Tensor,
    w_down: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    act: str = "silu",
    first: int = 0,
) -> torch.Tensor:
    """Dense-loop mixture of experts: ``w_gate_up[E, 2I, H]``, ``w_down[E, H, I]`` hold the experts
    ``first .. first + E - 1``; slots routed to other experts contribute nothing."""
    T, H = x.shape
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    E = w_gate_up.shape[0]
    for e in range(E):
        tok, slot = (topk_ids == e + first).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h = F.linear(x[tok], w_gate_up[e])
        h = act_and_mul(h, act)
        y = F.linear(h, w_down[e]).float()
        out.index_add_(0, tok, y * topk_weights[tok, slot].unsqueeze(1).float())
    return out.to(x.dtype)
