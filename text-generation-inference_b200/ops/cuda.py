"""ctypes bindings of the sm_100a kernel library (``libtgi_b200_kernels.so``, built by ``ops/build.py``).

Every wrapper allocates its outputs with torch (so they live in the caching allocator and are graph
capturable), passes raw pointers plus the current CUDA stream, and raises on a non-zero return code.
Kernels that wait on barriers report protocol time-outs through a device status word that
``check_status()`` reads; it is checked by tests and by the engine after each step, never inside a
captured graph.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path
from typing import Optional, Tuple

import torch

_LIB = None
_LIB_PATH = Path(__file__).resolve().parent / "libtgi_b200_kernels.so"
FP8 = torch.float8_e4m3fn

_ACT_CODES = {"silu": 0, "swish": 0, "gelu": 1, "gelu_python": 1, "gelu_new": 2, "gelu_fast": 2,
              "gelu_pytorch_tanh": 2, "gelu_tanh": 2, "relu": 3, "quick_gelu": 4}

c_void_p, c_int, c_float, c_ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong


class KernelError(RuntimeError):
    pass


def lib_path() -> Path:
    return _LIB_PATH


def load():
    """Load the kernel library; a missing library on a CUDA machine is an error, never a silent fallback."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not _LIB_PATH.exists():
        if os.environ.get("TGI_B200_AUTOBUILD", "1") == "1":
            from .build import build

            build()
        if not _LIB_PATH.exists():
            raise KernelError(
                f"{_LIB_PATH} is missing: build it with `python -m tgi_b200.ops.build` "
                "(the sm_100a kernels are required on CUDA devices)")
    _LIB = ctypes.CDLL(str(_LIB_PATH))
    for name in ("tgi_gemm_bf16", "tgi_gemm_fp8_block", "tgi_norm", "tgi_act_mul", "tgi_quant_act",
                 "tgi_rope_cache", "tgi_embedding", "tgi_argmax_logprob", "tgi_paged_attention", "tgi_paged_attention_ex",
                 "tgi_gemm_num_tiles", "tgi_attn_decode_splits", "tgi_attn_status", "tgi_lora_shrink",
                 "tgi_lora_expand", "tgi_moe_topk_softmax", "tgi_moe_sort", "tgi_moe_gather", "tgi_moe_grouped_gemm",
                 "tgi_moe_combine", "tgi_gemm_last_grid", "tgi_penalties", "tgi_gemm_wq", "tgi_wq_dequant", "tgi_qk_norm",
                 "tgi_quant_set_pow2", "tgi_peer_set_quant_pow2"):
        getattr(_LIB, name).restype = c_int
    _LIB.tgi_gemm_workspace_floats.restype = c_ll
    wide = os.environ.get("TGI_B200_GEMM_WIDE_M")
    if wide:
        _LIB.tgi_gemm_set_wide_m(c_int(int(wide)))
    if os.environ.get("TGI_B200_GEMM_PAIRS", "1") == "0":   # single-CTA 256 x 128 tiles instead of CTA pairs
        _LIB.tgi_gemm_set_pairs(c_int(0))
    if os.environ.get("TGI_B200_MX_PAIRS", "1") == "0":       # block-scaled mode on single CTAs only
        _LIB.tgi_gemm_set_mx_pairs(c_int(0))
    if os.environ.get("TGI_B200_GEMM_STREAMK_SMALL", "0") == "1":   # stream-K also below one tile per worker
        _LIB.tgi_gemm_set_streamk_small(c_int(1))
    # fp8 GEMMs run on the block-scaled MMA unless TGI_B200_FP8_MX=0 (then: per-K-block promotion, arbitrary scales)
    if os.environ.get("TGI_B200_FP8_MX", "1") == "1" and torch.cuda.is_available():
        set_fp8_mx(True)
    return _LIB


_FP8_MX = False


def set_fp8_mx(on: bool) -> None:
    """Block-scaled fp8 GEMMs on ``tcgen05.mma.kind::mxf8f6f4``: the tensor core applies the block scales, so they
    must be powers of two.  Switching it on makes every activation-quantising kernel round its scales up to a power
    of two; block-scaled weights have to be brought to power-of-two scales once (``requant_block_pow2``, done by
    ``Fp8Linear`` at load)."""
    global _FP8_MX
    lib = _LIB if _LIB is not None else load()
    v = c_int(1 if on else 0)
    lib.tgi_gemm_set_fp8_mx(v)
    _check(lib.tgi_quant_set_pow2(v), "quant_set_pow2")
    _check(lib.tgi_peer_set_quant_pow2(v), "peer_set_quant_pow2")
    _FP8_MX = bool(on)
    from . import reference

    reference.POW2_ACT_SCALES = bool(on)     # the PyTorch oracle quantises the same way


def fp8_mx() -> bool:
    return _FP8_MX


def requant_block_pow2(wq: torch.Tensor, scale: torch.Tensor, block: int = 128):
    """e4m3 weights ``[N, K]`` with one scale per ``block x block`` tile -> the same matrix with every scale rounded
    up to a power of two and the values re-rounded to e4m3 (``w * s = w' * s'`` up to that rounding).  Engines that
    feed block-scaled checkpoints to Blackwell's scale-factor MMA do the same (it takes E8M0 scale factors)."""
    scale = scale.float()
    mant, expo = torch.frexp(scale)                      # scale = mant * 2^expo, mant in [0.5, 1)
    s2 = torch.where(mant == 0.5, scale, torch.ldexp(torch.ones_like(scale), expo))
    ratio = scale / s2                                   # in (0.5, 1]
    N, K = wq.shape
    out = torch.empty_like(wq)
    rows = max(block, (1 << 26) // max(K, 1) // block * block)     # chunks of about 64 M elements
    for r0 in range(0, N, rows):
        r1 = min(N, r0 + rows)
        rr = ratio[r0 // block:(r1 + block - 1) // block].repeat_interleave(block, 0)[:r1 - r0]
        rr = rr.repeat_interleave(block, 1)[:, :K]
        out[r0:r1] = (wq[r0:r1].float() * rr).to(wq.dtype)
    return out, s2.contiguous()


def set_gemm_pairs(on: bool) -> None:
    """Use CTA pairs (``cta_group::2``, 256 x 256 tiles) for GEMMs with more than 128 tokens (default), or
    single CTAs on 256 x 128 tiles."""
    load().tgi_gemm_set_pairs(c_int(1 if on else 0))


def _ptr(t: Optional[torch.Tensor]):
    return c_void_p(0 if t is None else t.data_ptr())


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


LAUNCHES = 0  # kernel-launching library calls made so far (benchmarks read and reset it)


def _check(rc: int, what: str):
    global LAUNCHES
    LAUNCHES += 1
    if rc != 0:
        raise KernelError(f"{what} failed with code {rc}")


# ---- per-device state: split-K workspace, counters, status word --------------------------------
class _DeviceState:
    def __init__(self, device: torch.device):
        self.device = device
        self.sm_count = torch.cuda.get_device_properties(device).multi_processor_count
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.counters = torch.zeros(1 << 16, dtype=torch.int32, device=device)
        self.ws = torch.empty(int(os.environ.get("TGI_B200_SPLITK_WS_MB", "64")) << 18, dtype=torch.float32,
                              device=device)
        self.attn_part_o = None
        self.attn_part_ml = None


_STATES = {}


def state(device: torch.device) -> _DeviceState:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    st = _STATES.get(idx)
    if st is None:
        st = _STATES[idx] = _DeviceState(torch.device("cuda", idx))
    return st


def check_status(device: Optional[torch.device] = None) -> int:
    """Read (and clear) the kernels' error word; 0 means no kernel gave up on a wait."""
    dev = device or torch.device("cuda", torch.cuda.current_device())
    st = state(dev)
    code = int(st.status.item())
    if code != 0:
        st.status.zero_()
        st.counters.zero_()    # a kernel that gave up may have left split-tile counters half-way
    with torch.cuda.device(st.device):
        attn = int(load().tgi_attn_status(c_int(1)))   # decode attention: a page copy did not arrive in time
    if attn != 0 and code == 0:
        code = 100 + attn
    return code


# ---- scale tensors -----------------------------------------------------------------------------
def alloc_act_scales(T: int, groups: int, device) -> torch.Tensor:
    """Activation scales, logical shape ``[T, groups]`` stored K-block major with a 16-byte aligned pitch."""
    pitch = (max(T, 1) + 3) & ~3
    buf = torch.empty(groups, pitch, dtype=torch.float32, device=device)
    return buf[:, :T].t()


def _scale_storage(xs: torch.Tensor) -> Tuple[int, int]:
    """(data_ptr, pitch) of a ``[T, groups]`` scale view produced by ``alloc_act_scales``."""
    if xs.dim() != 2 or (xs.shape[0] > 1 and xs.stride(0) != 1):
        raise KernelError("activation scales must be K-block major (use ops.fp8_quant_act / the fused producers)")
    pitch = xs.stride(1) if xs.shape[1] > 1 else ((xs.shape[0] + 3) & ~3)
    return xs.data_ptr(), pitch


# ---- GEMMs -------------------------------------------------------------------------------------
def _gemm_ctas(lib, st, M: int, N: int, max_ctas: Optional[int]) -> int:
    """Grid size of the persistent stream-K GEMM: one CTA per SM, bounded by the scratch buffers."""
    ctas = st.sm_count if max_ctas is None else max(1, min(int(max_ctas), st.sm_count))
    while ctas > 1 and lib.tgi_gemm_workspace_floats(M, ctas) > st.ws.numel():
        ctas -= 1
    if lib.tgi_gemm_num_tiles(M, N) > st.counters.numel():
        raise KernelError("GEMM has more output tiles than tile counters; raise the counter buffer size")
    return ctas


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, max_ctas: Optional[int] = None,
              out: Optional[torch.Tensor] = None):
    lib = load()
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    M, K = x2.shape
    N = w.shape[0]
    assert w.shape[1] == K and w.is_contiguous()
    if getattr(out, "is_peer_push", False):
        # row-parallel GEMM of a tensor-parallel group: rows go straight to their owners' peer memory
        if M == 0:
            return out
        assert out.T == M and out.N == N
        st = state(x.device)
        ctas = _gemm_ctas(lib, st, M, N, max_ctas)
        _check(lib.tgi_gemm_push(c_int(0), _ptr(x2), c_void_p(0), c_int(0), _ptr(w), c_void_p(0), _ptr(bias), c_int(M),
                                 c_int(N), c_int(K), c_int(ctas), _ptr(st.ws), _ptr(st.counters), _ptr(st.status),
                                 *out.gemm_args(), _stream()), "gemm_push")
        return out
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    else:
        assert out.numel() == M * N and out.dtype == torch.bfloat16 and out.is_contiguous()
    if M == 0:
        return out.reshape(*lead, N)
    st = state(x.device)
    ctas = _gemm_ctas(lib, st, M, N, max_ctas)
    _check(lib.tgi_gemm_bf16(_ptr(x2), _ptr(w), _ptr(out), _ptr(bias), c_int(M), c_int(N), c_int(K), c_int(ctas),
                             _ptr(st.ws), _ptr(st.counters), _ptr(st.status), _stream()), "gemm_bf16")
    return out.reshape(*lead, N)


def gemm_fp8_block(xq, xs, wq, ws, out_dtype=torch.bfloat16, bias=None, max_ctas: Optional[int] = None, out=None):
    lib = load()
    M, K = xq.shape
    N = wq.shape[0]
    assert wq.shape[1] == K and wq.is_contiguous() and xq.is_contiguous()
    assert out_dtype == torch.bfloat16
    if getattr(out, "is_peer_push", False):
        if M == 0:
            return out
        assert out.T == M and out.N == N
        st = state(xq.device)
        sptr, pitch = _scale_storage(xs)
        ctas = _gemm_ctas(lib, st, M, N, max_ctas)
        if not ws.is_contiguous():
            ws = ws.contiguous()
        _check(lib.tgi_gemm_push(c_int(1), _ptr(xq), c_void_p(sptr), c_int(pitch), _ptr(wq), _ptr(ws), _ptr(bias),
                                 c_int(M), c_int(N), c_int(K), c_int(ctas), _ptr(st.ws), _ptr(st.counters),
                                 _ptr(st.status), *out.gemm_args(), _stream()), "gemm_push")
        return out
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=xq.device)
    else:
        assert out.shape == (M, N) and out.dtype == torch.bfloat16 and out.is_contiguous()
    if M == 0:
        return out
    st = state(xq.device)
    sptr, pitch = _scale_storage(xs)
    ctas = _gemm_ctas(lib, st, M, N, max_ctas)
    if not ws.is_contiguous():
        ws = ws.contiguous()
    _check(lib.tgi_gemm_fp8_block(_ptr(xq), c_void_p(sptr), c_int(pitch), _ptr(wq), _ptr(ws), _ptr(out), _ptr(bias),
                                  c_int(M), c_int(N), c_int(K), c_int(ctas), _ptr(st.ws), _ptr(st.counters),
                                  _ptr(st.status), _stream()), "gemm_fp8_block")
    return out


# ---- norms -------------------------------------------------------------------------------------
def _norm(x, residual, weight, bias, eps, w_offset, layer, quant):
    lib = load()
    assert x.dtype == torch.bfloat16 and x.is_contiguous()
    T, H = x.shape
    res_out = torch.empty_like(x) if residual is not None else x
    out = q = scales = None
    if quant:
        q = torch.empty(T, H, dtype=FP8, device=x.device)
        scales = alloc_act_scales(T, H // 128, x.device)
        sptr, pitch = _scale_storage(scales)
    else:
        out = torch.empty_like(x)
        sptr, pitch = 0, 0
    _check(lib.tgi_norm(_ptr(x), _ptr(residual), _ptr(weight), _ptr(bias), _ptr(out),
                        _ptr(res_out if residual is not None else None), _ptr(q), c_void_p(sptr), c_int(pitch),
                        c_int(T), c_int(H), c_float(eps), c_float(w_offset), c_int(1 if layer else 0), _stream()),
           "norm")
    return out, q, scales, res_out


def rms_norm(x, residual, weight, eps, unit_offset=False):
    out, _, _, res = _norm(x, residual, weight, None, eps, 1.0 if unit_offset else 0.0, False, False)
    return out, res


def rms_norm_quant(x, residual, weight, eps, unit_offset=False):
    _, q, s, res = _norm(x, residual, weight, None, eps, 1.0 if unit_offset else 0.0, False, True)
    return q, s, res


def layer_norm(x, residual, weight, bias, eps):
    out, _, _, res = _norm(x, residual, weight, bias, eps, 0.0, True, False)
    return out, res


def qk_norm(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, q_weight: torch.Tensor,
            k_weight: torch.Tensor, eps: float, unit_offset: bool = False, layer: bool = False) -> torch.Tensor:
    """Per-head RMSNorm (or bias-free LayerNorm) of the q and k heads of ``qkv[T, (nh + 2 nkv) D]``, in place.  The
    weights are ``[D]`` (shared by the heads) or ``[heads, D]``."""
    lib = load()
    assert qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1
    qw = q_weight.to(torch.bfloat16).contiguous()
    kw = k_weight.to(torch.bfloat16).contiguous()
    _check(lib.tgi_qk_norm(_ptr(qkv), c_ll(qkv.stride(0)), c_int(qkv.shape[0]), c_int(num_heads), c_int(num_kv_heads),
                           c_int(head_dim), _ptr(qw), _ptr(kw), c_int(head_dim if qw.dim() > 1 else 0),
                           c_int(head_dim if kw.dim() > 1 else 0), ctypes.c_float(eps),
                           ctypes.c_float(1.0 if unit_offset else 0.0), c_int(1 if layer else 0), _stream()), "qk_norm")
    return qkv


# ---- activation --------------------------------------------------------------------------------
def act_and_mul(gate_up, act="silu"):
    lib = load()
    T, I2 = gate_up.shape
    I = I2 // 2
    out = torch.empty(T, I, dtype=gate_up.dtype, device=gate_up.device)
    _check(lib.tgi_act_mul(_ptr(gate_up.contiguous()), _ptr(out), c_void_p(0), c_void_p(0), c_int(0), c_int(T),
                           c_int(I), c_int(_ACT_CODES[act]), _stream()), "act_and_mul")
    return out


def act_and_mul_quant(gate_up, act="silu"):
    lib = load()
    T, I2 = gate_up.shape
    I = I2 // 2
    q = torch.empty(T, I, dtype=FP8, device=gate_up.device)
    scales = alloc_act_scales(T, I // 128, gate_up.device)
    sptr, pitch = _scale_storage(scales)
    _check(lib.tgi_act_mul(_ptr(gate_up.contiguous()), c_void_p(0), _ptr(q), c_void_p(sptr), c_int(pitch), c_int(T),
                           c_int(I), c_int(_ACT_CODES[act]), _stream()), "act_and_mul_quant")
    return q, scales


def fp8_quant_act(x, group=128):
    lib = load()
    assert group == 128 and x.dtype == torch.bfloat16
    x = x.contiguous()
    T, K = x.shape
    q = torch.empty(T, K, dtype=FP8, device=x.device)
    scales = alloc_act_scales(T, K // 128, x.device)
    sptr, pitch = _scale_storage(scales)
    _check(lib.tgi_quant_act(_ptr(x), _ptr(q), c_void_p(sptr), c_int(pitch), c_int(T), c_int(K), _stream()),
           "fp8_quant_act")
    return q, scales


# ---- rope + cache ------------------------------------------------------------------------------
def rope_and_cache(qkv, positions, cos_sin, slots, k_cache, v_cache, num_heads, num_kv_heads, head_dim, rot_dim,
                   neox=True, k_scale=None, v_scale=None):
    lib = load()
    T = qkv.shape[0]
    qkv = qkv.contiguous()
    q = torch.empty(T, num_heads, head_dim, dtype=qkv.dtype, device=qkv.device)
    fp8 = k_cache.dtype == FP8
    num_slots = k_cache.shape[0] * k_cache.shape[1]
    _check(lib.tgi_rope_cache(_ptr(qkv), _ptr(positions), _ptr(cos_sin), _ptr(slots), _ptr(q), _ptr(k_cache),
                              _ptr(v_cache), _ptr(k_scale if fp8 else None), _ptr(v_scale if fp8 else None),
                              c_int(T), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(rot_dim),
                              c_int(1 if neox else 0), c_ll(num_slots), c_int(1 if fp8 else 0),
                              c_int(cos_sin.shape[0]), _stream()),
           "rope_and_cache")
    return q


# ---- attention ---------------------------------------------------------------------------------
def paged_attention(q, k_cache, v_cache, block_tables, cu_seqlens_q, kv_lens, scale, window=-1, softcap=0.0,
                    k_scale=None, v_scale=None, max_q=None, max_kv=None, nsplit: Optional[int] = None, horizon=None):
    lib = load()
    T, Hq, D = q.shape
    nblk, bs, Hkv, _ = k_cache.shape
    B = kv_lens.shape[0]
    out = torch.empty_like(q)
    if T == 0 or B == 0:
        return out
    if max_q is None:
        max_q = int((cu_seqlens_q[1:] - cu_seqlens_q[:-1]).max().item())
    if max_kv is None:
        max_kv = int(kv_lens.max().item())
    fp8 = k_cache.dtype == FP8
    st = state(q.device)
    part_o = part_ml = None
    if max_q == 1:
        if nsplit is None:
            nsplit = lib.tgi_attn_decode_splits(B, Hkv, Hq // Hkv, max_kv, st.sm_count)
        if nsplit > 1:
            need = B * Hq * nsplit
            if st.attn_part_o is None or st.attn_part_o.numel() < need * D:
                st.attn_part_o = torch.empty(need * D, dtype=torch.float32, device=q.device)
                st.attn_part_ml = torch.empty(need * 2, dtype=torch.float32, device=q.device)
            part_o, part_ml = st.attn_part_o, st.attn_part_ml
    else:
        nsplit = 1
    _check(lib.tgi_paged_attention_ex(
        _ptr(q.contiguous()), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables), _ptr(cu_seqlens_q), _ptr(kv_lens),
        _ptr(k_scale if fp8 else None), _ptr(v_scale if fp8 else None), _ptr(out), _ptr(part_o), _ptr(part_ml),
        c_int(B), c_int(max_q), c_int(block_tables.shape[1]), c_int(bs), c_int(nblk), c_int(Hq), c_int(Hkv), c_int(D),
        c_float(scale), c_float(softcap), c_int(window if window and window > 0 else -1), c_int(nsplit),
        c_int(1 if fp8 else 0), _ptr(horizon), _stream()), "paged_attention")
    return out


# ---- misc --------------------------------------------------------------------------------------
def embedding(ids, table):
    lib = load()
    if table.dtype != torch.bfloat16:
        return torch.nn.functional.embedding(ids.long(), table)
    T = ids.numel()
    ids32 = ids if ids.dtype == torch.int32 else ids.to(torch.int32)
    out = torch.empty(T, table.shape[1], dtype=table.dtype, device=table.device)
    _check(lib.tgi_embedding(_ptr(ids32.contiguous()), _ptr(table), _ptr(out), c_int(T), c_int(table.shape[1]),
                             c_int(table.shape[0]), _stream()), "embedding")
    return out.view(*ids.shape, table.shape[1])


def argmax_logprob(logits):
    lib = load()
    assert logits.dim() == 2 and logits.stride(1) == 1
    B, V = logits.shape
    if logits.dtype not in (torch.bfloat16, torch.float32):
        logits = logits.float()
    ids = torch.empty(B, dtype=torch.int64, device=logits.device)
    lp = torch.empty(B, dtype=torch.float32, device=logits.device)
    _check(lib.tgi_argmax_logprob(_ptr(logits), _ptr(ids), _ptr(lp), c_int(B), c_int(V), c_ll(logits.stride(0)),
                                  c_int(1 if logits.dtype == torch.float32 else 0), _stream()), "argmax_logprob")
    return ids, lp


def fused_sample(scores: torch.Tensor, temperature=None, top_k=None, top_p=None, do_sample=None, seeds=None, steps=None,
                 typical_p=None):
    """Temperature, top-k, top-p and sampling (Gumbel-max with a counter-based generator keyed by the
    request's seed and step) in one kernel; returns ``(ids int64 [B], logprobs fp32 [B])``.  Any stage
    whose tensor is ``None`` is off; rows with ``do_sample == 0`` take the argmax of the filtered scores."""
    lib = load()
    assert scores.dim() == 2 and scores.stride(1) == 1 and scores.dtype in (torch.float32, torch.bfloat16)
    B, V = scores.shape
    dev = scores.device
    ids = torch.empty(B, dtype=torch.int64, device=dev)
    lps = torch.empty(B, dtype=torch.float32, device=dev)
    if B == 0:
        return ids, lps

    def as_(t, dtype):
        return None if t is None else t.to(device=dev, dtype=dtype).contiguous()

    temperature, top_p = as_(temperature, torch.float32), as_(top_p, torch.float32)
    typical_p = as_(typical_p, torch.float32)
    top_k, steps = as_(top_k, torch.int32), as_(steps, torch.int32)
    do_sample, seeds = as_(do_sample, torch.uint8), as_(seeds, torch.int64)
    _check(lib.tgi_sample(_ptr(scores), c_ll(scores.stride(0)), c_int(1 if scores.dtype == torch.float32 else 0),
                          _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(typical_p), _ptr(do_sample), _ptr(seeds),
                          _ptr(steps), _ptr(ids), _ptr(lps), c_int(B), c_int(V), _stream()), "sample")
    return ids, lps


# ---- weight-only quantised GEMM ------------------------------------------------------------------
_WQ_SCRATCH = {}


def _wq_partial(device) -> torch.Tensor:
    """fp32 workspace of the K-split partial tiles (shared by all layers of a device)."""
    key = ("partial", device.index)
    t = _WQ_SCRATCH.get(key)
    if t is None:
        t = torch.empty(int(os.environ.get("TGI_B200_WQ_WS_MB", "64")) << 18, dtype=torch.float32, device=device)
        _WQ_SCRATCH[key] = t
    return t


def gemm_wq(x: torch.Tensor, wq: torch.Tensor, scale: torch.Tensor, zp: Optional[torch.Tensor], group: int, bits: int,
            bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x[M, K] (bf16) @ dequant(wq)[N, K]^T`` with the weights dequantised on their way into shared memory:
    ``wq`` uint8 ``[N, K/2]`` (4-bit, low nibble first) or int8 ``[N, K]``; ``scale`` / ``zp`` fp16 ``[K/group, N]``."""
    lib = load()
    st = state(x.device)
    M, K = x.shape
    N = wq.shape[0]
    out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    part = _wq_partial(x.device)
    x = x.contiguous()
    xh = torch.empty(M, K, dtype=torch.float16, device=x.device)       # fp16 copy of the tokens, written by the call
    _check(lib.tgi_gemm_wq(c_int(bits), _ptr(x), _ptr(xh), _ptr(wq), _ptr(scale), _ptr(zp), c_int(group), _ptr(out),
                           _ptr(part), c_ll(part.numel()), _ptr(bias), c_int(M), c_int(N), c_int(K), c_int(st.sm_count),
                           _ptr(st.status), _stream()), "gemm_wq")
    return out


def wq_dequant(wq: torch.Tensor, scale: torch.Tensor, zp: Optional[torch.Tensor], group: int, bits: int, K: int,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """bf16 ``[N, K]`` matrix of a packed weight (the numbers the fused GEMM feeds to the tensor cores)."""
    lib = load()
    N = wq.shape[0]
    if out is None:
        out = torch.empty(N, K, dtype=torch.bfloat16, device=wq.device)
    _check(lib.tgi_wq_dequant(c_int(bits), _ptr(wq), _ptr(scale), _ptr(zp), c_int(group), _ptr(out), c_int(N), c_int(K),
                              _stream()), "wq_dequant")
    return out


def wq_dequant_scratch(wq, scale, zp, group, bits, K) -> torch.Tensor:
    """Dequantise into a per-device scratch matrix that the next call overwrites (prefill-sized GEMMs)."""
    N = wq.shape[0]
    key = ("dequant", wq.device.index)
    t = _WQ_SCRATCH.get(key)
    if t is None or t.numel() < N * K:
        t = torch.empty(N * K, dtype=torch.bfloat16, device=wq.device)
        _WQ_SCRATCH[key] = t
    return wq_dequant(wq, scale, zp, group, bits, K, out=t[: N * K].view(N, K))


def penalties(logits: torch.Tensor, history: torch.Tensor, repetition_penalty: Optional[torch.Tensor],
              frequency_penalty: Optional[torch.Tensor], vocab_start: int = 0, logit_scale: float = 1.0) -> torch.Tensor:
    """fp32 copy of ``logits[B, V]`` (bf16 or fp32; ``V`` may be a vocabulary slice starting at ``vocab_start``) with
    the repetition and frequency penalties of the rows' token ``history[B, L]`` applied, in one kernel."""
    lib = load()
    B, V = logits.shape
    assert logits.stride(1) == 1 and logits.dtype in (torch.bfloat16, torch.float32)
    out = torch.empty(B, V, dtype=torch.float32, device=logits.device)
    history = history.to(device=logits.device, dtype=torch.int64).contiguous()
    rep = None if repetition_penalty is None else repetition_penalty.to(torch.float32).contiguous()
    freq = None if frequency_penalty is None else frequency_penalty.to(torch.float32).contiguous()
    _check(lib.tgi_penalties(_ptr(logits), c_int(1 if logits.dtype == torch.float32 else 0), c_ll(logits.stride(0)),
                             _ptr(out), c_ll(V), _ptr(history), c_int(history.shape[1]), _ptr(rep), _ptr(freq),
                             c_int(vocab_start), c_int(B), c_int(V), ctypes.c_float(logit_scale), _stream()), "penalties")
    return out


def moe_topk_softmax(router_logits: torch.Tensor, top_k: int, renormalize: bool = True):
    """Softmax over the router logits and top-k selection in one kernel: ``(weights fp32 [T, k], ids int32 [T, k])``."""
    lib = load()
    T, E = router_logits.shape
    if router_logits.dtype not in (torch.float32, torch.bfloat16):
        router_logits = router_logits.float()
    router_logits = router_logits.contiguous()
    w = torch.empty(T, top_k, dtype=torch.float32, device=router_logits.device)
    ids = torch.empty(T, top_k, dtype=torch.int32, device=router_logits.device)
    _check(lib.tgi_moe_topk_softmax(_ptr(router_logits), c_int(1 if router_logits.dtype == torch.float32 else 0), c_int(T),
                                    c_int(E), c_int(top_k), c_int(1 if renormalize else 0), _ptr(w), _ptr(ids), _stream()),
           "moe_topk_softmax")
    return w, ids


def moe_experts(x, w_gate_up, w_down, topk_weights, topk_ids, act="silu", first: int = 0):
    """Routed expert MLPs of the experts ``first .. first + E_local - 1`` held in ``w_gate_up [E_local, 2I, H]`` /
    ``w_down [E_local, H, I]``: ``out[t] = sum_slot w[t, slot] * MLP_{id[t, slot]}(x[t])`` over the slots whose
    expert is local.  Five launches (group, gather, two grouped tcgen05 GEMMs with the activation and the routing
    weight fused into their epilogues, combine), no host synchronisation, fixed buffer shapes: the whole sequence
    is CUDA-graph capturable and only routed rows are computed."""
    lib = load()
    st = state(x.device)
    T, H = x.shape
    E_local, I2, _ = w_gate_up.shape
    I = I2 // 2
    k = topk_ids.shape[1]
    entries = T * k
    dev = x.device
    if T == 0:
        return torch.zeros(0, H, dtype=x.dtype, device=dev)
    assert x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and w_down.dtype == torch.bfloat16
    assert w_gate_up.is_contiguous() and w_down.is_contiguous() and tuple(w_down.shape) == (E_local, H, I)
    ids = topk_ids.to(torch.int32).contiguous()
    tw = topk_weights.to(torch.float32).contiguous()
    pos = torch.empty(entries, dtype=torch.int32, device=dev)
    order = torch.empty(entries, dtype=torch.int32, device=dev)
    offsets = torch.empty(E_local + 1, dtype=torch.int32, device=dev)
    grouped = torch.empty(entries, H, dtype=torch.bfloat16, device=dev)
    hidden = torch.empty(entries, I, dtype=torch.bfloat16, device=dev)
    y = torch.empty(entries, H, dtype=torch.bfloat16, device=dev)
    out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    s = _stream()
    x = x.contiguous()
    _check(lib.tgi_moe_sort(_ptr(ids), c_int(entries), c_int(first), c_int(E_local), _ptr(pos), _ptr(order), _ptr(offsets),
                            s), "moe_sort")
    _check(lib.tgi_moe_gather(_ptr(x), _ptr(order), _ptr(offsets), c_int(E_local), c_int(k), c_int(H), c_int(entries),
                              _ptr(grouped), s), "moe_gather")
    _check(lib.tgi_moe_grouped_gemm(c_int(0), _ptr(grouped), c_int(entries), _ptr(w_gate_up), c_int(E_local), c_int(I2),
                                    c_int(H), _ptr(offsets), c_int(_ACT_CODES[act]), c_void_p(0), c_void_p(0),
                                    _ptr(hidden), c_int(st.sm_count), _ptr(st.status), s), "moe_grouped_gemm(gate_up)")
    _check(lib.tgi_moe_grouped_gemm(c_int(1), _ptr(hidden), c_int(entries), _ptr(w_down), c_int(E_local), c_int(H),
                                    c_int(I), _ptr(offsets), c_int(0), _ptr(tw), _ptr(order), _ptr(y),
                                    c_int(st.sm_count), _ptr(st.status), s), "moe_grouped_gemm(down)")
    _check(lib.tgi_moe_combine(_ptr(y), _ptr(pos), c_int(T), c_int(k), c_int(H), _ptr(out), s), "moe_combine")
    return out


# ---- multi-adapter LoRA ------------------------------------------------------------------------
def lora_shrink(x: torch.Tensor, a_ptrs: torch.Tensor, ranks: torch.Tensor, token_adapter: torch.Tensor,
                rmax: int) -> torch.Tensor:
    """``v[t] = A_{adapter(t)} x[t]`` in fp32, ``[T, rmax]`` (zero rows for tokens without adapter)."""
    T, H = x.shape
    v = torch.empty(T, rmax, dtype=torch.float32, device=x.device)
    _check(load().tgi_lora_shrink(_ptr(x.contiguous()), _ptr(a_ptrs), _ptr(ranks), _ptr(token_adapter), _ptr(v),
                                  c_int(T), c_int(H), c_int(rmax), _stream()), "lora_shrink")
    return v


def lora_expand(v: torch.Tensor, b_ptrs: torch.Tensor, ranks: torch.Tensor, scales: torch.Tensor,
                token_adapter: torch.Tensor, out: torch.Tensor, col0: int, ncols: int):
    """``out[t, col0:col0+ncols] += scale * B_{adapter(t)} v[t]`` in place (``out`` bf16, rows contiguous)."""
    T, rmax = v.shape
    if out.stride(1) != 1:
        raise KernelError("lora_expand needs unit stride along the columns of `out`")
    _check(load().tgi_lora_expand(_ptr(v), _ptr(b_ptrs), _ptr(ranks), _ptr(scales), _ptr(token_adapter), _ptr(out),
                                  c_ll(out.stride(0)), c_int(col0), c_int(T), c_int(ncols), c_int(rmax), _stream()),
           "lora_expand")
