"""Quantisation config discovery and weight-loading strategies.

Role of the reference's ``utils/quantization.py`` (``_get_quantizer_config``
``:47-121`` and ``get_loader`` ``:124-221``), ``layers/fp8.py`` loader
(``:187-396``), ``layers/gptq/__init__.py`` loader (``:93-479``),
``layers/eetq.py``, ``layers/bnb.py``, ``layers/exl2.py``, ``layers/marlin/*``
and ``layers/compressed_tensors/*``.

A *loader* turns checkpoint tensors of one linear layer into a *weight object*;
the weight object's ``get_linear(bias)`` returns the callable used in the
forward pass (``models/layers.py``).  Formats:

========================= ============================================================
``None``                  bf16/fp16 tensors as they are
``fp8``                   e4m3 checkpoints (per-tensor, per-channel, 128x128 block
                          scales ``weight_scale_inv``) or on-the-fly conversion
``gptq`` / ``awq``        int4/int8 packed ``qweight/qzeros/scales/g_idx``
``marlin``                same checkpoints as gptq/awq (repacking is an
                          implementation detail of another kernel family)
``exl2``                  ``q_weight/q_scale/q_invperm/q_scale_max/q_groups``
``eetq`` / ``bitsandbytes*``  on-the-fly int8 / nf4 / fp4 weight-only quantisation
``compressed-tensors``    config groups mapping to fp8 / int8 / packed int4
========================= ============================================================

On B200 the tensor-core native formats are bf16 and e4m3, so weight-only integer
formats are unpacked to bf16 once at load (``dequantize()``) unless a dedicated
kernel is registered; the *checkpoint format support* is complete, the memory
saving of int4 is traded for bf16 tensor-core throughput.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from pathlib import Path
from typing import List, Optional, Sequence, Union

import torch

from ..ops import reference as ref

FP8 = torch.float8_e4m3fn


# ---------------------------------------------------------------------------------------------
# weight objects
# ---------------------------------------------------------------------------------------------
class Weight:
    def get_linear(self, bias: Optional[torch.Tensor]):
        raise NotImplementedError


@dataclass
class UnquantizedWeight(Weight):
    weight: torch.Tensor

    def get_linear(self, bias):
        from ..models.layers import FastLinear

        return FastLinear(self.weight, bias)


@dataclass
class Fp8Weight(Weight):
    """e4m3 weight.  ``weight_scale`` is per-tensor ``[]``, per-channel ``[N]`` or per-block ``[N/128,K/128]``."""

    weight: torch.Tensor
    dtype: torch.dtype
    weight_scale: Optional[torch.Tensor] = None
    input_scale: Optional[torch.Tensor] = None
    activation_scale_ub: Optional[float] = None
    weight_block_size: Optional[Sequence[int]] = None
    force_block: bool = True

    def get_linear(self, bias):
        from ..models.layers import Fp8Linear

        w, s, blk = self.weight, self.weight_scale, self.weight_block_size
        if s is None:
            # Unquantised tensor handed to an fp8 loader (``--quantize fp8``): convert now.  Block
            # scales are the native format of the sm_100a GEMM, so on-the-fly conversion uses them.
            if self.force_block and w.shape[1] % 128 == 0:
                w, s = ref.fp8_quant_block_weight(w.float())
                blk = [128, 128]
            else:
                w, s = ref.fp8_quant_per_tensor(w)
        return Fp8Linear(w, s, bias, self.dtype, self.input_scale, self.activation_scale_ub, blk)


@dataclass
class GPTQWeight(Weight):
    """Packed int (2/3/4/8-bit) weight in GPTQ (``awq=False``) or AWQ (``awq=True``) layout."""

    qweight: torch.Tensor
    qzeros: torch.Tensor
    scales: torch.Tensor
    g_idx: Optional[torch.Tensor]
    bits: int
    groupsize: int
    awq: bool = False
    sym: bool = False
    dtype: torch.dtype = torch.bfloat16

    def dequantize(self) -> torch.Tensor:
        return dequantize_gptq(self)

    def get_linear(self, bias):
        from ..models.layers import FastLinear, PackedQuantLinear

        packed = pack_gptq_for_kernel(self)
        if packed is not None:     # 4-bit (8-bit) weights stay packed on the device and are dequantised inside the GEMM
            return PackedQuantLinear(*packed, bias=bias, dtype=self.dtype)
        return FastLinear(self.dequantize().to(self.dtype), bias)


@dataclass
class Exl2Weight(Weight):
    q_weight: torch.Tensor
    q_scale: torch.Tensor
    q_invperm: torch.Tensor
    q_scale_max: torch.Tensor
    q_groups: torch.Tensor
    dtype: torch.dtype = torch.bfloat16

    def get_linear(self, bias):
        from ..models.layers import FastLinear

        return FastLinear(dequantize_exl2(self).to(self.dtype), bias)


@dataclass
class Int8Weight(Weight):
    """Weight-only int8, one scale per output channel (EETQ, bitsandbytes int8, compressed-tensors W8A16)."""

    qweight: torch.Tensor
    scale: torch.Tensor
    dtype: torch.dtype

    @classmethod
    def quantize(cls, w: torch.Tensor, dtype) -> "Int8Weight":
        s = w.float().abs().amax(dim=1, keepdim=True).clamp_min(1e-8) / 127.0
        return cls((w.float() / s).round().clamp(-127, 127).to(torch.int8), s.squeeze(1), dtype)

    def dequantize(self):
        return (self.qweight.float() * self.scale.float().unsqueeze(1)).to(self.dtype)

    def get_linear(self, bias):
        from ..models.layers import FastLinear, PackedQuantLinear

        N, K = self.qweight.shape
        if K % 64 == 0 and N % 8 == 0 and self.dtype == torch.bfloat16 and float(self.scale.abs().max()) < 6e4:
            scale = self.scale.float().view(1, N).to(torch.float16).contiguous()
            return PackedQuantLinear(self.qweight.contiguous(), scale, None, K, 8, None, K, bias=bias, dtype=self.dtype)
        return FastLinear(self.dequantize(), bias)


_NF4 = [-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
        -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
        0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941,
        0.7229568362236023, 1.0]
_FP4 = [0.0, 0.0052083333, 0.6666667, 1.0, 0.3333333, 0.5, 0.1666667, 0.25,
        -0.0, -0.0052083333, -0.6666667, -1.0, -0.3333333, -0.5, -0.1666667, -0.25]


@dataclass
class Codebook4Weight(Weight):
    """4-bit codebook quantisation with absmax per 64-element block (bitsandbytes NF4 / FP4)."""

    codes: torch.Tensor  # uint8, two codes per byte
    absmax: torch.Tensor
    shape: tuple
    kind: str
    dtype: torch.dtype
    blocksize: int = 64

    @classmethod
    def quantize(cls, w: torch.Tensor, kind: str, dtype, blocksize: int = 64) -> "Codebook4Weight":
        book = torch.tensor(_NF4 if kind == "nf4" else _FP4, dtype=torch.float32, device=w.device)
        flat = w.float().reshape(-1)
        pad = (-flat.numel()) % blocksize
        if pad:
            flat = torch.cat([flat, flat.new_zeros(pad)])
        blocks = flat.view(-1, blocksize)
        absmax = blocks.abs().amax(dim=1, keepdim=True).clamp_min(1e-12)
        idx = ((blocks / absmax).unsqueeze(-1) - book).abs().argmin(dim=-1).to(torch.uint8).reshape(-1)
        codes = (idx[0::2] << 4) | idx[1::2]
        return cls(codes, absmax.squeeze(1), tuple(w.shape), kind, dtype, blocksize)

    def dequantize(self):
        book = torch.tensor(_NF4 if self.kind == "nf4" else _FP4, dtype=torch.float32, device=self.codes.device)
        idx = torch.stack([self.codes >> 4, self.codes & 0xF], dim=1).reshape(-1).long()
        vals = book[idx].view(-1, self.blocksize) * self.absmax.unsqueeze(1)
        n = 1
        for s in self.shape:
            n *= s
        return vals.reshape(-1)[:n].view(self.shape).to(self.dtype)

    def get_linear(self, bias):
        from ..models.layers import FastLinear

        return FastLinear(self.dequantize(), bias)


# ---------------------------------------------------------------------------------------------
# unpacking helpers
# ---------------------------------------------------------------------------------------------
_AWQ_ORDER = [0, 4, 1, 5, 2, 6, 3, 7]


def _unpack_int32(packed: torch.Tensor, bits: int, dim: int) -> torch.Tensor:
    """Unpack ``32/bits`` little-endian fields from each int32 along ``dim``."""
    per = 32 // bits
    shifts = torch.arange(0, 32, bits, device=packed.device, dtype=torch.int32)[:per]
    mask = (1 << bits) - 1
    if dim == 0:
        out = (packed.unsqueeze(1) >> shifts.view(1, -1, 1)) & mask
        return out.reshape(packed.shape[0] * per, packed.shape[1])
    out = (packed.unsqueeze(2) >> shifts.view(1, 1, -1)) & mask
    return out.reshape(packed.shape[0], packed.shape[1] * per)


def _pack_int32(vals: torch.Tensor, bits: int, dim: int) -> torch.Tensor:
    """Inverse of ``_unpack_int32``: ``32/bits`` little-endian fields per int32 along ``dim`` (0 or 1)."""
    per = 32 // bits
    v = vals.to(torch.int64) & ((1 << bits) - 1)
    shifts = torch.arange(0, 32, bits, device=vals.device, dtype=torch.int64)[:per]
    if dim == 0:
        v = v.view(vals.shape[0] // per, per, vals.shape[1])
        word = (v << shifts.view(1, -1, 1)).sum(1)
    else:
        v = v.view(vals.shape[0], vals.shape[1] // per, per)
        word = (v << shifts.view(1, 1, -1)).sum(2)
    word = torch.where(word >= (1 << 31), word - (1 << 32), word)        # two's complement of the top field
    return word.to(torch.int32)


def pack_gptq_for_kernel(w: "GPTQWeight"):
    """Canonical packed form of a 4-bit GPTQ / AWQ layer for the weight-only GEMM (``ops/csrc/gemm_wq_sm100.cu``), or
    ``None`` when the layer does not fit it (other bit widths, group sizes that are no multiple of 64, odd shapes).

    Returns ``(wq uint8 [N, K/2], scale fp16 [G, N], zp fp16 [G, N], group, bits, perm, K)``: element ``k`` of output
    row ``n`` sits in byte ``k // 2`` (even ``k`` in the low nibble) and equals ``(q - zp[k // group, n]) * scale``.
    With activation ordering (``g_idx`` not sorted) the K axis is reordered once so that groups are contiguous;
    ``perm`` then tells the linear how to permute the activations' columns (reference: the exllama kernels'
    ``column_remap``, ``server/exllama_kernels/exllama_kernels/cuda_func/column_remap.cu``).
    """
    if w.bits != 4 or w.dtype != torch.bfloat16:
        return None
    bits = 4
    if w.awq:
        iw = _unpack_int32(w.qweight, bits, dim=1)
        iz = _unpack_int32(w.qzeros, bits, dim=1)
        inv = torch.tensor(_AWQ_ORDER, device=iw.device).argsort()
        iw = iw.view(iw.shape[0], -1, 8)[:, :, inv].reshape(iw.shape[0], -1)
        zeros = iz.view(iz.shape[0], -1, 8)[:, :, inv].reshape(iz.shape[0], -1)
    else:
        iw = _unpack_int32(w.qweight, bits, dim=0)
        zeros = _unpack_int32(w.qzeros, bits, dim=1) + 1
    K, N = iw.shape
    group = w.groupsize if w.groupsize > 0 else K
    if K % 64 != 0 or group % 64 != 0 or N % 8 != 0 or K % group != 0:
        return None
    perm = None
    if w.g_idx is not None and not w.awq:
        gi = w.g_idx.long()
        if not bool((gi[1:] >= gi[:-1]).all()):
            perm = torch.argsort(gi, stable=True)
            if not torch.equal(gi[perm], torch.arange(K, device=gi.device) // group):
                return None      # groups of unequal size: leave it to the dequantised path
            iw = iw[perm]
    scales = w.scales.float()
    if float(scales.abs().max()) >= 6e4:
        return None
    wt = iw.t().contiguous().to(torch.uint8)                       # [N, K]
    wq = (wt[:, 0::2] | (wt[:, 1::2] << 4)).contiguous()
    zp = zeros[:, :N].to(torch.float16).contiguous()
    return wq, scales.to(torch.float16).contiguous(), zp, group, bits, perm, K


def dequantize_gptq(w: GPTQWeight) -> torch.Tensor:
    """Return the ``[N_out, K_in]`` floating matrix of a GPTQ or AWQ layer.

    GPTQ: ``qweight[K/pack, N]`` packed along K, ``qzeros[G, N/pack]``, stored zero is ``z-1``.
    AWQ:  ``qweight[K, N/pack]`` packed along N with the nibble order 0,4,1,5,2,6,3,7, zero stored as is.
    """
    bits = w.bits
    if w.awq:
        iw = _unpack_int32(w.qweight, bits, dim=1)
        iz = _unpack_int32(w.qzeros, bits, dim=1)
        per = 32 // bits
        if bits == 4:
            inv = torch.tensor(_AWQ_ORDER, device=iw.device).argsort()
            iw = iw.view(iw.shape[0], -1, per)[:, :, inv].reshape(iw.shape[0], -1)
            iz = iz.view(iz.shape[0], -1, per)[:, :, inv].reshape(iz.shape[0], -1)
        zeros = iz
    else:
        iw = _unpack_int32(w.qweight, bits, dim=0)
        zeros = _unpack_int32(w.qzeros, bits, dim=1) + 1
    K, N = iw.shape
    groupsize = w.groupsize if w.groupsize > 0 else K
    if w.g_idx is not None and not w.awq:
        gi = w.g_idx.long()
    else:
        gi = torch.arange(K, device=iw.device) // groupsize
    scales = w.scales.float()[gi]  # [K, N]
    z = zeros[:, :N].float()[gi]
    return ((iw.float() - z) * scales).t().contiguous()


def dequantize_exl2(w: Exl2Weight) -> torch.Tensor:
    """Unpack an EXL2 mixed-bit-width matrix (rows grouped by bit width) to ``[N_out, K_in]``.

    ``q_groups`` holds ``(bits, first_packed_row)`` per group, ``q_scale`` 4-bit packed group scales
    squared and multiplied by ``q_scale_max``; ``q_invperm`` undoes the row permutation.
    """
    groups = w.q_groups.view(-1, 2).tolist()
    N = w.q_weight.shape[1]
    K = w.q_invperm.shape[0]
    ngroups = len(groups)
    gsize = K // ngroups if ngroups else K
    qs = _unpack_int32(w.q_scale, 4, dim=1)[:, :N].float() + 1
    scale = qs * qs * (w.q_scale_max.float().view(-1, 1) / 256.0)
    rows = []
    for g, (bits, start) in enumerate(groups):
        nrows_packed = gsize * bits // 32
        blk = w.q_weight[start : start + nrows_packed]
        if 32 % bits == 0:
            vals = _unpack_int32(blk, bits, dim=0)
        else:  # 3/5/6-bit rows: read fields out of the concatenated bit stream
            words = blk.to(torch.int64) & 0xFFFFFFFF
            k = torch.arange(gsize, device=blk.device)
            bitpos = k * bits
            wi, off = bitpos // 32, bitpos % 32
            lo = words[wi] >> off.view(-1, 1)
            hi = torch.where(
                (off + bits > 32).view(-1, 1), words[(wi + 1).clamp(max=words.shape[0] - 1)] << (32 - off).view(-1, 1), 0
            )
            vals = ((lo | hi) & ((1 << bits) - 1)).to(torch.int32)
        centre = 1 << (bits - 1)
        rows.append((vals.float() - centre) * scale[g].view(1, -1))
    full = torch.cat(rows, dim=0)[:K]
    return full[w.q_invperm.long()].t().contiguous()


# ---------------------------------------------------------------------------------------------
# loaders
# ---------------------------------------------------------------------------------------------
class WeightsLoader:
    def get_weights(self, weights, prefix: str) -> Weight:
        raise NotImplementedError

    def get_weights_col_packed(self, weights, prefix: str, block_sizes) -> Weight:
        raise NotImplementedError

    def get_weights_col(self, weights, prefix: str) -> Weight:
        return self.get_multi_weights_col(weights, [prefix], 0)

    def get_multi_weights_col(self, weights, prefixes: List[str], dim: int) -> Weight:
        raise NotImplementedError

    def get_weights_row(self, weights, prefix: str) -> Weight:
        raise NotImplementedError


class DefaultWeightsLoader(WeightsLoader):
    def __init__(self, weight_class=UnquantizedWeight):
        self.weight_class = weight_class

    def get_weights(self, weights, prefix):
        return self.weight_class(weights.get_tensor(f"{prefix}.weight"))

    def get_weights_col_packed(self, weights, prefix, block_sizes):
        return self.weight_class(weights.get_packed_sharded(f"{prefix}.weight", 0, block_sizes))

    def get_multi_weights_col(self, weights, prefixes, dim):
        w = [weights.get_sharded(f"{p}.weight", dim=0) for p in prefixes]
        return self.weight_class(torch.cat(w, dim=dim) if len(w) > 1 else w[0])

    def get_weights_row(self, weights, prefix):
        return self.weight_class(weights.get_sharded(f"{prefix}.weight", dim=1))


class OnTheFlyLoader(DefaultWeightsLoader):
    """Load unquantised tensors and quantise them at load (eetq, bitsandbytes, bitsandbytes-nf4/fp4)."""

    def __init__(self, kind: str):
        def make(w):
            if kind in ("eetq", "bitsandbytes"):
                return Int8Weight.quantize(w, w.dtype)
            return Codebook4Weight.quantize(w, "nf4" if kind.endswith("nf4") else "fp4", w.dtype)

        super().__init__(make)
        self.kind = kind


class Fp8Loader(WeightsLoader):
    """fp8 checkpoints and ``--quantize fp8`` (the reference's ``HybridFP8UnquantLoader``)."""

    def __init__(self, activation_scale_ub: Optional[float] = None, to_fp8: bool = False,
                 weight_block_size: Optional[Sequence[int]] = None):
        self.activation_scale_ub = activation_scale_ub
        self.to_fp8 = to_fp8
        self.weight_block_size = list(weight_block_size) if weight_block_size else None

    # scale helpers -------------------------------------------------------------------------
    def _wrap(self, weights, w, scale=None, input_scale=None, block=None) -> Weight:
        if w.dtype == FP8:
            return Fp8Weight(w, weights.dtype, scale, input_scale, self.activation_scale_ub, block)
        if self.to_fp8:
            return Fp8Weight(w, weights.dtype, activation_scale_ub=self.activation_scale_ub)
        return UnquantizedWeight(w)

    @staticmethod
    def _input_scale(weights, prefix) -> Optional[torch.Tensor]:
        if weights.has_tensor(f"{prefix}.input_scale"):
            return weights.get_tensor(f"{prefix}.input_scale", to_dtype=False).float().reshape(-1).max()
        return None

    def _block_scale_shard(self, weights, prefix, dim, exact=True):
        """Shard of ``weight_scale_inv`` matching a weight shard along ``dim``."""
        name = f"{prefix}.weight_scale_inv"
        full_w = weights.get_shape(f"{prefix}.weight")
        world, rank = weights.process_group.size(), weights.process_group.rank()
        per = full_w[dim] // world
        blk = self.weight_block_size[dim]
        if per % blk != 0 and world > 1:
            raise ValueError(f"{prefix}: shard of {per} rows is not a multiple of the {blk}-wide scale block")
        sl = weights._slice(name)
        t = sl.slice_dim(dim, rank * per // blk, (rank + 1) * per // blk)
        return weights._finish(t, True, False).float()

    def get_weights(self, weights, prefix):
        w = weights.get_tensor(f"{prefix}.weight")
        if w.dtype != FP8:
            return self._wrap(weights, w)
        if self.weight_block_size is not None and weights.has_tensor(f"{prefix}.weight_scale_inv"):
            s = weights.get_tensor(f"{prefix}.weight_scale_inv", to_dtype=False).float()
            return self._wrap(weights, w, s, None, self.weight_block_size)
        s = weights.get_tensor(f"{prefix}.weight_scale", to_dtype=False).float()
        return self._wrap(weights, w, s.reshape(-1) if s.numel() > 1 else s.reshape(()), self._input_scale(weights, prefix))

    def get_weights_col_packed(self, weights, prefix, block_sizes):
        w = weights.get_packed_sharded(f"{prefix}.weight", 0, block_sizes)
        if w.dtype != FP8:
            return self._wrap(weights, w)
        if self.weight_block_size is not None and weights.has_tensor(f"{prefix}.weight_scale_inv"):
            s = weights.get_packed_sharded(f"{prefix}.weight_scale_inv", 0, block_sizes, to_dtype=False).float()
            return self._wrap(weights, w, s, None, self.weight_block_size)
        s = weights.get_tensor(f"{prefix}.weight_scale", to_dtype=False)
        if s.numel() > 1:
            s = weights.get_packed_sharded(f"{prefix}.weight_scale", 0, block_sizes, to_dtype=False)
        s = s.float().reshape(-1) if s.numel() > 1 else s.float().reshape(())
        return self._wrap(weights, w, s, self._input_scale(weights, prefix))

    def get_multi_weights_col(self, weights, prefixes, dim):
        ws = [weights.get_sharded(f"{p}.weight", dim=0, to_device=False) for p in prefixes]
        w = (torch.cat([x.view(torch.uint8) for x in ws], dim=dim).view(ws[0].dtype) if ws[0].dtype == FP8
             else torch.cat(ws, dim=dim)).to(weights.device)
        if w.dtype != FP8:
            return self._wrap(weights, w)
        if self.weight_block_size is not None and weights.has_tensor(f"{prefixes[0]}.weight_scale_inv"):
            s = torch.cat([self._block_scale_shard(weights, p, 0) for p in prefixes], dim=dim)
            return self._wrap(weights, w, s, None, self.weight_block_size)
        scales = []
        for p, x in zip(prefixes, ws):
            s = weights.get_tensor(f"{p}.weight_scale", to_dtype=False).float()
            if s.numel() > 1:
                s = weights.get_sharded(f"{p}.weight_scale", dim=0, to_dtype=False).float().reshape(-1)
            else:  # per-tensor scales of the fused parts differ: widen to per-channel
                s = s.reshape(1).expand(x.shape[0])
            scales.append(s.to(weights.device))
        in_scales = [self._input_scale(weights, p) for p in prefixes]
        in_scale = torch.stack([s for s in in_scales if s is not None]).max() if any(
            s is not None for s in in_scales) else None
        return self._wrap(weights, w, torch.cat(scales), in_scale)

    def get_weights_row(self, weights, prefix):
        w = weights.get_sharded(f"{prefix}.weight", dim=1)
        if w.dtype != FP8:
            return self._wrap(weights, w)
        if self.weight_block_size is not None and weights.has_tensor(f"{prefix}.weight_scale_inv"):
            s = self._block_scale_shard(weights, prefix, 1)
            return self._wrap(weights, w, s, None, self.weight_block_size)
        s = weights.get_tensor(f"{prefix}.weight_scale", to_dtype=False).float()
        s = s.reshape(-1) if s.numel() > 1 else s.reshape(())
        return self._wrap(weights, w, s, self._input_scale(weights, prefix))


class GPTQLoader(WeightsLoader):
    """GPTQ / AWQ packed-int checkpoints (also what the reference's Marlin loaders read)."""

    def __init__(self, bits: int, groupsize: int, desc_act: bool, quant_method: str, sym: bool = False,
                 modules_to_not_convert: Optional[List[str]] = None):
        self.bits, self.groupsize, self.desc_act = bits, groupsize, desc_act
        self.quant_method, self.sym = quant_method, sym
        self.modules_to_not_convert = modules_to_not_convert or []

    @property
    def awq(self):
        return self.quant_method == "awq"

    def _skip(self, prefix: str) -> bool:
        return any(m in prefix for m in self.modules_to_not_convert)

    def _mk(self, weights, qweight, qzeros, scales, g_idx) -> GPTQWeight:
        return GPTQWeight(qweight, qzeros, scales, g_idx, self.bits, self.groupsize, self.awq, self.sym, weights.dtype)

    def get_weights(self, weights, prefix):
        if self._skip(prefix) or not weights.has_tensor(f"{prefix}.qweight"):
            return DefaultWeightsLoader().get_weights(weights, prefix)
        g_idx = None if self.awq or not weights.has_tensor(f"{prefix}.g_idx") else weights.get_tensor(
            f"{prefix}.g_idx", to_dtype=False)
        return self._mk(weights, weights.get_tensor(f"{prefix}.qweight", to_dtype=False),
                        weights.get_tensor(f"{prefix}.qzeros", to_dtype=False),
                        weights.get_tensor(f"{prefix}.scales"), g_idx)

    def get_weights_col_packed(self, weights, prefix, block_sizes):
        if self._skip(prefix) or not weights.has_tensor(f"{prefix}.qweight"):
            return DefaultWeightsLoader().get_weights_col_packed(weights, prefix, block_sizes)
        qweight = weights.get_packed_sharded(f"{prefix}.qweight", 1, block_sizes, to_dtype=False)
        qzeros = weights.get_packed_sharded(f"{prefix}.qzeros", 1, block_sizes, to_dtype=False)
        scales = weights.get_packed_sharded(f"{prefix}.scales", 1, block_sizes)
        g_idx = None if self.awq or not weights.has_tensor(f"{prefix}.g_idx") else weights.get_tensor(
            f"{prefix}.g_idx", to_dtype=False)
        return self._mk(weights, qweight, qzeros, scales, g_idx)

    def get_multi_weights_col(self, weights, prefixes, dim):
        if self._skip(prefixes[0]) or not weights.has_tensor(f"{prefixes[0]}.qweight"):
            return DefaultWeightsLoader().get_multi_weights_col(weights, prefixes, dim)
        qweight = torch.cat([weights.get_sharded(f"{p}.qweight", 1, to_dtype=False) for p in prefixes], dim=1)
        qzeros = torch.cat([weights.get_sharded(f"{p}.qzeros", 1, to_dtype=False) for p in prefixes], dim=1)
        scales = torch.cat([weights.get_sharded(f"{p}.scales", 1) for p in prefixes], dim=1)
        g_idx = None
        if not self.awq and weights.has_tensor(f"{prefixes[0]}.g_idx"):
            gs = [weights.get_tensor(f"{p}.g_idx", to_dtype=False) for p in prefixes]
            for g in gs[1:]:
                if not torch.equal(g, gs[0]):
                    raise ValueError("fused GPTQ projections must share g_idx")
            g_idx = gs[0]
        return self._mk(weights, qweight, qzeros, scales, g_idx)

    def get_weights_row(self, weights, prefix):
        if self._skip(prefix) or not weights.has_tensor(f"{prefix}.qweight"):
            return DefaultWeightsLoader().get_weights_row(weights, prefix)
        world, rank = weights.process_group.size(), weights.process_group.rank()
        qweight = weights.get_sharded(f"{prefix}.qweight", 0, to_dtype=False)
        g_idx = None
        K_full = weights.get_shape(f"{prefix}.qweight")[0] * (1 if self.awq else 32 // self.bits)
        groupsize = self.groupsize if self.groupsize > 0 else K_full
        if not self.awq and weights.has_tensor(f"{prefix}.g_idx"):
            g_full = weights.get_tensor(f"{prefix}.g_idx", to_dtype=False)
            per = g_full.shape[0] // world
            g_idx = g_full[rank * per : (rank + 1) * per]
        if self.groupsize > 0 and world > 1 and g_idx is None or (
            g_idx is not None and world > 1 and not self.desc_act and self.groupsize > 0
        ):
            # group-aligned shards: scales/zeros can be sliced along the group dimension
            qzeros = weights.get_sharded(f"{prefix}.qzeros", 0, to_dtype=False)
            scales = weights.get_sharded(f"{prefix}.scales", 0)
            if g_idx is not None:
                g_idx = g_idx - g_idx[0]
        else:
            qzeros = weights.get_tensor(f"{prefix}.qzeros", to_dtype=False)
            scales = weights.get_tensor(f"{prefix}.scales")
        return self._mk(weights, qweight, qzeros, scales, g_idx)


class Exl2Loader(WeightsLoader):
    """EXL2 checkpoints; tensor parallelism is not defined for this format (as in the reference)."""

    def _load(self, weights, prefix):
        if weights.process_group.size() > 1:
            raise RuntimeError("exl2 weights cannot be sharded")
        g = lambda n: weights.get_tensor(f"{prefix}.{n}", to_dtype=False)
        return Exl2Weight(g("q_weight"), g("q_scale"), g("q_invperm"), g("q_scale_max"), g("q_groups"), weights.dtype)

    def get_weights(self, weights, prefix):
        return self._load(weights, prefix)

    def get_weights_col_packed(self, weights, prefix, block_sizes):
        raise RuntimeError("column-packed weights are not supported for exl2")

    def get_weights_col(self, weights, prefix):
        return self._load(weights, prefix)

    def get_multi_weights_col(self, weights, prefixes, dim):
        raise ValueError("get_multi_weights_col is not supported for exl2")

    def get_weights_row(self, weights, prefix):
        return self._load(weights, prefix)


class CompressedTensorsLoader(WeightsLoader):
    """``compressed-tensors`` checkpoints: per-module-group schemes mapped onto the loaders above.

    Handles float8 weights (``weight_scale``/``input_scale``), int8 weights with per-channel scales
    (W8A8-int served as W8A16) and packed int4/int8 ``weight_packed``/``weight_scale``/``weight_zero_point``.
    """

    def __init__(self, config: dict):
        # 2:4-sparse checkpoints ("marlin-24") are stored in the permuted layout of one particular CUDA kernel
        # (reference: ``layers/compressed_tensors/wna16_int_24.py``); that layout is not decoded here
        if str(config.get("format", "")).lower() in ("marlin-24", "marlin_24"):
            raise NotImplementedError("compressed-tensors checkpoints in the 2:4-sparse `marlin-24` format are not "
                                      "supported; use the dense pack-quantized or fp8 variant of the model")
        self.ignore = config.get("ignore", []) or []
        self.groups = []
        for g in (config.get("config_groups") or {}).values():
            self.groups.append((g.get("targets", []), g.get("weights") or {}, g.get("input_activations")))
        self._fp8 = Fp8Loader()
        self._default = DefaultWeightsLoader()

    def _scheme(self, prefix: str):
        if any(prefix.endswith(i) or i in prefix for i in self.ignore):
            return None
        for targets, w, a in self.groups:
            if "Linear" in targets or any(t in prefix for t in targets):
                return w
        return None

    def _int_weight(self, weights, prefix, getter) -> Weight:
        if weights.has_tensor(f"{prefix}.weight_packed"):
            # pack-quantized int4: `weight_packed` int32 [N, K/8] (fields along K, offset binary), `weight_scale`
            # [N, G], optionally `weight_zero_point` int32 [N/8, G] (fields along N).  Re-expressed in the GPTQ layout
            # so that the layer is served by the weight-only GEMM (packed on the device) like any other 4-bit layer.
            packed = getter(f"{prefix}.weight_packed", False)
            scale = getter(f"{prefix}.weight_scale", True).float()
            bits = 4
            iw = _unpack_int32(packed, bits, dim=1)                                  # [N, K], 0..15
            N, K = iw.shape
            scale = scale.reshape(N, -1)
            G = scale.shape[1]
            gs = K // G
            if weights.has_tensor(f"{prefix}.weight_zero_point"):
                zp = _unpack_int32(getter(f"{prefix}.weight_zero_point", False), bits, dim=0)[:N].reshape(N, G)
            else:
                zp = torch.full((N, G), 8, dtype=iw.dtype, device=iw.device)
            if N % 8 == 0 and K % 8 == 0 and K % G == 0:
                return GPTQWeight(qweight=_pack_int32(iw.t().contiguous(), bits, dim=0),
                                  qzeros=_pack_int32((zp.t() - 1).contiguous(), bits, dim=1),
                                  scales=scale.t().contiguous().to(weights.dtype), g_idx=None, bits=bits, groupsize=gs,
                                  awq=False, sym=not weights.has_tensor(f"{prefix}.weight_zero_point"),
                                  dtype=weights.dtype)
            w = (iw.float() - zp.float().repeat_interleave(gs, dim=1)[:, :K]) * scale.repeat_interleave(gs, dim=1)[:, :K]
            return UnquantizedWeight(w.to(weights.dtype))
        q = getter(f"{prefix}.weight", False)
        scale = getter(f"{prefix}.weight_scale", True).float().reshape(-1)
        return Int8Weight(q.to(torch.int8), scale, weights.dtype)

    def _dispatch(self, method, weights, prefix_or_list, *args):
        first = prefix_or_list[0] if isinstance(prefix_or_list, list) else prefix_or_list
        sch = self._scheme(first)
        if sch is None:
            return getattr(self._default, method)(weights, prefix_or_list, *args)
        if sch.get("type") == "float":
            return getattr(self._fp8, method)(weights, prefix_or_list, *args)
        return None

    def get_weights(self, weights, prefix):
        r = self._dispatch("get_weights", weights, prefix)
        if r is not None:
            return r
        return self._int_weight(weights, prefix, lambda n, d: weights.get_tensor(n, to_dtype=d))

    def get_weights_col_packed(self, weights, prefix, block_sizes):
        r = self._dispatch("get_weights_col_packed", weights, prefix, block_sizes)
        if r is not None:
            return r
        return self._int_weight(
            weights, prefix, lambda n, d: weights.get_packed_sharded(n, 0, block_sizes, to_dtype=d))

    def get_multi_weights_col(self, weights, prefixes, dim):
        r = self._dispatch("get_multi_weights_col", weights, prefixes, dim)
        if r is not None:
            return r
        parts = [self._int_weight(weights, p, lambda n, d: weights.get_sharded(n, 0, to_dtype=d)) for p in prefixes]
        if all(isinstance(p, Int8Weight) for p in parts):
            return Int8Weight(torch.cat([p.qweight for p in parts], 0), torch.cat([p.scale for p in parts], 0),
                              weights.dtype)
        if all(isinstance(p, GPTQWeight) for p in parts) and len({(p.bits, p.groupsize) for p in parts}) == 1:
            return GPTQWeight(torch.cat([p.qweight for p in parts], 1), torch.cat([p.qzeros for p in parts], 1),
                              torch.cat([p.scales for p in parts], 1), None, parts[0].bits, parts[0].groupsize, False,
                              all(p.sym for p in parts), parts[0].dtype)
        return UnquantizedWeight(torch.cat([p.weight if isinstance(p, UnquantizedWeight) else p.dequantize()
                                            for p in parts], 0))

    def get_weights_row(self, weights, prefix):
        r = self._dispatch("get_weights_row", weights, prefix)
        if r is not None:
            return r

        def getter(n, d):
            t_shape = weights.get_shape(n)
            if len(t_shape) == 2 and t_shape[1] > 1 and not n.endswith("weight_packed"):
                return weights.get_sharded(n, 1, to_dtype=d)
            if n.endswith("weight_packed"):
                return weights.get_sharded(n, 1, to_dtype=d)
            return weights.get_tensor(n, to_dtype=d)

        return self._int_weight(weights, prefix, getter)


# ---------------------------------------------------------------------------------------------
# config discovery
# ---------------------------------------------------------------------------------------------
@dataclass
class QuantizerConfig:
    bits: int = 4
    groupsize: int = -1
    desc_act: bool = False
    quant_method: str = "gptq"
    sym: bool = False
    checkpoint_format: Optional[str] = None
    weight_block_size: Optional[List[int]] = None
    modules_to_not_convert: Optional[List[str]] = None
    raw: Optional[dict] = None


def read_quantizer_config(model_path: Union[str, os.PathLike, None], config: Optional[dict] = None) -> Optional[QuantizerConfig]:
    """Find quantisation parameters: ``config.json:quantization_config``, else ``quantize_config.json``
    (AutoGPTQ), else ``quant_config.json`` (AutoAWQ)."""
    q = (config or {}).get("quantization_config")
    if q is None and model_path is not None:
        root = Path(model_path)
        for fname, method in (("quantize_config.json", "gptq"), ("quant_config.json", "awq")):
            f = root / fname
            if f.exists():
                q = json.loads(f.read_text())
                q.setdefault("quant_method", method)
                if method == "awq":
                    q = {"bits": q.get("w_bit", 4), "group_size": q.get("q_group_size", 128),
                         "quant_method": "awq", "version": q.get("version", "gemm")}
                break
    if q is None:
        return None
    return QuantizerConfig(
        bits=int(q.get("bits", q.get("w_bit", 4)) or 4),
        groupsize=int(q.get("group_size", q.get("q_group_size", -1)) or -1),
        desc_act=bool(q.get("desc_act", False)),
        quant_method=str(q.get("quant_method", "gptq")),
        sym=bool(q.get("sym", False)),
        checkpoint_format=q.get("checkpoint_format"),
        weight_block_size=q.get("weight_block_size"),
        modules_to_not_convert=q.get("modules_to_not_convert") or q.get("ignored_layers"),
        raw=q,
    )


def get_loader(quantize: Optional[str], model_path=None, config: Optional[dict] = None) -> WeightsLoader:
    """Map ``--quantize`` (or the checkpoint's own quantisation config) to a loader."""
    qc = read_quantizer_config(model_path, config)
    if quantize is None and qc is not None:
        quantize = {"fbgemm_fp8": "fp8"}.get(qc.quant_method, qc.quant_method)
    if quantize in (None, "", "none"):
        return DefaultWeightsLoader()
    if quantize in ("gptq", "awq", "marlin"):
        if qc is None:
            raise RuntimeError(f"--quantize {quantize} needs quantisation parameters in the checkpoint")
        method = qc.quant_method if quantize == "marlin" else quantize
        return GPTQLoader(qc.bits, qc.groupsize, qc.desc_act, method, qc.sym, qc.modules_to_not_convert)
    if quantize == "fp8":
        raw = (qc.raw if qc else None) or {}
        return Fp8Loader(activation_scale_ub=raw.get("activation_scale_ub"),
                         to_fp8=qc is None or qc.quant_method not in ("fp8", "fbgemm_fp8"),
                         weight_block_size=qc.weight_block_size if qc else None)
    if quantize == "exl2":
        return Exl2Loader()
    if quantize in ("eetq", "bitsandbytes", "bitsandbytes-nf4", "bitsandbytes-fp4"):
        return OnTheFlyLoader(quantize)
    if quantize == "compressed-tensors":
        return CompressedTensorsLoader((qc.raw if qc else None) or {})
    raise ValueError(f"unknown quantization method {quantize}")
