"""Linear / embedding / head building blocks with tensor parallelism.

Counterparts in the reference: ``layers/linear.py:21-44`` (``FastLinear``),
``layers/fp8.py:428-579`` (``Fp8Linear``), ``layers/tensor_parallel.py:39-249``
(column / row linear, vocab-parallel embedding and head), ``layers/speculative.py``.

These are plain callables, not ``nn.Module``s: the forward pass is a flat list of
kernel launches that gets captured into a CUDA graph, and nothing here needs
autograd, hooks or state dicts.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .. import ops
from ..ops import reference as ref
from ..parallel import dist as pdist

FP8 = torch.float8_e4m3fn


class FastLinear:
    """``y = x @ W^T + b`` with ``W[N,K]`` in the serving dtype."""

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        self.weight = weight
        self.bias = bias

    @property
    def out_features(self):
        return self.weight.shape[0]

    def __call__(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        return ops.linear(x, self.weight, self.bias, out=out)


class PackedQuantLinear:
    """Weight-only quantised linear whose weights stay packed on the device: 4-bit (GPTQ / AWQ / symmetric, after the
    one-time repack of ``utils.quantization.pack_gptq_for_kernel``) or int8 with one scale per output channel.

    Steps of up to ``fused_max_tokens`` rows run the fused kernel that dequantises the weight tile on its way into
    shared memory (``ops/csrc/gemm_wq_sm100.cu``): a decode step streams a quarter (half) of the bf16 bytes.
    Larger steps are compute bound: the matrix is dequantised into a scratch buffer shared by all layers and the
    bf16 GEMM runs on it.  Reference: ``layers/marlin/gptq.py:371-440``, ``layers/gptq/exllamav2.py``,
    ``layers/awq/quantize/cuda.py:19-49``, ``layers/eetq.py:27-47``."""

    fused_max_tokens = int(__import__("os").environ.get("TGI_B200_WQ_FUSED_TOKENS", "512"))

    def __init__(self, wq, scale, zp, group: int, bits: int, perm, in_features: int, bias=None, dtype=torch.bfloat16):
        self.wq, self.scale, self.zp, self.group, self.bits = wq, scale, zp, int(group), int(bits)
        self.perm, self.in_features, self.bias, self.dtype = perm, int(in_features), bias, dtype

    @property
    def out_features(self):
        return self.wq.shape[0]

    @property
    def weight(self) -> torch.Tensor:
        """Dequantised ``[N, K]`` matrix in the original column order (merges, LoRA base lookups, tests)."""
        w = self.dequantize()
        if self.perm is not None:
            inv = torch.empty_like(self.perm)
            inv[self.perm] = torch.arange(self.perm.numel(), device=self.perm.device)
            w = w[:, inv]
        return w

    def dequantize(self) -> torch.Tensor:
        """bf16 ``[N, K]`` in the kernel's column order: bf16((q - zp) * scale), the GEMM's operand."""
        if self.wq.is_cuda and ops.use_native(self.wq):
            return ops.native().wq_dequant(self.wq, self.scale, self.zp, self.group, self.bits, self.in_features)
        K, N = self.in_features, self.wq.shape[0]
        if self.bits == 4:
            q = torch.stack([self.wq & 0xF, self.wq >> 4], dim=2).reshape(N, K).float()
            z = self.zp.float() if self.zp is not None else torch.full_like(self.scale.float(), 8.0)
        else:
            q = self.wq.float()
            z = torch.zeros_like(self.scale.float())
        gi = torch.arange(K, device=self.wq.device) // self.group
        return ((q - z.t()[:, gi]) * self.scale.float().t()[:, gi]).to(torch.bfloat16)

    def __call__(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        if self.perm is not None:
            x2 = x2.index_select(1, self.perm)
        if x2.is_cuda and ops.use_native(x2) and x2.dtype == torch.bfloat16:
            if x2.shape[0] <= self.fused_max_tokens:
                y = ops.native().gemm_wq(x2, self.wq, self.scale, self.zp, self.group, self.bits, self.bias)
            else:
                w = ops.native().wq_dequant_scratch(self.wq, self.scale, self.zp, self.group, self.bits, self.in_features)
                y = ops.linear(x2, w, self.bias)
        else:
            y = torch.nn.functional.linear(x2.float(), self.dequantize().float(),
                                           None if self.bias is None else self.bias.float()).to(x.dtype)
        y = y.view(*shape[:-1], y.shape[-1])
        if out is not None:
            out.copy_(y)
            return out
        return y


class Fp8Linear:
    """e4m3 weight with per-tensor, per-channel or 128x128-block scales.

    Block-scaled weights use dynamically 1x128-quantised activations and the block-scaled GEMM; an
    already quantised activation can be passed as ``(xq, xs)`` so the producer kernel (RMSNorm or
    SwiGLU) fuses the quantisation.  Per-tensor/per-channel weights are served by re-expressing the
    scales per block when the shape allows it, otherwise by dequantising once at load.
    """

    def __init__(self, qweight, scale, bias, dtype, input_scale=None, scale_upper_bound=None,
                 weight_block_size: Optional[Sequence[int]] = None):
        self.dtype = dtype
        self.bias = bias
        self.input_scale = input_scale
        self.scale_upper_bound = scale_upper_bound
        N, K = qweight.shape
        self.block = None
        self.dense = None
        if weight_block_size is not None:
            assert list(weight_block_size) == [128, 128], "only 128x128 weight blocks are supported"
            self.qweight, self.scale, self.block = qweight, scale.float().contiguous(), 128
        elif K % 128 == 0:
            # Express per-tensor / per-channel scales on the block grid: a per-channel scale cannot
            # be represented per block, so it is applied in the GEMM epilogue instead.
            nb, kb = (N + 127) // 128, K // 128
            if scale.numel() == 1:
                self.qweight, self.block = qweight, 128
                self.scale = scale.float().reshape(1, 1).expand(nb, kb).contiguous()
            else:
                self.qweight, self.block = qweight, 128
                self.scale = torch.ones(nb, kb, dtype=torch.float32, device=qweight.device)
                self.channel_scale = scale.float().reshape(-1).contiguous()
        else:
            s = scale.float().reshape(-1, 1) if scale.numel() > 1 else scale.float()
            self.dense = FastLinear((qweight.float() * s).to(dtype), bias)
        if not hasattr(self, "channel_scale"):
            self.channel_scale = None
        if self.block is not None and qweight.is_cuda:
            from ..ops import cuda as K

            if K.fp8_mx():       # the scale-factor MMA takes power-of-two scales: requantise once
                self.qweight, self.scale = K.requant_block_pow2(self.qweight, self.scale, self.block)

    @property
    def out_features(self):
        return self.dense.out_features if self.dense is not None else self.qweight.shape[0]

    @property
    def wants_quantized_input(self) -> bool:
        return self.dense is None

    def __call__(self, x, x_scale: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.dense is not None:
            return self.dense(x, out=out)
        if x_scale is None:
            x, x_scale = ops.fp8_quant_act(x)
        if self.channel_scale is None:
            return ops.gemm_fp8_block(x, x_scale, self.qweight, self.scale, self.dtype, self.bias, out=out)
        y = ops.gemm_fp8_block(x, x_scale, self.qweight, self.scale, self.dtype, None)
        # one elementwise kernel: the product is formed in fp32 (type promotion) and stored in the output dtype,
        # in place or straight into the caller's buffer
        dst = y if out is None else (out.fallback if getattr(out, "is_peer_push", False) else out)
        torch.mul(y, self.channel_scale, out=dst)
        if self.bias is not None:
            dst.add_(self.bias)
        return dst if out is None else out


def get_linear(weight, bias):
    """Checkpoint weight object (or raw tensor) -> callable linear."""
    if isinstance(weight, torch.Tensor):
        return FastLinear(weight, bias)
    return weight.get_linear(bias)


class TensorParallelColumnLinear:
    """Output features sharded across ranks; no communication."""

    def __init__(self, linear):
        self.linear = linear

    @classmethod
    def load(cls, config, prefix: str, weights, bias: bool):
        w = weights.get_weights_col(prefix)
        b = weights.get_sharded(f"{prefix}.bias", dim=0) if bias else None
        return cls(get_linear(w, b))

    @classmethod
    def load_multi(cls, config, prefixes: List[str], weights, bias: bool, dim: int = 0):
        w = weights.get_multi_weights_col(prefixes, dim)
        b = torch.cat([weights.get_sharded(f"{p}.bias", dim=0) for p in prefixes], dim=dim) if bias else None
        return cls(get_linear(w, b))

    @classmethod
    def load_qkv(cls, config, prefix: str, weights, bias: bool, num_heads: int, num_key_value_heads: int):
        """A checkpoint that stores q, k, v fused in one matrix (Phi-3, GPT-2 style ``c_attn`` ...)."""
        w = weights.get_weights_col_packed_qkv(prefix, num_heads, num_key_value_heads)
        b = (weights.get_packed_sharded(f"{prefix}.bias", 0, [num_heads, num_key_value_heads, num_key_value_heads])
             if bias else None)
        return cls(get_linear(w, b))

    @classmethod
    def load_gate_up(cls, config, prefix: str, weights, bias: bool):
        w = weights.get_weights_col_packed_gate_up(prefix)
        b = weights.get_packed_sharded(f"{prefix}.bias", 0, 2) if bias else None
        return cls(get_linear(w, b))

    def __call__(self, x, x_scale=None):
        if x_scale is not None:
            return self.linear(x, x_scale)
        return self.linear(x)


class TensorParallelRowLinear:
    """Input features sharded; partial sums are reduced across ranks (bias lives on rank 0 only)."""

    def __init__(self, linear, process_group, comm=None):
        self.linear = linear
        self.process_group = process_group
        self.comm = comm

    @classmethod
    def load(cls, config, prefix: str, weights, bias: bool, comm=None):
        w = weights.get_weights_row(prefix)
        b = weights.get_tensor(f"{prefix}.bias") if bias and weights.process_group.rank() == 0 else None
        return cls(get_linear(w, b), weights.process_group, comm)

    def __call__(self, x, x_scale=None, reduce: bool = True, out: Optional[torch.Tensor] = None):
        """``out`` receives the (partial) product when given, e.g. a peer-memory buffer that the
        fused reduction reads; it implies ``reduce=False`` semantics for the caller to finish."""
        if out is not None:
            return self.linear(x, x_scale, out=out) if x_scale is not None else self.linear(x, out=out)
        out = self.linear(x, x_scale) if x_scale is not None else self.linear(x)
        if reduce and self.process_group.size() > 1:
            if self.comm is not None:
                return self.comm.all_reduce(out)
            pdist.all_reduce(out, self.process_group)
        return out


class TensorParallelEmbedding:
    """Vocab-parallel embedding: each rank owns a ceil-div block of rows; foreign ids hit a zero row."""

    def __init__(self, prefix: str, weights, reduce: bool = True, comm=None):
        w = weights.get_partial_sharded(f"{prefix}.weight", dim=0)
        pg = weights.process_group
        num = weights.get_shape(f"{prefix}.weight")[0]
        block = (num + pg.size() - 1) // pg.size()
        self.min_id = pg.rank() * block
        self.max_id = min(num, (pg.rank() + 1) * block)
        self.null_idx = w.shape[0]
        self.process_group = pg
        self.reduce = reduce
        self.comm = comm
        self.weight = torch.cat([w, w.new_zeros(1, w.shape[1])], dim=0) if pg.size() > 1 else w

    def local_rows(self, ids: torch.Tensor) -> torch.Tensor:
        """This rank's contribution to the embedding: the row for ids it owns, zeros for the others."""
        if self.process_group.size() == 1:
            return ops.embedding(ids, self.weight)
        local = torch.where((ids < self.min_id) | (ids >= self.max_id), self.null_idx, ids - self.min_id)
        return ops.embedding(local.to(ids.dtype), self.weight)

    def __call__(self, ids: torch.Tensor) -> torch.Tensor:
        if self.process_group.size() == 1:
            return ops.embedding(ids, self.weight)
        out = self.local_rows(ids)
        if self.reduce:
            if self.comm is not None:
                return self.comm.all_reduce(out)
            pdist.all_reduce(out, self.process_group)
        return out


class TensorParallelHead:
    """Vocab-parallel lm_head.

    ``__call__`` returns full logits ``[B, V]`` (all-gather of the shards; used when the sampler needs
    the whole distribution).  ``local_logits`` returns the rank's ``[B, V/tp]`` slice together with the
    first vocabulary id it covers, for the distributed sampling path that never gathers logits.
    """

    def __init__(self, linear, process_group, should_gather: bool, vocab_start: int = 0):
        self.linear = linear
        self.process_group = process_group
        self.should_gather = should_gather
        self.vocab_start = vocab_start

    @classmethod
    def load(cls, config, prefix: str, weights):
        pg = weights.process_group
        total = weights.get_shape(f"{prefix}.weight")[0]
        has_bias = weights.has_tensor(f"{prefix}.bias")      # GPT-J, Phi: the head carries a bias
        if total % pg.size() == 0 and pg.size() > 1:
            w = weights.get_sharded(f"{prefix}.weight", dim=0)
            b = weights.get_sharded(f"{prefix}.bias", dim=0) if has_bias else None
            return cls(FastLinear(w, b), pg, True, pg.rank() * (total // pg.size()))
        # Vocabulary not divisible: every rank keeps the full head (as the reference does).
        b = weights.get_tensor(f"{prefix}.bias") if has_bias else None
        return cls(FastLinear(weights.get_tensor(f"{prefix}.weight"), b), pg, False, 0)

    def local_logits(self, x: torch.Tensor):
        return self.linear(x), self.vocab_start

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        local = self.linear(x)
        if not self.should_gather:
            return local
        return self.gather(local)

    def gather(self, local: torch.Tensor) -> torch.Tensor:
        world = self.process_group.size()
        B, Vl = local.shape
        # concatenated along dim 0 (the one layout every backend accepts), then viewed per rank
        gathered = local.new_empty(world * B, Vl)
        pdist.all_gather_into(gathered, local.contiguous(), self.process_group)
        return gathered.view(world, B, Vl).permute(1, 0, 2).reshape(B, world * Vl)
