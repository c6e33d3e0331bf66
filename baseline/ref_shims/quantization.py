"""Local `quantization` kernel module for the reference (hub: kernels-community/quantization, built
from vllm's csrc/quantization): the same entry points from the installed vllm wheel."""
from vllm import _custom_ops as _ops
from vllm.scalar_type import scalar_types  # noqa: F401

scaled_fp8_quant = _ops.scaled_fp8_quant
scaled_int8_quant = _ops.scaled_int8_quant
cutlass_scaled_mm = _ops.cutlass_scaled_mm
cutlass_scaled_mm_azp = _ops.cutlass_scaled_mm_azp
cutlass_scaled_mm_supports_fp8 = _ops.cutlass_scaled_mm_supports_fp8
gptq_marlin_repack = _ops.gptq_marlin_repack
awq_marlin_repack = _ops.awq_marlin_repack


def _absent(name):
    def f(*a, **k):
        raise NotImplementedError(f"{name} is not provided by the installed vllm wheel")

    return f


marlin_gemm = _absent("marlin_gemm")
gptq_marlin_gemm = _absent("gptq_marlin_gemm")
gptq_marlin_24_gemm = _absent("gptq_marlin_24_gemm")
fp8_marlin_gemm = _absent("fp8_marlin_gemm")
