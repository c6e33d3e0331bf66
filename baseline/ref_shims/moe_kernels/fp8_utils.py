"""Local `moe_kernels.fp8_utils` for the reference (`layers/fp8.py:25-29`): the block-scaled fp8 Triton
GEMM and the 1x128 activation quantiser, from the installed vllm wheel (same lineage as the hub kernel)."""
from vllm.model_executor.layers.quantization.utils.fp8_utils import (  # noqa: F401
    per_token_group_quant_fp8,
    w8a8_triton_block_scaled_mm as w8a8_block_fp8_matmul,
)
