"""helion_b200 -- hand-written sm_100a (B200) kernels behind the call signatures of the
quantized-inference operators that pytorch/helion ships: NVFP4 GEMV / GEMM / grouped MoE GEMM
and the fused FP8 activation-quant producers.

``helion_b200.ops`` holds the drop-in entry points (also registered as ``torch.ops.helion_b200.*``),
``helion_b200.layouts`` the host-side format helpers, ``helion_b200.build`` compiles the C-ABI
library ``libhelion_b200.so`` declared in ``include/helion_b200.h``.
"""

from . import layouts
from .grouped import grouped_gemm
from .grouped import grouped_gemm_deepgemm
from .grouped import grouped_gemm_direct
from .grouped import grouped_gemm_split_sizes
from .grouped import grouped_gemm_jagged
from .grouped import grouped_gemm_jagged_persistent
from .grouped import moe_matmul_ogs
from .grouped import moe_matmul_ogs_helion_kernel_args_gen
from .layouts import swizzle_fp8_scales
from .layouts import swizzled_scale_numel
from .layouts import swizzled_scale_offsets
from .layouts import unswizzle_fp8_scales
from .ops import HostPipelinedMatmul
from .ops import nvfp4_gemv_bf16in
from .ops import nvfp4_gemv_bf16in_batched
from .ops import nvfp4_gemv_fp4in
from .ops import nvfp4_quantize
from .ops import nvfp4_scaled_matmul
from .ops import nvfp4_w4a4_matmul
from .ops import nvfp4_w4a16_matmul
from .ops import per_token_group_fp8_quant
from .ops import dynamic_per_token_scaled_fp8_quant
from .ops import scaled_mm
from .ops import silu_mul_fp8
from .ops import rms_norm_dynamic_per_token_quant
from .ops import rms_norm_nvfp4_quant
from .ops import silu_and_mul_nvfp4_quant
from .ops import rms_norm_per_block_quant
from .ops import silu_and_mul_per_block_quant

__all__ = [
    "grouped_gemm",
    "grouped_gemm_deepgemm",
    "grouped_gemm_direct",
    "grouped_gemm_split_sizes",
    "grouped_gemm_jagged",
    "grouped_gemm_jagged_persistent",
    "moe_matmul_ogs",
    "moe_matmul_ogs_helion_kernel_args_gen",
    "layouts",
    "nvfp4_gemv_bf16in",
    "nvfp4_gemv_bf16in_batched",
    "nvfp4_gemv_fp4in",
    "nvfp4_quantize",
    "nvfp4_scaled_matmul",
    "nvfp4_w4a4_matmul",
    "nvfp4_w4a16_matmul",
    "per_token_group_fp8_quant",
    "dynamic_per_token_scaled_fp8_quant",
    "scaled_mm",
    "silu_mul_fp8",
    "rms_norm_dynamic_per_token_quant",
    "rms_norm_nvfp4_quant",
    "silu_and_mul_nvfp4_quant",
    "rms_norm_per_block_quant",
    "silu_and_mul_per_block_quant",
    "swizzle_fp8_scales",
    "swizzled_scale_numel",
    "swizzled_scale_offsets",
    "unswizzle_fp8_scales",
]
