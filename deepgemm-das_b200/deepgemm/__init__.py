"""deepgemm -- grouped MoE GEMM for NVIDIA B200 (sm_100a), drop-in for the grouped-GEMM part
of HYGON-AI/deepgemm-das (names re-exported as in the reference's deepgemm/__init__.py:25-110).

Importing the package loads libdeepgemm_b200.so (ImportError if it has not been built) and
registers the ``torch.ops.deep_gemm.*`` custom ops.  There is no CPU implementation of any
GEMM entry point.
"""
from . import _cabi  # noqa: F401  (loads the shared library; fails loudly when it is missing)
from . import op  # noqa: F401  (registers torch.ops.deep_gemm.*)
from .einsum import einsum, fp8_einsum
from .gemm import fp8_gemm, fp8_gemm_hipc
from .group_gemm_weight_pack import (
    marlin_bf16_masked_weight,
    marlin_fp8_contiguous_weight,
    marlin_fp8_masked_weight,
    marlin_i8_contiguous_weight,
    marlin_i8_masked_weight,
    pack_bf16_masked_weight,
    pack_fp8_contiguous_weight,
    pack_fp8_masked_weight,
    pack_i8_contiguous_weight,
    pack_i8_contiguous_weight_gfx936_asm_inplace,
    pack_i8_masked_weight,
    pack_i8_masked_weight_gfx936_asm_inplace,
    pack_int8_weight_enk_to_w6_gfx936_pack_permute,
    pack_int8_weight_enk_to_w6_low_latency,
    pack_int8_weight_enk_to_w6_low_latency_inplace,
    pack_w4a8_moe_hipc_weight,
    pack_w4a8_moe_hipc_weight_inplace,
    pack_w4a8_weight_k_contiguous,
    pack_w8a8_gfx936_weight_to_w6,
    unpack_weight,
    view_w4a8_moe_hipc_weight_n32_layout,
)
from .m_group_gemm import (
    m_grouped_fp8_gemm_nt_masked,
    m_grouped_fp8_gemm_nt_masked_ll,
    m_grouped_fp8_gemm_nt_masked_ll_tensor_wise,
    m_grouped_fp8_gemm_nt_masked_tensor_wise,
    m_grouped_w8a8_gemm_nt_masked_ll,
)
from .m_group_gemm_nt_contiguous import (
    get_m_grouped_fp8_contiguous_config,
    m_grouped_bf16_gemm_nt_contiguous,
    m_grouped_i8_gemm_nt_contiguous_nopad,
    m_grouped_fp8_gemm_nt_contiguous,
    m_grouped_fp8_gemm_nt_contiguous_tensor_wise,
    m_grouped_i8_gemm_nt_contiguous,
    m_grouped_w4a8_gemm_nt_contiguous_hipc,
)
from .m_group_gemm_nt_masked import (
    m_grouped_bf16_gemm_nt_masked,
    m_grouped_bf16_gemm_nt_masked_hipc,
    m_grouped_i8_gemm_nt_masked,
    m_grouped_w4a8_gemm_nt_masked,
    m_grouped_w4a8_gemm_nt_masked_hipc,
    m_grouped_w8a8_gemm_nt_compact_masked,
    m_grouped_w8a8_gemm_nt_masked,
    m_grouped_w8a8_gemm_nt_masked_gfx936,
    m_grouped_w8a8_gemm_nt_masked_gfx936_pack_permute,
    m_grouped_w8a8_gemm_nt_masked_impl,
)

from .legacy_compat import *  # noqa: F401,F403  (old names, as the reference re-exports them)
from .quant_group import quant_group_capacity, quantize_group_rows
from .moe_marlin_prefill import assert_moe_prefill_down_fp8_shapes, moe_w8a8_marlin_prefill_down_fp8
from .moe_chain import combine_rows, expert_mlp_contiguous, moe_forward, silu_mul_quant
from .print_size import install_op_size_printer
from ._core import check_device_status

install_op_size_printer(op)  # no-op unless DEEPGEMM_PRINT_OP_SIZE is set

__version__ = "0.1.0"
