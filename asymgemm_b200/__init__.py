"""asymgemm_b200: B200 (sm_100a) implementation of AsymGEMM's m-grouped asymmetric MoE GEMM.

Exports the operator names of the reference package (asym_gemm/__init__.py:37-96) for this path.
Importing the package does not touch the GPU; the first operator call loads ``libasymgemm_b200.so`` and
raises if it has not been built.
"""
from .api import (  # noqa: F401
    check_status,
    get_mk_alignment_for_contiguous_layout,
    get_num_sms,
    launch_sm_cap,
    m_grouped_bf16_asym_gemm_nt_contiguous,
    m_grouped_bf16_asym_gemm_nt_masked,
    m_grouped_fp4_asym_gemm_nt_contiguous,
    m_grouped_fp4_asym_gemm_nt_masked,
    m_grouped_fp8_asym_gemm_nt_contiguous,
    m_grouped_fp8_asym_gemm_nt_masked,
    m_grouped_int8_asym_gemm_nt_contiguous,
    m_grouped_int8_asym_gemm_nt_masked,
    set_fp8_scale_mode,
    set_num_sms,
    set_split_segments,
    set_tile_config,
    prefetch_weights,
    prepare_weights,
    release_weights,
    set_use_scratch,
    set_weight_path,
    get_weight_path,
    set_wait_limit_ms,
)
from .layout_api import (  # noqa: F401
    get_arch_major,
    get_arch_pair,
    get_compile_mode,
    get_mn_major_tma_aligned_packed_ue8m0_tensor,
    get_mn_major_tma_aligned_tensor,
    get_tc_util,
    get_tma_aligned_size,
    set_compile_mode,
    set_tc_util,
    transform_sf_into_required_layout,
)
from . import ep, expert_cache, int8_moe, moe_ops, testing, utils  # noqa: F401

__version__ = "0.1.0"


def init(*_args, **_kwargs) -> None:
    """Kept for drop-in compatibility: the reference initialises its JIT here (csrc/apis/runtime.hpp:44-47)."""
    return None
