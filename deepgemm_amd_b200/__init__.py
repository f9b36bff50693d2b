"""B200 (sm_100a) block-scaled FP8 / FP8xFP4 GEMMs behind the `deep_gemm` operator interface.

Importing the package loads the C-ABI library (deepgemm_amd_b200/lib/libdeepgemm_b200.so) and tells it where
its device headers and kernel cache live; no CUDA context is created until the first GPU call
(the reference pins the same property in tests/test_lazy_init.py:18-19).
"""
from . import _lib, epilogue, testing, utils  # noqa: F401
from .api import *  # noqa: F401,F403
from .api import (  # noqa: F401
    fp8_fp4_gemm_nt, fp8_fp4_gemm_nn, fp8_fp4_gemm_tn, fp8_fp4_gemm_tt,
    fp8_gemm_nt, fp8_gemm_nn, fp8_gemm_tn, fp8_gemm_tt, fp4_gemm_nt,
    m_grouped_fp8_fp4_gemm_nt_contiguous, m_grouped_fp8_fp4_gemm_nn_contiguous, m_grouped_fp8_fp4_gemm_nt_masked,
    m_grouped_fp8_gemm_nt_contiguous, m_grouped_fp8_gemm_nn_contiguous, m_grouped_fp4_gemm_nt_contiguous,
    m_grouped_fp8_gemm_nt_masked, m_grouped_fp4_gemm_nt_masked,
    k_grouped_fp8_gemm_tn_contiguous, get_k_grouped_mn_major_tma_aligned_packed_ue8m0_tensor,
    transform_k_grouped_sf_into_required_layout, fp8_einsum,
    bf16_gemm_nt, bf16_gemm_nn, bf16_gemm_tn, bf16_gemm_tt,
    m_grouped_bf16_gemm_nt_contiguous, m_grouped_bf16_gemm_nn_contiguous, m_grouped_bf16_gemm_nt_masked,
    k_grouped_bf16_gemm_tn_contiguous, einsum, k_grouped_fp4_gemm_nt_contiguous, k_grouped_fp8_gemm_nt_contiguous,
    transform_sf_into_required_layout, get_tma_aligned_size, get_mn_major_tma_aligned_tensor,
    get_mn_major_tma_aligned_packed_ue8m0_tensor,
    set_mk_alignment_for_contiguous_layout, get_mk_alignment_for_contiguous_layout,
    get_theoretical_mk_alignment_for_contiguous_layout,
    get_m_alignment_for_contiguous_layout, get_k_alignment_for_contiguous_layout,
    init, shutdown, set_num_sms, get_num_sms, set_tc_util, get_tc_util, set_pdl, get_pdl,
    use_deterministic_algorithms, set_ignore_compile_dims, set_block_size_multiple_of,
    get_gemm_config, precompile_gemm, kernel_status, reset_kernel_status, per_token_cast, selftest_bounded_wait, HAS_COMPILED_BINDING,
)

__version__ = "0.1.0"

init(_lib.PKG_DIR)
