"""Import path of the reference's layout helpers (deep_gemm/utils/layout.py re-exports the extension's functions)."""
from ..api import (  # noqa: F401
    get_tma_aligned_size, get_mn_major_tma_aligned_tensor, get_mn_major_tma_aligned_packed_ue8m0_tensor,
    get_k_grouped_mn_major_tma_aligned_packed_ue8m0_tensor, transform_sf_into_required_layout,
    get_mk_alignment_for_contiguous_layout, set_mk_alignment_for_contiguous_layout,
    get_theoretical_mk_alignment_for_contiguous_layout,
    get_m_alignment_for_contiguous_layout, get_k_alignment_for_contiguous_layout,
)
