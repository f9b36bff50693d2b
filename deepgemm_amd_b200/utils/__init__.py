from .quant import (  # noqa: F401
    align, ceil_div, ceil_to_ue8m0, pack_ue8m0_to_int, unpack_ue8m0_from_int,
    per_token_cast_to_fp8, per_block_cast_to_fp8, per_token_cast_to_fp4,
    per_channel_cast_to_fp8, per_custom_dims_cast_to_fp8, transpose_packed_fp4,
    cast_back_from_fp8, cast_back_from_fp4,
)
from ..api import (  # noqa: F401
    get_k_grouped_mn_major_tma_aligned_packed_ue8m0_tensor,
    get_tma_aligned_size, get_mn_major_tma_aligned_tensor, get_mn_major_tma_aligned_packed_ue8m0_tensor,
    transform_sf_into_required_layout,
    get_mk_alignment_for_contiguous_layout, set_mk_alignment_for_contiguous_layout,
    get_theoretical_mk_alignment_for_contiguous_layout,
    get_m_alignment_for_contiguous_layout, get_k_alignment_for_contiguous_layout,
)
from . import math, layout  # noqa: F401,E402
