"""Import path of the reference's quantisation helpers (deep_gemm/utils/math.py); the code lives in .quant."""
from .quant import *  # noqa: F401,F403
from .quant import (  # noqa: F401
    align, ceil_div, ceil_to_ue8m0, pack_ue8m0_to_int, unpack_ue8m0_from_int, per_token_cast_to_fp8, per_block_cast_to_fp8,
    per_channel_cast_to_fp8, per_custom_dims_cast_to_fp8, per_token_cast_to_fp4, transpose_packed_fp4, cast_back_from_fp8, cast_back_from_fp4,
)
