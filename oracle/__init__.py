"""CPU oracle for the block-scaled FP8 / FP8xFP4 GEMM path.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this
module; it is used by ``tests/``, by the smoke check and by the CPU-baseline
leg of the benchmark as the *checker* of the CUDA path, never as the thing
that is shipped or measured as the product.

The functions restate, in numpy, the algorithm of the reference's own Python
helpers (``deep_gemm/utils/math.py``, ``deep_gemm/testing/numeric.py``,
``tests/test_layout.py``, ``tests/generators.py``); every function cites the
reference lines it follows.  Parity is *pinned*: ``tests/golden/*.npz`` holds
outputs of the reference's Python run on seeded inputs (the generator script
sits beside them) and ``tests/test_oracle_golden.py`` compares this module
against them bit for bit.
"""
from .quant import (  # noqa: F401
    align, ceil_div, bf16_round, ceil_to_ue8m0, pack_ue8m0_to_int, unpack_ue8m0_from_int,
    e4m3_encode, e4m3_decode, e2m1_encode, e2m1_decode,
    per_token_cast_to_fp8, per_block_cast_to_fp8, per_token_cast_to_fp4,
    cast_back_from_fp8, cast_back_from_fp4, transpose_packed_fp4, fp4_to_e4m3_bytes, stochastic_round_to_bf16,
)
from .layout import (  # noqa: F401
    get_tma_aligned_size, mn_major_tma_aligned_packed_ue8m0, mn_major_tma_aligned_fp32,
    broadcast_sf_along_mn, unpack_mn_major_packed_ue8m0,
)
from .gemm import (  # noqa: F401
    calc_diff, dequant_gemm_nt, m_grouped_contiguous_ref, m_grouped_masked_ref,
    make_contiguous_layout, count_bytes, make_psum_layout, m_grouped_psum_ref,
    k_grouped_slices, k_grouped_pack_sf, k_grouped_ref,
)
from .parallel import host_threads, in_row_chunks, seeded_bf16_rows, quantise_dense_parallel  # noqa: F401
