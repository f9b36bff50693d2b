"""ctypes binding of the C-ABI library (include/deepgemm_b200.h).

There is no CPU or PyTorch fallback: if the shared library has not been built the import fails,
and every GEMM call needs a CUDA device.
"""
from __future__ import annotations

import ctypes as C
import os

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "lib", "libdeepgemm_b200.so")

DG_OK = 0
DG_FP8_E4M3, DG_FP4_E2M1_X2, DG_BF16, DG_FP32 = 0, 1, 2, 3
DG_MAJOR_K, DG_MAJOR_MN = 0, 1
DG_GEMM_DENSE, DG_GEMM_M_GROUPED_CONTIGUOUS, DG_GEMM_M_GROUPED_MASKED, DG_GEMM_M_GROUPED_CONTIGUOUS_PSUM = 0, 1, 2, 3
DG_GEMM_K_GROUPED_CONTIGUOUS, DG_GEMM_BATCHED = 4, 5


class GemmArgs(C.Structure):
    _fields_ = [
        ("a", C.c_void_p), ("sfa", C.c_void_p), ("b", C.c_void_p), ("sfb", C.c_void_p), ("d", C.c_void_p),
        ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32), ("num_groups", C.c_int32),
        ("a_dtype", C.c_int32), ("b_dtype", C.c_int32), ("d_dtype", C.c_int32),
        ("major_a", C.c_int32), ("major_b", C.c_int32),
        ("lda", C.c_int64), ("ldb", C.c_int64), ("ldd", C.c_int64),
        ("sfa_pitch", C.c_int64), ("sfb_pitch", C.c_int64),
        ("gran_k_a", C.c_int32), ("gran_k_b", C.c_int32),
        ("accumulate", C.c_int32), ("has_alpha", C.c_int32), ("alpha", C.c_float),
        ("grouped_layout", C.c_void_p), ("expected_m", C.c_int32), ("stream", C.c_void_p),
        ("use_psum_layout", C.c_int32), ("ensure_zero_padding", C.c_int32),
        ("sfd", C.c_void_p), ("sfd_pitch", C.c_int64),
        ("batch_stride_a", C.c_int64), ("batch_stride_b", C.c_int64), ("batch_stride_d", C.c_int64),
        ("stochastic_rounding", C.c_int32),
        ("reduce_batches", C.c_int32),
    ]


class GemmConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "block_m", "block_n", "block_k", "num_stages", "cluster_size", "raster_group", "num_ctas",
        "smem_bytes", "tmem_cols", "num_tiles", "waves_x100", "num_splits", "kb_per_split", "split_in_cluster", "swap_ab", "store_buffers", "a_rows")]

    def as_dict(self):
        return {n: getattr(self, n) for n, _ in self._fields_}


# name -> (restype, argtypes); exactly the symbols include/deepgemm_b200.h declares
SIGNATURES = {
    "dg_last_error": (C.c_char_p, []),
    "dg_init": (C.c_int, [C.c_char_p]),
    "dg_shutdown": (C.c_int, []),
    "dg_is_shut_down": (C.c_int, []),
    "dg_set_num_sms": (C.c_int, [C.c_int]),
    "dg_get_num_sms": (C.c_int, []),
    "dg_set_tc_util": (C.c_int, [C.c_int]),
    "dg_get_tc_util": (C.c_int, []),
    "dg_set_pdl": (C.c_int, [C.c_int]),
    "dg_get_pdl": (C.c_int, []),
    "dg_set_mk_alignment_for_contiguous_layout": (C.c_int, [C.c_int]),
    "dg_get_mk_alignment_for_contiguous_layout": (C.c_int, []),
    "dg_get_theoretical_mk_alignment_for_contiguous_layout": (C.c_int, [C.c_int]),
    "dg_get_tma_aligned_size": (C.c_int, [C.c_int, C.c_int]),
    "dg_pack_fp32_into_ue8m0": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                          C.c_int64, C.c_int64, C.c_int64, C.c_void_p]),
    "dg_pack_fp32_into_ue8m0_psum": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int64, C.c_int64,
                                               C.c_void_p, C.c_int, C.c_void_p]),
    "dg_pack_k_grouped_fp32_into_ue8m0": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                                    C.c_int, C.c_int, C.c_void_p]),
    "dg_transpose_fp32_mn_major": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                             C.c_int64, C.c_int64, C.c_int64, C.c_void_p]),
    "dg_per_token_cast": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int, C.c_int,
                                    C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "dg_fp8_fp4_gemm": (C.c_int, [C.POINTER(GemmArgs)]),
    "dg_fp8_fp4_gemm_noalloc": (C.c_int, [C.POINTER(GemmArgs)]),
    "dg_m_grouped_fp8_fp4_gemm_contiguous": (C.c_int, [C.POINTER(GemmArgs)]),
    "dg_m_grouped_fp8_fp4_gemm_masked": (C.c_int, [C.POINTER(GemmArgs)]),
    "dg_k_grouped_fp8_gemm_contiguous": (C.c_int, [C.POINTER(GemmArgs)]),
    "dg_fp8_bmm": (C.c_int, [C.POINTER(GemmArgs)]),
    "dg_gemm_precompile": (C.c_int, [C.c_int, C.POINTER(GemmArgs)]),
    "dg_get_gemm_config": (C.c_int, [C.c_int, C.POINTER(GemmArgs), C.POINTER(GemmConfig)]),
    "dg_enumerate_tiles": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                     C.c_int, C.c_int, C.c_void_p, C.c_int]),
    "dg_jit_compile": (C.c_int, [C.c_char_p, C.c_char_p, C.c_char_p, C.c_char_p, C.POINTER(C.c_void_p)]),
    "dg_jit_kernel_path": (C.c_char_p, [C.c_void_p]),
    "dg_jit_max_active_clusters": (C.c_int, [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(C.c_int)]),
    "dg_jit_launch": (C.c_int, [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_int, C.c_void_p,
                                C.POINTER(C.c_void_p)]),
    "dg_kernel_status": (C.c_int, []),
    "dg_reset_kernel_status": (C.c_int, []),
    "dg_selftest_bounded_wait": (C.c_int, [C.c_uint32, C.c_void_p, C.POINTER(C.c_uint64)]),
}


def _load():
    if not os.path.isfile(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python deepgemm_amd_b200/build.py` "
            "(there is no CPU or PyTorch fallback for the GEMM path)")
    lib = C.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        if not hasattr(lib, name):
            raise ImportError(f"{LIB_PATH} is older than the sources (no symbol {name}): rebuild it with "
                              "`python deepgemm_amd_b200/build.py --force`")
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


lib = _load()


def last_error() -> str:
    return (lib.dg_last_error() or b"").decode("utf-8", "replace")


def check(rc: int) -> None:
    """Every failed check surfaces as RuntimeError, as the reference's DGException does through pybind
    (csrc/utils/exception.hpp:13-41)."""
    if rc != DG_OK:
        raise RuntimeError(last_error() or f"deepgemm_b200 error {rc}")
