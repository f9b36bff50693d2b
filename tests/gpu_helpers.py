"""Shared helpers of the GPU parity tests: seeded inputs, oracle quantisation, upload with exact strides."""
from __future__ import annotations

import numpy as np
import torch

import oracle


def seeded_bf16(shape, seed: int, scale: float = 1.0) -> np.ndarray:
    """N(0, 1) * scale rounded to bfloat16, as float32 (the reference's `torch.randn(..., dtype=bfloat16)` inputs,
    tests/generators.py:356-357, drawn here from numpy's generator so CPU and GPU boxes agree)."""
    rng = np.random.default_rng(seed)
    return oracle.bf16_round((rng.standard_normal(shape) * scale).astype(np.float32))


def upload_strided(view: np.ndarray, strides) -> torch.Tensor:
    """Upload a (possibly padded, MN-major) numpy view keeping the element strides the oracle reports."""
    span = 1 + sum((n - 1) * s for n, s in zip(view.shape, strides))
    flat = np.lib.stride_tricks.as_strided(view, (span,), (view.itemsize,)).copy()
    return torch.as_strided(torch.from_numpy(flat).cuda(), tuple(view.shape), tuple(strides))


def packed_sf_cuda(sf_rows: np.ndarray) -> torch.Tensor:
    """float32 per-row scales [G?, mn, sf_k] -> packed UE8M0 int32 on the GPU in the MN-major TMA-aligned layout."""
    view, strides = oracle.mn_major_tma_aligned_packed_ue8m0(sf_rows)
    return upload_strided(view, strides)


def fp8_cuda(q: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(q)).cuda().view(torch.float8_e4m3fn)


def fp4_cuda(q: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(q).view(np.int8)).cuda()


def quantise_dense(a: np.ndarray, b: np.ndarray, b_fp4: bool = False, gran_k_a: int = 128):
    """Oracle quantisation of tests/generators.py:371-373: A per token 1 x gran_k_a; B per 128 x 128 block
    (FP8) or per token 1 x 32 (FP4).  Returns numpy pieces with per-row FP32 scales."""
    qa, sfa = oracle.per_token_cast_to_fp8(a, True, gran_k_a)
    if b_fp4:
        qb, sfb_rows = oracle.per_token_cast_to_fp4(b, True, 32)
        sfb_raw = sfb_rows
    else:
        qb, sfb_raw = oracle.per_block_cast_to_fp8(b, True, 128)
        sfb_rows = oracle.broadcast_sf_along_mn(sfb_raw, b.shape[0], 128)
    return qa, sfa, qb, sfb_rows, sfb_raw


def diff_report(d: np.ndarray, ref: np.ndarray) -> str:
    d = d.astype(np.float64)
    ref = ref.astype(np.float64)
    err = np.abs(d - ref)
    bad = err > (1e-2 * np.abs(ref) + 1e-2 * np.abs(ref).mean() + 1e-6)
    rows = np.where(bad.any(axis=1))[0]
    cols = np.where(bad.any(axis=0))[0]
    msg = f"calc_diff={oracle.calc_diff(d, ref):.3e} max_err={err.max():.4g} ref_rms={np.sqrt((ref**2).mean()):.4g} bad={bad.mean():.4f}"
    if rows.size:
        msg += f" bad_rows[{rows.size}]={rows[:6].tolist()}..{rows[-1]} bad_cols[{cols.size}]={cols[:6].tolist()}..{cols[-1]}"
        r, c = rows[0], np.where(bad[rows[0]])[0][0]
        msg += f" first=({r},{c}) got={d[r, c]:.5g} want={ref[r, c]:.5g}"
    return msg


# Chunked, threaded forms for the benchmark's full sizes (the same bytes as one call; see oracle/parallel.py)
in_row_chunks = oracle.in_row_chunks
quantise_dense_parallel = oracle.quantise_dense_parallel
