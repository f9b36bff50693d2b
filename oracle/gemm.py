"""Dequantise-then-matmul reference of the block-scaled GEMMs, in numpy (test oracle only).

``D = (SFA . A) (SFB . B)^T`` accumulated in float32 (float64 on request), the value the
reference's torch path gives for ``cast_back_from_fp8(A) @ cast_back_from_fp8(B).T``
(deep_gemm/utils/math.py:155-176), plus the grouped walks of tests/generators.py:378-485.
"""
from __future__ import annotations

import random
from typing import Optional, Sequence

import numpy as np

from .quant import align, cast_back_from_fp4, cast_back_from_fp8, ceil_div, e4m3_decode


def calc_diff(x: np.ndarray, y: np.ndarray) -> float:
    """1 - 2<x,y>/(|x|^2+|y|^2) in float64 (deep_gemm/testing/numeric.py:5-11)."""
    x = np.asarray(x, dtype=np.float64)
    y = np.asarray(y, dtype=np.float64)
    denom = (x * x + y * y).sum()
    if denom == 0:
        return 0.0
    return float(1.0 - 2.0 * (x * y).sum() / denom)


def count_bytes(*arrays) -> int:
    """deep_gemm/testing/numeric.py:14-21."""
    total = 0
    for t in arrays:
        if isinstance(t, (tuple, list)):
            total += count_bytes(*t)
        elif t is not None:
            total += t.size * t.itemsize
    return total


def _dequant(data: np.ndarray, sf: np.ndarray, gran_k: int, is_fp4: bool) -> np.ndarray:
    """``sf`` is float32 per row ``[mn, ceil(k/gran_k)]`` (already broadcast along MN)."""
    return cast_back_from_fp4(data, sf, gran_k) if is_fp4 else cast_back_from_fp8(data, sf, gran_k)


def dequant_gemm_nt(a, sfa, b, sfb, gran_k_a: int = 128, gran_k_b: int = 128,
                    a_is_fp4: bool = False, b_is_fp4: bool = False,
                    c: Optional[np.ndarray] = None, alpha: float = 1.0,
                    acc_dtype=np.float32) -> np.ndarray:
    """D[M,N] = alpha * deq(A)[M,K] @ deq(B)[N,K]^T (+ C).  Per-row SFs."""
    da = _dequant(a, sfa, gran_k_a, a_is_fp4).astype(acc_dtype)
    db = _dequant(b, sfb, gran_k_b, b_is_fp4).astype(acc_dtype)
    d = da @ db.T
    if alpha != 1.0:
        d = d * acc_dtype(alpha)
    if c is not None:
        d = d + np.asarray(c, dtype=acc_dtype)
    return d


def make_contiguous_layout(num_groups: int, expected_m: int, alignment: int, seed: int = 0,
                           actual_ms: Optional[Sequence[int]] = None):
    """Per-expert token counts ``int(expected * U(0.7, 1.3))`` aligned up, -1 on padding rows
    (tests/generators.py:383-404).  Returns (m_total, actual_ms, aligned_ms, grouped_layout int32)."""
    if actual_ms is None:
        rng = random.Random(seed)
        actual_ms = [int(expected_m * rng.uniform(0.7, 1.3)) for _ in range(num_groups)]
    aligned_ms = [align(a, alignment) for a in actual_ms]
    m = sum(aligned_ms)
    layout = np.empty(m, dtype=np.int32)
    start = 0
    for i, (am, al) in enumerate(zip(actual_ms, aligned_ms)):
        layout[start:start + am] = i
        layout[start + am:start + al] = -1
        start += al
    return m, list(actual_ms), aligned_ms, layout


def m_grouped_contiguous_ref(a, sfa, b, sfb, aligned_ms: Sequence[int], gran_k_a: int = 128, gran_k_b: int = 128,
                             b_is_fp4: bool = False, groups: Optional[Sequence[int]] = None) -> np.ndarray:
    """Rows of segment i times expert i's weight (tests/generators.py:396-408).
    ``b``/``sfb`` are ``[G, N, ...]`` with per-row SFs.  ``groups`` restricts the experts computed;
    rows of skipped experts are NaN."""
    n = b.shape[1]
    d = np.full((a.shape[0], n), np.nan, dtype=np.float32)
    start = 0
    for i, al in enumerate(aligned_ms):
        if groups is None or i in groups:
            d[start:start + al] = dequant_gemm_nt(a[start:start + al], sfa[start:start + al], b[i], sfb[i],
                                                  gran_k_a, gran_k_b, False, b_is_fp4)
        start += al
    return d


def make_psum_layout(actual_ms: Sequence[int], alignment: int):
    """Prefix-sum form of the contiguous layout (tests/generators.py:388-404, docs/scaling-factor-format.md 7.3):
    group i occupies rows [align(ends[i-1], alignment), ends[i]).  Returns (m_total, starts, ends int32)."""
    starts, ends, start = [], [], 0
    for am in actual_ms:
        starts.append(start)
        ends.append(start + am)
        start = align(start + am, alignment)
    return start, starts, np.asarray(ends, dtype=np.int32)


def m_grouped_psum_ref(a, sfa, b, sfb, ends: Sequence[int], alignment: int, gran_k_a: int = 128, gran_k_b: int = 128,
                       b_is_fp4: bool = False) -> np.ndarray:
    """Rows [start_i, ends[i]) times expert i's weight; every other row is NaN (scheduler/gemm.cuh:205-225 of the
    reference walks the same ranges)."""
    d = np.full((a.shape[0], b.shape[1]), np.nan, dtype=np.float32)
    start = 0
    for i, end in enumerate(ends):
        end = int(end)
        if end > start:
            d[start:end] = dequant_gemm_nt(a[start:end], sfa[start:end], b[i], sfb[i], gran_k_a, gran_k_b, False, b_is_fp4)
        start = align(max(end, start), alignment)
    return d


def k_grouped_slices(ks: Sequence[int], alignment: int, psum: bool):
    """(start, length, padded length) of every group's slice of K and the grouped_layout the GEMM takes
    (tests/generators.py:551-572, docs/scaling-factor-format.md 5.1): slices start on multiples of the alignment;
    the layout holds the padded lengths, or with ``psum`` the elements where the slices end."""
    slices, start = [], 0
    for k in ks:
        padded = align(k, alignment)
        slices.append((start, int(k), padded))
        start += padded
    layout = [s0 + k for s0, k, _ in slices] if psum else [p for _, _, p in slices]
    return slices, np.asarray(layout, dtype=np.int32), start


def k_grouped_pack_sf(sf_rows: np.ndarray, slices, gran_k: int) -> np.ndarray:
    """FP32 power-of-two scales [sum of padded_k / gran_k, mn] -> packed UE8M0 [sum ceil(rows_g / 4), mn] uint32, every
    group starting a new packed row, unused slots zero (docs/scaling-factor-format.md 5.2, 7.4)."""
    out, row = [], 0
    for _, _, padded in slices:
        rows = padded // gran_k
        block = np.zeros((ceil_div(rows, 4) * 4, sf_rows.shape[1]), dtype=np.uint32)
        block[:rows] = sf_rows[row:row + rows].view(np.uint32) >> 23
        block = block.reshape(-1, 4, sf_rows.shape[1])
        out.append(block[:, 0] | (block[:, 1] << 8) | (block[:, 2] << 16) | (block[:, 3] << 24))
        row += rows
    return np.concatenate(out, axis=0) if out else np.zeros((0, sf_rows.shape[1]), dtype=np.uint32)


def k_grouped_ref(a_q, sfa, b_q, sfb, slices, gran_k: int = 128) -> np.ndarray:
    """D[g] = (dequantised A[slice g])^T (dequantised B[slice g]) in float32 (tests/generators.py:583-587).
    a_q [sum_k, m] e4m3 bytes with scales sfa [sum_k / gran_k, m] (one per gran_k elements of K and column)."""
    a = e4m3_decode(a_q) * np.repeat(sfa, gran_k, axis=0)[:a_q.shape[0]]
    b = e4m3_decode(b_q) * np.repeat(sfb, gran_k, axis=0)[:b_q.shape[0]]
    d = np.zeros((len(slices), a_q.shape[1], b_q.shape[1]), dtype=np.float32)
    for g, (s0, k, _) in enumerate(slices):
        if k:
            d[g] = a[s0:s0 + k].T.astype(np.float32) @ b[s0:s0 + k].astype(np.float32)
    return d


def m_grouped_masked_ref(a, sfa, b, sfb, masked_m: Sequence[int], gran_k_a: int = 128, gran_k_b: int = 128,
                         b_is_fp4: bool = False) -> np.ndarray:
    """einsum('gmk,gnk->gmn') on the first masked_m[g] rows (tests/generators.py:453,464).
    Rows at or beyond masked_m[g] are NaN (the contract leaves them untouched)."""
    g, max_m = a.shape[0], a.shape[1]
    n = b.shape[1]
    d = np.full((g, max_m, n), np.nan, dtype=np.float32)
    for i in range(g):
        mm = int(masked_m[i])
        if mm:
            d[i, :mm] = dequant_gemm_nt(a[i, :mm], sfa[i, :mm], b[i], sfb[i], gran_k_a, gran_k_b, False, b_is_fp4)
    return d
