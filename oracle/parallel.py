"""Row-chunked, threaded application of the oracle's quantisers and generators (test oracle only).

The quantisers in `quant.py` treat row blocks independently (rows for the per-token casts, bands of 128 rows for the
128 x 128 block cast), so applying them to chunks of rows and stacking the pieces gives the same bytes as one call over
the whole array.  numpy releases the GIL inside its loops, so a thread pool over chunks uses all host cores and keeps
every temporary inside the caches: at the benchmark's full sizes (10^8 elements) this is ~15x faster than one call.
"""
from __future__ import annotations

import os
from concurrent.futures import ThreadPoolExecutor

import numpy as np

from .quant import bf16_round, per_block_cast_to_fp8, per_token_cast_to_fp4, per_token_cast_to_fp8
from .layout import broadcast_sf_along_mn


def host_threads() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return os.cpu_count() or 1


def in_row_chunks(fn, x: np.ndarray, rows_per_chunk: int = 512, threads: int | None = None):
    """`fn(chunk) -> (data, scales)` over chunks of `rows_per_chunk` rows of `x`, pieces stacked along the rows.
    `rows_per_chunk` must be a multiple of the quantiser's row granularity (128 for the block cast)."""
    starts = range(0, x.shape[0], rows_per_chunk)
    with ThreadPoolExecutor(max_workers=threads or host_threads()) as pool:
        pieces = list(pool.map(lambda s: fn(x[s:s + rows_per_chunk]), starts))
    return np.concatenate([p[0] for p in pieces]), np.concatenate([p[1] for p in pieces])


def seeded_bf16_rows(shape, seed: int, rows_per_chunk: int = 512, threads: int | None = None) -> np.ndarray:
    """N(0, 1) rounded to bfloat16 (as float32), every chunk of rows drawn from its own generator seeded with
    (seed, chunk index): reproducible whatever the thread count."""
    rows, cols = shape
    out = np.empty(shape, dtype=np.float32)

    def fill(i):
        s = i * rows_per_chunk
        rng = np.random.default_rng([seed, i])
        out[s:s + rows_per_chunk] = bf16_round(rng.standard_normal((min(rows_per_chunk, rows - s), cols), dtype=np.float32))

    with ThreadPoolExecutor(max_workers=threads or host_threads()) as pool:
        list(pool.map(fill, range(-(-rows // rows_per_chunk))))
    return out


def quantise_dense_parallel(a: np.ndarray, b: np.ndarray, b_fp4: bool = False):
    """A per token 1 x 128 (e4m3), B per 128 x 128 block (e4m3) or per token 1 x 32 (e2m1), as the reference's generator
    prepares a dense case (tests/generators.py:371-373); scales come back per row, FP32."""
    qa, sfa = in_row_chunks(lambda x: per_token_cast_to_fp8(x, True, 128), a)
    if b_fp4:
        qb, sfb_rows = in_row_chunks(lambda x: per_token_cast_to_fp4(x, True, 32), b)
    else:
        qb, sfb_raw = in_row_chunks(lambda x: per_block_cast_to_fp8(x, True, 128), b, 512)
        sfb_rows = broadcast_sf_along_mn(sfb_raw, b.shape[0], 128)
    return qa, sfa, qb, sfb_rows
