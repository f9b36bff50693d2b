"""Scaling-factor layout transforms of the reference, restated in numpy (test oracle only).

The packed layout is the public contract of docs/scaling-factor-format.md:42-63:
int32 ``[G, mn, ceil(sf_k/4)]`` with element strides
``(ceil(sf_k/4) * align(mn,4), 1, align(mn,4))`` ("MN-major, TMA-aligned").
numpy cannot hold that view and its padding in one object portably, so the
functions return ``(storage, shape, strides)`` where ``storage`` is the flat
int32 buffer (padding zero-filled), plus helpers to index it.
"""
from __future__ import annotations

import numpy as np

from .quant import align, ceil_div


def get_tma_aligned_size(x: int, element_size: int) -> int:
    """csrc/utils/math.hpp:23-27."""
    assert 16 % element_size == 0
    return align(x, 16 // element_size)


def broadcast_sf_along_mn(sf: np.ndarray, mn: int, gran_mn: int) -> np.ndarray:
    """``sf.index_select(-2, arange(mn) // gran_mn)`` (csrc/apis/layout.hpp:47-49)."""
    if gran_mn == 1:
        return sf
    return np.take(sf, np.arange(mn) // gran_mn, axis=-2)


def mn_major_tma_aligned_packed_ue8m0(sf: np.ndarray):
    """float32 power-of-two SF ``[G?, mn, sf_k]`` -> packed UE8M0 in the MN-major TMA-aligned layout.

    Follows the pure-torch model the reference's own layout test compares against
    (tests/test_layout.py:20-42; same as csrc/jit_kernels/impls/smxx_layout.hpp:108-131):
    byte = float bits >> 23, four consecutive K scales per int32 little-endian, K tail and MN
    padding zero, then transposed so MN is contiguous with pitch align(mn, 4).

    Returns ``(view, strides)``: ``view`` is a numpy array of shape ``[G?, mn, packed_k]`` whose
    *memory* is laid out exactly as the reference's tensor (numpy strides in bytes reflect it) and
    ``strides`` is the element-stride tuple torch would report.
    """
    sf = np.asarray(sf, dtype=np.float32)
    squeeze = sf.ndim == 2
    if squeeze:
        sf = sf[None]
    g, mn, k = sf.shape
    ue8m0 = (np.ascontiguousarray(sf).view(np.int32) >> 23).astype(np.uint8)
    amn, ak = get_tma_aligned_size(mn, 4), align(k, 4)
    padded = np.zeros((g, amn, ak), dtype=np.uint8)
    padded[:, :mn, :k] = ue8m0
    packed = padded.reshape(-1).view(np.int32).reshape(g, amn, ak // 4)
    storage = np.ascontiguousarray(packed.transpose(0, 2, 1))          # [g, packed_k, amn]: mn contiguous
    view = storage.transpose(0, 2, 1)[:, :mn, :]                         # [g, mn, packed_k]
    strides = ((ak // 4) * amn, 1, amn)
    if squeeze:
        return view[0], strides[1:]
    return view, strides


def mn_major_tma_aligned_fp32(sf: np.ndarray):
    """float32 SF ``[G?, mn, sf_k]`` -> same values, MN-major with pitch align(mn, 4)
    (csrc/jit_kernels/impls/smxx_layout.hpp:60-106; checked by tests/test_layout.py:61-69)."""
    sf = np.asarray(sf, dtype=np.float32)
    squeeze = sf.ndim == 2
    if squeeze:
        sf = sf[None]
    g, mn, k = sf.shape
    amn = get_tma_aligned_size(mn, 4)
    storage = np.zeros((g, k, amn), dtype=np.float32)
    storage[:, :, :mn] = sf.transpose(0, 2, 1)
    view = storage.transpose(0, 2, 1)[:, :mn, :]
    strides = (k * amn, 1, amn)
    if squeeze:
        return view[0], strides[1:]
    return view, strides


def unpack_mn_major_packed_ue8m0(packed: np.ndarray, sf_k: int) -> np.ndarray:
    """Inverse of the packing: int32 ``[..., mn, packed_k]`` -> float32 ``[..., mn, sf_k]``."""
    packed = np.ascontiguousarray(packed, dtype=np.int32)
    b = packed.view(np.uint8).reshape(*packed.shape[:-1], packed.shape[-1] * 4)[..., :sf_k]
    return (b.astype(np.int32) << 23).view(np.float32)


__all__ = [
    "get_tma_aligned_size", "broadcast_sf_along_mn", "mn_major_tma_aligned_packed_ue8m0",
    "mn_major_tma_aligned_fp32", "unpack_mn_major_packed_ue8m0", "ceil_div",
]
