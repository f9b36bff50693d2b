"""Quantisers and de-quantisers of the reference, restated in numpy (test oracle only).

Every array that the reference holds as ``torch.bfloat16`` is held here as a
``float32`` array whose values are exactly representable in bfloat16 (use
``bf16_round``).  All arithmetic is done in float32 in the same order as the
reference's torch code, so outputs are bit-identical (pinned by the golden
fixtures under ``tests/golden``).
"""
from __future__ import annotations

import numpy as np


def ceil_div(x: int, y: int) -> int:
    """deep_gemm/utils/math.py:5-6."""
    return (x + y - 1) // y


def align(x: int, y: int) -> int:
    """deep_gemm/utils/math.py:9-10."""
    return ceil_div(x, y) * y


def bf16_round(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest-even bfloat16, returned as float32 (what ``tensor.bfloat16().float()`` gives)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32).astype(np.uint64)
    rounded = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    out = rounded.astype(np.uint32).view(np.float32)
    return np.where(np.isnan(x), x, out).astype(np.float32)


def ceil_to_ue8m0(x: np.ndarray) -> np.ndarray:
    """Round a positive float32 up to a power of two (deep_gemm/utils/math.py:13-16)."""
    bits = np.abs(np.asarray(x, dtype=np.float32)).view(np.int32)
    exp = ((bits >> 23) & 0xFF) + ((bits & 0x7FFFFF) != 0).astype(np.int32)
    return (np.clip(exp, 1, 254) << 23).astype(np.int32).view(np.float32)


def pack_ue8m0_to_int(x: np.ndarray) -> np.ndarray:
    """Four power-of-two float32 along the last axis -> one int32, little-endian by K
    (deep_gemm/utils/math.py:19-23)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    assert x.shape[-1] % 4 == 0
    xi = x.view(np.int32)
    assert (xi >= 0).all() and ((xi & 0x7FFFFF) == 0).all()
    return np.ascontiguousarray((xi >> 23).astype(np.uint8)).view(np.int32)


def unpack_ue8m0_from_int(packed: np.ndarray) -> np.ndarray:
    """deep_gemm/utils/math.py:151-152."""
    packed = np.ascontiguousarray(packed, dtype=np.int32)
    return (packed.view(np.uint8).astype(np.int32) << 23).view(np.float32)


# ---------------------------------------------------------------------------------------------
# float8_e4m3fn: 1 sign, 4 exponent (bias 7), 3 mantissa, no infinity, 0x7F/0xFF = NaN, max 448.
# ---------------------------------------------------------------------------------------------
def _e4m3_positive_values() -> np.ndarray:
    codes = np.arange(128, dtype=np.int32)
    e, m = codes >> 3, codes & 7
    vals = np.where(e == 0, m / 8.0 * 2.0 ** -6, (1.0 + m / 8.0) * 2.0 ** (e - 7.0))
    vals = vals.astype(np.float64)
    vals[127] = 480.0  # the slot the NaN code occupies on the rounding grid
    return vals


_E4M3_POS = _e4m3_positive_values()
_E4M3_MID = (_E4M3_POS[:-1] + _E4M3_POS[1:]) / 2.0


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """float32 -> float8_e4m3fn byte, round-to-nearest-even, no saturation (what
    ``tensor.to(torch.float8_e4m3fn)`` does at deep_gemm/utils/math.py:40,59,72)."""
    x = np.asarray(x, dtype=np.float32)
    a = np.abs(x).astype(np.float64)
    idx = np.searchsorted(_E4M3_MID, a, side="left")          # number of midpoints strictly below a
    idx_c = np.minimum(idx, 126)
    tie = (idx < 127) & (a == _E4M3_MID[idx_c])
    code = np.where(tie, idx + (idx & 1), idx)                # ties go to the even code
    code = np.minimum(code, 127)
    code = np.where(np.isnan(x), 127, code).astype(np.uint8)
    sign = (np.signbit(x)).astype(np.uint8) << 7
    return (code | sign).astype(np.uint8)


def e4m3_decode(b: np.ndarray) -> np.ndarray:
    """float8_e4m3fn byte -> float32 (``tensor.float()``)."""
    b = np.asarray(b, dtype=np.uint8)
    mag = _E4M3_POS.astype(np.float32).copy()
    mag[127] = np.nan
    v = mag[(b & 0x7F).astype(np.int64)]
    return np.where((b & 0x80) != 0, -v, v).astype(np.float32)


# ---------------------------------------------------------------------------------------------
# float4_e2m1: values {0, .5, 1, 1.5, 2, 3, 4, 6}, sign in bit 3.
# ---------------------------------------------------------------------------------------------
_E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)


def e2m1_encode(x: np.ndarray) -> np.ndarray:
    """float32 -> 4-bit code in an int8, ties to even mantissa (deep_gemm/utils/math.py:84-96)."""
    x = np.asarray(x, dtype=np.float32)
    ax = np.abs(x)
    code = np.zeros(x.shape, dtype=np.uint8)
    for boundary, round_up in zip((0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0),
                                  (False, True, False, True, False, True, False)):
        b = np.float32(boundary)
        code += (ax >= b).astype(np.uint8) if round_up else (ax > b).astype(np.uint8)
    sign = (x < 0) & (code != 0)
    return (code | (sign.astype(np.uint8) << 3)).astype(np.uint8).view(np.int8)


def e2m1_decode(code: np.ndarray) -> np.ndarray:
    """4-bit code -> float32 (deep_gemm/utils/math.py:144-148)."""
    code = np.asarray(code).astype(np.int32)
    idx = code & 7
    v = _E2M1_VALUES[idx]
    return np.where(((code & 8) != 0) & (idx != 0), -v, v).astype(np.float32)


# ---------------------------------------------------------------------------------------------
# Casts
# ---------------------------------------------------------------------------------------------
def _sf_from_amax(amax: np.ndarray, qmax: float, use_ue8m0: bool) -> np.ndarray:
    sf = (amax.astype(np.float32) / np.float32(qmax)).astype(np.float32)
    return ceil_to_ue8m0(sf) if use_ue8m0 else sf


def _pad_pack_sf(sf: np.ndarray) -> np.ndarray:
    num_sf = sf.shape[-1]
    if num_sf % 4:
        sf = np.pad(sf, ((0, 0), (0, align(num_sf, 4) - num_sf)), constant_values=1.0)
    return pack_ue8m0_to_int(sf)


def per_token_cast_to_fp8(x: np.ndarray, use_ue8m0: bool, gran_k: int = 128, use_packed_ue8m0: bool = False):
    """1 x gran_k scaling along K (deep_gemm/utils/math.py:26-49).
    Returns (uint8 e4m3 bytes [m, n], float32 SF [m, ceil(n/gran_k)] or packed int32)."""
    x = np.asarray(x, dtype=np.float32)
    assert x.ndim == 2 and (not use_packed_ue8m0 or use_ue8m0)
    m, n = x.shape
    padded_n = align(n, gran_k)
    xp = np.zeros((m, padded_n), dtype=np.float32)
    xp[:, :n] = x
    xv = xp.reshape(m, padded_n // gran_k, gran_k)
    amax = np.maximum(np.abs(xv).max(axis=2), np.float32(1e-4))
    sf = _sf_from_amax(amax, 448.0, use_ue8m0)
    inv = (np.float32(1.0) / sf).astype(np.float32)
    q = e4m3_encode((xv * inv[:, :, None]).astype(np.float32)).reshape(m, padded_n)[:, :n]
    q = np.ascontiguousarray(q)
    return (q, _pad_pack_sf(sf)) if use_packed_ue8m0 else (q, sf)


def per_block_cast_to_fp8(x: np.ndarray, use_ue8m0: bool, gran_k: int = 128):
    """gran_k x gran_k block scaling (deep_gemm/utils/math.py:62-72).
    Returns (uint8 [m, n], float32 SF [ceil(m/g), ceil(n/g)])."""
    x = np.asarray(x, dtype=np.float32)
    assert x.ndim == 2
    m, n = x.shape
    pm, pn = align(m, gran_k), align(n, gran_k)
    xp = np.zeros((pm, pn), dtype=np.float32)
    xp[:m, :n] = x
    xv = xp.reshape(pm // gran_k, gran_k, pn // gran_k, gran_k)
    amax = np.maximum(np.abs(xv).max(axis=(1, 3), keepdims=True), np.float32(1e-4))
    sf = _sf_from_amax(amax, 448.0, use_ue8m0)
    inv = (np.float32(1.0) / sf).astype(np.float32)
    q = e4m3_encode((xv * inv).astype(np.float32)).reshape(pm, pn)[:m, :n]
    return np.ascontiguousarray(q), sf.reshape(pm // gran_k, pn // gran_k)


def per_token_cast_to_fp4(x: np.ndarray, use_ue8m0: bool, gran_k: int = 128, use_packed_ue8m0: bool = False):
    """1 x gran_k scaling to e2m1, two codes per byte, even K in the low nibble
    (deep_gemm/utils/math.py:99-125).  Returns (int8 [m, n/2], SF)."""
    x = np.asarray(x, dtype=np.float32)
    m, n = x.shape
    assert n % 2 == 0 and (not use_packed_ue8m0 or use_ue8m0)
    padded_n = align(n, gran_k)
    xp = np.zeros((m, padded_n), dtype=np.float32)
    xp[:, :n] = x
    xv = xp.reshape(m, -1, gran_k)
    amax = np.maximum(np.abs(xv).max(axis=2), np.float32(1e-4))
    sf = _sf_from_amax(amax, 6.0, use_ue8m0)
    inv = (np.float32(1.0) / sf).astype(np.float32)
    codes = e2m1_encode((xv * inv[:, :, None]).astype(np.float32)).reshape(m, padded_n).view(np.uint8)
    packed = ((codes[:, 0::2] & 0x0F) | ((codes[:, 1::2] & 0x0F) << 4)).astype(np.uint8).view(np.int8)
    packed = np.ascontiguousarray(packed[:, : n // 2])
    return (packed, _pad_pack_sf(sf)) if use_packed_ue8m0 else (packed, sf)


def transpose_packed_fp4(a: np.ndarray) -> np.ndarray:
    """[m, n/2] packed along n -> [n, m/2] packed along m (deep_gemm/utils/math.py:128-141)."""
    a = np.asarray(a).view(np.uint8)
    m, n2 = a.shape
    assert m % 2 == 0
    codes = np.empty((m, n2 * 2), dtype=np.uint8)
    codes[:, 0::2], codes[:, 1::2] = a & 0x0F, (a >> 4) & 0x0F
    ct = np.ascontiguousarray(codes.T)
    return ((ct[:, 0::2] & 0x0F) | ((ct[:, 1::2] & 0x0F) << 4)).astype(np.uint8).view(np.int8)


def cast_back_from_fp8(x_fp8: np.ndarray, sf: np.ndarray, gran_k: int = 128, use_packed_ue8m0: bool = False):
    """e4m3 bytes * per-row SF -> float32 (deep_gemm/utils/math.py:169-176)."""
    m, n = x_fp8.shape
    if use_packed_ue8m0:
        sf = unpack_ue8m0_from_int(sf)
    group_idx = np.arange(n) // gran_k
    return (e4m3_decode(x_fp8) * np.asarray(sf, dtype=np.float32)[:, group_idx]).astype(np.float32)


def cast_back_from_fp4(packed: np.ndarray, sf: np.ndarray, gran_k: int = 128, use_packed_ue8m0: bool = False):
    """packed e2m1 * per-row SF -> float32 (deep_gemm/utils/math.py:155-167)."""
    p = np.asarray(packed).view(np.uint8)
    m, n2 = p.shape
    n = n2 * 2
    if use_packed_ue8m0:
        sf = unpack_ue8m0_from_int(sf)
    codes = np.zeros((m, n), dtype=np.uint8)
    codes[:, 0::2], codes[:, 1::2] = p & 0x0F, (p >> 4) & 0x0F
    group_idx = np.arange(n) // gran_k
    return (e2m1_decode(codes) * np.asarray(sf, dtype=np.float32)[:, group_idx]).astype(np.float32)


_E2M1_TO_E4M3 = np.array([0x00, 0x30, 0x38, 0x3C, 0x40, 0x44, 0x48, 0x4C], dtype=np.uint8)


def fp4_to_e4m3_bytes(packed: np.ndarray) -> np.ndarray:
    """Re-encode packed e2m1 [m, k/2] as e4m3 bytes [m, k] without requantising (tests/utils.py:82-95)."""
    p = np.asarray(packed).view(np.uint8)
    lo, hi = p & 0xF, p >> 4
    out = np.empty((p.shape[0], p.shape[1] * 2), dtype=np.uint8)
    out[:, 0::2] = _E2M1_TO_E4M3[lo & 7] | ((lo & 8) << 4)
    out[:, 1::2] = _E2M1_TO_E4M3[hi & 7] | ((hi & 8) << 4)
    return out


def stochastic_round_to_bf16(x: np.ndarray) -> np.ndarray:
    """float32 [..., n] (n % 4 == 0) -> bfloat16 bits (uint16) rounded stochastically as the reference's
    BF16StochasticRounding epilogue does (tests/utils.py:53-79): the four values of columns 4q .. 4q+3 and q are hashed
    into four 16-bit random numbers that are added to the values' low 16 bits before truncation."""
    shape = x.shape
    v = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64).reshape(*shape[:-1], -1, 4)
    q = np.arange(shape[-1] // 4, dtype=np.uint64)
    m32 = np.uint64(0xFFFFFFFF)
    h = (v[..., 0] * np.uint64(0x5671d42b) + v[..., 1] * np.uint64(0x9995e499) + v[..., 2] * np.uint64(0xace1b8a5) +
         v[..., 3] * np.uint64(0xe153538d) + q) & m32
    h = ((h ^ (h >> np.uint64(23))) * np.uint64(0x7feb352d)) & m32
    h ^= h >> np.uint64(16)
    h1 = (h * np.uint64(0x846ca68b)) & m32
    h2 = (h * np.uint64(0xd35a2d97)) & m32
    h1 ^= h1 >> np.uint64(11)
    h2 ^= h2 >> np.uint64(11)
    rnd = np.stack((h1 & np.uint64(0xFFFF), h1 >> np.uint64(16), h2 & np.uint64(0xFFFF), h2 >> np.uint64(16)), axis=-1)
    out = (v >> np.uint64(16)) + (((v & np.uint64(0xFFFF)) + rnd) >> np.uint64(16))
    return out.astype(np.uint16).reshape(shape)
