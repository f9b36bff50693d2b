// Arithmetic of the per-token (1 x 32 / 1 x 128) quantisation shared by the cast kernel and the GEMM's quantising
// epilogue, so that the two give the same bits: amax over the block, clamp to 1e-4, scale = amax / qmax rounded up to
// a power of two, value * (1 / scale), round to nearest even (deep_gemm/utils/math.py:13-49 of the reference).
#pragma once

#include <cstdint>
#include <cuda_fp8.h>

namespace dg {

// The smallest power of two that is >= x (x positive and finite), as a float; its UE8M0 code is bits >> 23
__device__ __forceinline__ float ceil_to_power_of_two(float x) {
    const uint32_t bits = __float_as_uint(x);
    uint32_t exponent = ((bits >> 23) & 0xFFu) + ((bits & 0x7FFFFFu) != 0 ? 1u : 0u);
    exponent = exponent < 1u ? 1u : (exponent > 254u ? 254u : exponent);
    return __uint_as_float(exponent << 23);
}

__device__ __forceinline__ float e4m3_block_scale(float amax) {
    return ceil_to_power_of_two(fmaxf(amax, 1e-4f) / 448.0f);          // IEEE division, as torch computes it
}

__device__ __forceinline__ uint32_t ue8m0_code(float power_of_two) { return __float_as_uint(power_of_two) >> 23; }

// Four values, already multiplied by 1 / scale, to four e4m3 bytes (first value in the low byte)
__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
    return lo | (hi << 16);
}

__device__ __forceinline__ float bf16_lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t packed) { return __uint_as_float(packed & 0xFFFF0000u); }

}  // namespace dg
