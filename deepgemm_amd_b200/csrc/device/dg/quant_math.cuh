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

// Stochastic rounding of FP32 to BF16 as the reference's BF16StochasticRounding epilogue defines it
// (tests/utils.py:53-79 of the reference states the arithmetic): the four values of columns 4q .. 4q+3 of a row are
// hashed together with q into four 16-bit random numbers; each value's low 16 bits plus its random number carry into
// the high 16 bits, which are the result.  Deterministic in the accumulator bits and the column, so reruns agree.
__device__ __forceinline__ void stochastic_round_quartet(uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t quartet,
                                                         uint32_t& packed_ab, uint32_t& packed_cd) {
    uint32_t h = a * 0x5671d42bu + b * 0x9995e499u + c * 0xace1b8a5u + d * 0xe153538du + quartet;
    h = (h ^ (h >> 23)) * 0x7feb352du;
    h ^= h >> 16;
    uint32_t h1 = h * 0x846ca68bu, h2 = h * 0xd35a2d97u;
    h1 ^= h1 >> 11;
    h2 ^= h2 >> 11;
    auto round = [](uint32_t v, uint32_t random16) { return ((v >> 16) + (((v & 0xFFFFu) + random16) >> 16)) & 0xFFFFu; };
    packed_ab = round(a, h1 & 0xFFFFu) | (round(b, h1 >> 16) << 16);
    packed_cd = round(c, h2 & 0xFFFFu) | (round(d, h2 >> 16) << 16);
}

}  // namespace dg
