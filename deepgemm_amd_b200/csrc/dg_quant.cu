// Per-token (1 x gran_k) quantisation of BF16 activations to float8_e4m3 or packed float4_e2m1, writing the scales
// either as FP32 [m, k / gran_k] or directly in the layout the GEMMs consume (UE8M0, four exponents per int32,
// MN-major, pitch align(m, 4)), so that no scale-transform kernel runs between the cast and the GEMM
// (docs/scaling-factor-format.md:123-139 of the reference describes producing pre-transformed scales in the cast).
// Arithmetic follows deep_gemm/utils/math.py:26-49,99-125 exactly: amax over the block, clamp to 1e-4,
// scale = amax / 448 (or / 6), rounded up to a power of two, x * (1 / scale), round to nearest even.
//
// HBM-bound streaming kernel: 2 bytes read and 1 (0.5) byte written per element plus 1/gran_k byte of scale.
// One CTA handles 16 rows x 512 columns: 16-byte loads (8 BF16 per thread), block maxima by warp shuffles over the
// lanes that share a block, 8-byte (4-byte) stores, and the 16 packed scale words of a 512-column span leave the CTA
// as one coalesced 64-byte row of the MN-major scale tensor.
#include "dg_common.hpp"

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "device/dg/quant_math.cuh"

namespace dg {
namespace {

constexpr int kRowsPerCta = 16;
constexpr int kColsPerCta = 512;

// e2m1 code of a value already divided by its scale: round to nearest, ties to the even mantissa, no negative zero
__device__ __forceinline__ uint32_t e2m1_code(float x) {
    const float a = fabsf(x);
    uint32_t code = (a > 0.25f) + (a >= 0.75f) + (a > 1.25f) + (a >= 1.75f) + (a > 2.5f) + (a >= 3.5f) + (a > 5.0f);
    if (x < 0.0f && code != 0) code |= 8u;
    return code;
}

// kGranK: 32 or 128 elements per scale.  kFP4: packed e2m1 output (two codes per byte).  kPacked: UE8M0 int32 scales.
template <int kGranK, bool kFP4, bool kPacked, bool kUE8M0>
__global__ void __launch_bounds__(256)
per_token_cast_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, uint8_t* __restrict__ q, int64_t ldq,
                      void* __restrict__ sf_out, int64_t sf_pitch, int m, int k) {
    constexpr int kLanesPerBlock = kGranK / 8;                 // threads sharing one scale (8 elements each)
    constexpr float kQMax = kFP4 ? 6.0f : 448.0f;
    __shared__ uint32_t packed_words[kColsPerCta / 128][kRowsPerCta];   // [int32 column within the CTA][row]

    const int row_in_cta = threadIdx.x / 16, lane16 = threadIdx.x % 16;
    const int row = blockIdx.y * kRowsPerCta + row_in_cta;
    const int col0 = blockIdx.x * kColsPerCta;

    uint32_t my_bytes = 0;                                     // this thread's scale exponents, one byte per 128-column step
    #pragma unroll
    for (int step = 0; step < kColsPerCta / 128; ++step) {
        const int col = col0 + step * 128 + lane16 * 8;
        const bool in_range = row < m && col < k;
        float v[8];
        if (in_range) {
            const uint4 raw = *reinterpret_cast<const uint4*>(x + static_cast<int64_t>(row) * ldx + col);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
            #pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(h[i]);
                v[2 * i] = f.x;
                v[2 * i + 1] = f.y;
            }
        } else {
            #pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0.0f;
        }
        float amax = 0.0f;
        #pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
        #pragma unroll
        for (int off = kLanesPerBlock / 2; off > 0; off /= 2)
            amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, off));
        float sf = fmaxf(amax, 1e-4f) / kQMax;                 // IEEE division, as torch computes it
        if (kUE8M0) sf = ceil_to_power_of_two(sf);
        const float inv = 1.0f / sf;
        if (in_range) {
            if constexpr (!kFP4) {
                uint32_t lo = 0, hi = 0;
                #pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t b0 = __nv_cvt_float_to_fp8(v[i] * inv, __NV_SATFINITE, __NV_E4M3);
                    const uint32_t b1 = __nv_cvt_float_to_fp8(v[4 + i] * inv, __NV_SATFINITE, __NV_E4M3);
                    lo |= b0 << (8 * i);
                    hi |= b1 << (8 * i);
                }
                *reinterpret_cast<uint2*>(q + static_cast<int64_t>(row) * ldq + col) = make_uint2(lo, hi);
            } else {
                uint32_t word = 0;
                #pragma unroll
                for (int i = 0; i < 8; ++i) word |= e2m1_code(v[i] * inv) << (4 * i);      // even K in the low nibble
                *reinterpret_cast<uint32_t*>(q + static_cast<int64_t>(row) * ldq + col / 2) = word;
            }
        }
        // Scales
        if constexpr (!kPacked) {
            if (in_range && lane16 % kLanesPerBlock == 0)
                reinterpret_cast<float*>(sf_out)[static_cast<int64_t>(row) * sf_pitch + col / kGranK] = sf;
        } else {
            const uint32_t exponent = __float_as_uint(sf) >> 23;
            if constexpr (kGranK == 128) {
                // one exponent per 128 columns: byte `step` of the row's word for this 512-column span
                my_bytes |= (col < k ? exponent : 0u) << (8 * step);
            } else {
                // four exponents per 128 columns (lanes 0, 4, 8, 12 hold them): one word per step
                uint32_t word = 0;
                #pragma unroll
                for (int b = 0; b < 4; ++b) {
                    const uint32_t e = __shfl_sync(0xFFFFFFFFu, exponent, (threadIdx.x % 32) / 16 * 16 + b * 4);
                    word |= (col0 + step * 128 + b * 32 < k ? e : 0u) << (8 * b);
                }
                if (lane16 == 0) packed_words[step][row_in_cta] = word;
            }
        }
    }
    if constexpr (kPacked) {
        if constexpr (kGranK == 128) {
            if (lane16 == 0) packed_words[0][row_in_cta] = my_bytes;
        }
        __syncthreads();
        // MN-major store: consecutive rows are consecutive int32
        constexpr int kWordsPerRow = kGranK == 128 ? 1 : kColsPerCta / 128;
        const int32_t word_col0 = kGranK == 128 ? blockIdx.x : blockIdx.x * kWordsPerRow;
        const int total_word_cols = (k + kGranK * 4 - 1) / (kGranK * 4);
        for (int i = threadIdx.x; i < kWordsPerRow * kRowsPerCta; i += blockDim.x) {
            const int w = i / kRowsPerCta, r = i % kRowsPerCta;
            const int out_row = blockIdx.y * kRowsPerCta + r;
            if (out_row < m && word_col0 + w < total_word_cols)
                reinterpret_cast<uint32_t*>(sf_out)[static_cast<int64_t>(word_col0 + w) * sf_pitch + out_row] = packed_words[w][r];
        }
    }
}

template <int kGranK, bool kFP4>
int launch(const void* x, int64_t ldx, void* q, int64_t ldq, void* sf, int64_t sf_pitch, int m, int k, bool packed, bool ue8m0,
           cudaStream_t stream) {
    const dim3 grid(ceil_div(k, kColsPerCta), ceil_div(m, kRowsPerCta));
    const auto* xp = static_cast<const __nv_bfloat16*>(x);
    auto* qp = static_cast<uint8_t*>(q);
    if (packed)
        per_token_cast_kernel<kGranK, kFP4, true, true><<<grid, 256, 0, stream>>>(xp, ldx, qp, ldq, sf, sf_pitch, m, k);
    else if (ue8m0)
        per_token_cast_kernel<kGranK, kFP4, false, true><<<grid, 256, 0, stream>>>(xp, ldx, qp, ldq, sf, sf_pitch, m, k);
    else
        per_token_cast_kernel<kGranK, kFP4, false, false><<<grid, 256, 0, stream>>>(xp, ldx, qp, ldq, sf, sf_pitch, m, k);
    DG_CUDA_RT(cudaGetLastError());
    return DG_OK;
}

}  // namespace
}  // namespace dg

using namespace dg;

extern "C" int dg_per_token_cast(const void* x_bf16, int64_t ldx, void* q, int64_t ldq, void* sf, int64_t sf_pitch,
                                 int m, int k, int out_dtype, int gran_k, int packed_ue8m0, int use_ue8m0, void* stream) {
    DG_REQUIRE(m >= 0 && k >= 0);
    DG_REQUIRE(out_dtype == DG_FP8_E4M3 || out_dtype == DG_FP4_E2M1_X2);
    DG_REQUIRE(gran_k == 32 || gran_k == 128);
    DG_REQUIRE(!packed_ue8m0 || use_ue8m0);
    if (m == 0 || k == 0) return DG_OK;
    DG_REQUIRE(x_bf16 != nullptr && q != nullptr && sf != nullptr);
    DG_REQUIRE(k % 16 == 0);                                            // 16-byte loads; the GEMM's K pitch rule anyway
    DG_REQUIRE(ldx >= k && ldx % 8 == 0 && reinterpret_cast<uintptr_t>(x_bf16) % 16 == 0);
    const bool fp4 = out_dtype == DG_FP4_E2M1_X2;
    DG_REQUIRE(ldq >= (fp4 ? k / 2 : k) && ldq % 8 == 0 && reinterpret_cast<uintptr_t>(q) % 8 == 0);
    if (packed_ue8m0) DG_REQUIRE(sf_pitch >= align_up(m, 4));
    else DG_REQUIRE(sf_pitch >= ceil_div(k, gran_k));
    auto s = static_cast<cudaStream_t>(stream);
    if (gran_k == 128) return fp4 ? launch<128, true>(x_bf16, ldx, q, ldq, sf, sf_pitch, m, k, packed_ue8m0, use_ue8m0, s)
                                  : launch<128, false>(x_bf16, ldx, q, ldq, sf, sf_pitch, m, k, packed_ue8m0, use_ue8m0, s);
    return fp4 ? launch<32, true>(x_bf16, ldx, q, ldq, sf, sf_pitch, m, k, packed_ue8m0, use_ue8m0, s)
               : launch<32, false>(x_bf16, ldx, q, ldq, sf, sf_pitch, m, k, packed_ue8m0, use_ue8m0, s);
}
