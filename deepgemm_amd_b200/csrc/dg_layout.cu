// Scaling-factor layout kernels: FP32 power-of-two scales -> packed UE8M0 int32 in the MN-major,
// TMA-aligned layout, and the plain FP32 MN-major transpose.  Same results as the reference's
// transpose_and_pack_fp32_into_ue8m0 / pack_fp32_into_ue8m0 / transpose_fp32
// (deep_gemm/include/deep_gemm/impls/smxx_layout.cuh:13,78,195) and its pure-torch fallback
// (csrc/jit_kernels/impls/smxx_layout.hpp:108-131), for any input strides, with the broadcast of a
// coarser MN granularity (csrc/apis/layout.hpp:47-49) folded into the read.
//
// HBM-bound byte shuffling: a 32(mn) x 32(packed k) tile goes through shared memory so that both
// the reads (contiguous along K in the usual input) and the writes (contiguous along MN) coalesce.
#include "dg_common.hpp"

namespace dg {
namespace {

constexpr int kTileMN = 32;
constexpr int kTileK = 32;      // packed words along K per tile (128 scales)

// Prefix-sum layout of the m-grouped contiguous GEMM: group g holds rows [align(ends[g-1], alignment), ends[g]);
// every other row is padding whose input scale may be uninitialised.
__device__ __forceinline__ bool row_in_a_group(int row, const int* __restrict__ ends, int num_groups, int alignment) {
    int start = 0;
    for (int g = 0; g < num_groups; ++g) {
        const int end = ends[g];
        if (row < end) return row >= start;
        start = (max(end, start) + alignment - 1) / alignment * alignment;
    }
    return false;
}

// Input element (g, row, k) sits at g * sg + (row / gran_mn) * sm + k * sk.  With `psum_ends` (the prefix-sum layout,
// num_psum_groups entries) rows outside every group are not read and get the scale code 0, a finite value
// (docs/scaling-factor-format.md 7.3 of the reference).
__global__ void __launch_bounds__(256)
pack_fp32_into_ue8m0_kernel(const float* __restrict__ sf, int32_t* __restrict__ out,
                            int mn, int sf_k, int packed_k, int aligned_mn, int gran_mn,
                            int64_t sg, int64_t sm, int64_t sk, int* status,
                            const int* __restrict__ psum_ends, int num_psum_groups, int psum_alignment) {
    __shared__ uint32_t tile[kTileK][kTileMN + 1];
    const int g = blockIdx.z;
    const int mn0 = blockIdx.x * kTileMN, pk0 = blockIdx.y * kTileK;
    const float* src = sf + g * sg;
    // Read: thread (ty, tx) covers row mn0 + ty + 8 i and packed word pk0 + tx (4 scales, K-contiguous reads)
    const int tx = threadIdx.x % 32, ty = threadIdx.x / 32;
    #pragma unroll
    for (int i = 0; i < kTileMN / 8; ++i) {
        const int r = mn0 + ty + 8 * i, pk = pk0 + tx;
        uint32_t word = 0;
        const bool gap = psum_ends != nullptr && r < mn && !row_in_a_group(r, psum_ends, num_psum_groups, psum_alignment);
        if (r < mn && pk < packed_k && !gap) {
            const float* row = src + static_cast<int64_t>(r / gran_mn) * sm;
            #pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int k = pk * 4 + j;
                if (k < sf_k) {
                    const uint32_t bits = __float_as_uint(row[static_cast<int64_t>(k) * sk]);
                    // A scale must be a positive power of two (sign and mantissa clear); report, do not trap
                    if ((bits & 0x807FFFFFu) != 0 && status != nullptr) atomicCAS(status, 0, static_cast<int>(0x89000000u));
                    word |= (bits >> 23) << (8 * j);
                }
            }
        }
        tile[tx][ty + 8 * i] = word;
    }
    __syncthreads();
    // Write: thread (ty, tx) covers packed word pk0 + ty + 8 i and row mn0 + tx (MN-contiguous writes)
    int32_t* dst = out + static_cast<int64_t>(g) * packed_k * aligned_mn;
    #pragma unroll
    for (int i = 0; i < kTileK / 8; ++i) {
        const int pk = pk0 + ty + 8 * i, r = mn0 + tx;
        if (pk < packed_k && r < aligned_mn)
            dst[static_cast<int64_t>(pk) * aligned_mn + r] = static_cast<int32_t>(tile[ty + 8 * i][tx]);   // pitch padding gets 0
    }
}

// K-grouped scales: input FP32 [sf_rows, mn] contiguous (one row per gran_k elements of K, groups one after another,
// each covering its padded slice), output int32 [packed_rows, mn]: four input rows per word, every group starting a
// new output row, the unused slots of a group's last row zero.  `layout` holds the slices' lengths or, with `psum`,
// their prefix sums (slices then start on multiples of `alignment`).  One CTA: one output row x 256 columns; every
// thread finds the row's group by walking the layout (at most a few hundred entries).
__global__ void __launch_bounds__(256)
pack_k_grouped_fp32_into_ue8m0_kernel(const float* __restrict__ sf, int32_t* __restrict__ out, const int* __restrict__ layout,
                                      int num_groups, int mn, int sf_rows, int gran_k, int alignment, int psum, int* status) {
    const int out_row = blockIdx.y, col = blockIdx.x * 256 + threadIdx.x;
    int k_start = 0, in_row0 = 0, out_row0 = 0, group_rows = 0;
    bool found = false;
    for (int g = 0; g < num_groups && !found; ++g) {
        const int v = max(layout[g], 0);
        const int len = psum ? max(v - k_start, 0) : v;
        const int padded = (len + alignment - 1) / alignment * alignment;
        group_rows = padded / gran_k;
        const int packed = (group_rows + 3) / 4;
        if (out_row < out_row0 + packed) {
            found = true;
        } else {
            k_start += padded; in_row0 += group_rows; out_row0 += packed;
        }
    }
    if (col >= mn) return;
    uint32_t word = 0;
    if (found) {
        #pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int r = (out_row - out_row0) * 4 + j;
            if (r < group_rows && in_row0 + r < sf_rows) {
                const uint32_t bits = __float_as_uint(sf[static_cast<int64_t>(in_row0 + r) * mn + col]);
                if ((bits & 0x807FFFFFu) != 0 && status != nullptr) atomicCAS(status, 0, static_cast<int>(0x89000000u));
                word |= (bits >> 23) << (8 * j);
            }
        }
    }
    out[static_cast<int64_t>(out_row) * mn + col] = static_cast<int32_t>(word);     // rows past the last group: zero
}

__global__ void __launch_bounds__(256)
transpose_fp32_kernel(const float* __restrict__ sf, float* __restrict__ out, int mn, int sf_k, int aligned_mn,
                      int64_t sg, int64_t sm, int64_t sk) {
    __shared__ float tile[kTileK][kTileMN + 1];
    const int g = blockIdx.z;
    const int mn0 = blockIdx.x * kTileMN, k0 = blockIdx.y * kTileK;
    const float* src = sf + g * sg;
    const int tx = threadIdx.x % 32, ty = threadIdx.x / 32;
    #pragma unroll
    for (int i = 0; i < kTileMN / 8; ++i) {
        const int r = mn0 + ty + 8 * i, k = k0 + tx;
        tile[tx][ty + 8 * i] = (r < mn && k < sf_k) ? src[static_cast<int64_t>(r) * sm + static_cast<int64_t>(k) * sk] : 0.0f;
    }
    __syncthreads();
    float* dst = out + static_cast<int64_t>(g) * sf_k * aligned_mn;
    #pragma unroll
    for (int i = 0; i < kTileK / 8; ++i) {
        const int k = k0 + ty + 8 * i, r = mn0 + tx;
        if (k < sf_k && r < aligned_mn) dst[static_cast<int64_t>(k) * aligned_mn + r] = tile[ty + 8 * i][tx];
    }
}

}  // namespace
}  // namespace dg

using namespace dg;

extern "C" {

int dg_pack_fp32_into_ue8m0(const float* sf, int32_t* out, int num_groups, int mn, int sf_k, int gran_mn,
                            int64_t in_stride_group, int64_t in_stride_mn, int64_t in_stride_k, void* stream) {
    DG_REQUIRE(num_groups > 0 && mn >= 0 && sf_k >= 0 && gran_mn > 0);
    if (mn == 0 || sf_k == 0) return DG_OK;
    DG_REQUIRE(sf != nullptr && out != nullptr);
    DG_REQUIRE(num_groups <= 65535);
    int rc = ensure_status_word();
    if (rc != DG_OK) return rc;
    const int packed_k = ceil_div(sf_k, 4), aligned_mn = align_up(mn, 4);
    const dim3 grid(ceil_div(aligned_mn, kTileMN), ceil_div(packed_k, kTileK), num_groups);
    DG_REQUIRE(grid.y <= 65535);
    pack_fp32_into_ue8m0_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        sf, out, mn, sf_k, packed_k, aligned_mn, gran_mn, in_stride_group, in_stride_mn, in_stride_k, state().status_device,
        nullptr, 0, 1);
    DG_CUDA_RT(cudaGetLastError());
    return DG_OK;
}

int dg_pack_fp32_into_ue8m0_psum(const float* sf, int32_t* out, int mn, int sf_k, int64_t in_stride_mn, int64_t in_stride_k,
                                 const int32_t* psum_layout, int num_psum_groups, void* stream) {
    DG_REQUIRE(mn >= 0 && sf_k >= 0 && num_psum_groups > 0);
    if (mn == 0 || sf_k == 0) return DG_OK;
    DG_REQUIRE(sf != nullptr && out != nullptr && psum_layout != nullptr);
    int rc = ensure_status_word();
    if (rc != DG_OK) return rc;
    const int packed_k = ceil_div(sf_k, 4), aligned_mn = align_up(mn, 4);
    const dim3 grid(ceil_div(aligned_mn, kTileMN), ceil_div(packed_k, kTileK), 1);
    DG_REQUIRE(grid.y <= 65535);
    pack_fp32_into_ue8m0_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        sf, out, mn, sf_k, packed_k, aligned_mn, 1, 0, in_stride_mn, in_stride_k, state().status_device,
        psum_layout, num_psum_groups, state().mk_alignment);
    DG_CUDA_RT(cudaGetLastError());
    return DG_OK;
}

int dg_pack_k_grouped_fp32_into_ue8m0(const float* sf, int32_t* out, const int32_t* grouped_layout, int num_groups,
                                      int mn, int sf_rows, int packed_rows, int gran_k, int use_psum_layout, void* stream) {
    DG_REQUIRE(num_groups > 0 && mn >= 0 && sf_rows >= 0 && packed_rows >= 0);
    DG_REQUIRE(gran_k == 32 || gran_k == 128);
    DG_REQUIRE(mn % 4 == 0);                                              // smxx_layout.hpp:229
    DG_REQUIRE(state().mk_alignment % 128 == 0);
    if (mn == 0 || packed_rows == 0) return DG_OK;
    DG_REQUIRE(sf != nullptr && out != nullptr && grouped_layout != nullptr);
    DG_REQUIRE(packed_rows <= 65535);
    int rc = ensure_status_word();
    if (rc != DG_OK) return rc;
    const dim3 grid(ceil_div(mn, 256), packed_rows, 1);
    pack_k_grouped_fp32_into_ue8m0_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        sf, out, grouped_layout, num_groups, mn, sf_rows, gran_k, state().mk_alignment, use_psum_layout != 0, state().status_device);
    DG_CUDA_RT(cudaGetLastError());
    return DG_OK;
}

int dg_transpose_fp32_mn_major(const float* sf, float* out, int num_groups, int mn, int sf_k,
                               int64_t in_stride_group, int64_t in_stride_mn, int64_t in_stride_k, void* stream) {
    DG_REQUIRE(num_groups > 0 && mn >= 0 && sf_k >= 0);
    if (mn == 0 || sf_k == 0) return DG_OK;
    DG_REQUIRE(sf != nullptr && out != nullptr);
    DG_REQUIRE(num_groups <= 65535);
    const int aligned_mn = align_up(mn, 4);
    const dim3 grid(ceil_div(aligned_mn, kTileMN), ceil_div(sf_k, kTileK), num_groups);
    DG_REQUIRE(grid.y <= 65535);
    transpose_fp32_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        sf, out, mn, sf_k, aligned_mn, in_stride_group, in_stride_mn, in_stride_k);
    DG_CUDA_RT(cudaGetLastError());
    return DG_OK;
}

}  // extern "C"
