// Second pass of a split-K GEMM: D[m][n] = convert(alpha * sum over slices s of panel_s[m][n]), the panels being
// the FP32 partial results the GEMM kernel stored in the workspace.  Slices are added in index order by one thread
// per four columns, so the sum is bitwise reproducible.  HBM/L2-bound streaming: 4 * S bytes read and 2 (or 4)
// written per output element, 16-byte loads, fully coalesced.
#include "dg_common.hpp"

#include <cuda_bf16.h>

namespace dg {
namespace {

template <bool kOutFP32>
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ ws, void* __restrict__ d, int m, int n, int64_t ld_ws, int64_t panel_stride,
                     int64_t ldd, int num_splits, float alpha) {
    const int col = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    const int row = blockIdx.y;
    if (col >= n || row >= m) return;
    const float* src = ws + static_cast<int64_t>(row) * ld_ws + col;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    #pragma unroll 4
    for (int s = 0; s < num_splits; ++s) {
        const float4 q = __ldcg(reinterpret_cast<const float4*>(src + s * panel_stride));
        acc.x += q.x; acc.y += q.y; acc.z += q.z; acc.w += q.w;
    }
    acc.x *= alpha; acc.y *= alpha; acc.z *= alpha; acc.w *= alpha;
    if constexpr (kOutFP32) {
        float* out = reinterpret_cast<float*>(d) + static_cast<int64_t>(row) * ldd + col;
        if (col + 4 <= n) {
            *reinterpret_cast<float4*>(out) = acc;
        } else {
            const float v[4] = {acc.x, acc.y, acc.z, acc.w};
            for (int e = 0; col + e < n; ++e) out[e] = v[e];
        }
    } else {
        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(d) + static_cast<int64_t>(row) * ldd + col;
        if (col + 4 <= n) {
            const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
            uint2 packed;
            packed.x = *reinterpret_cast<const uint32_t*>(&lo);
            packed.y = *reinterpret_cast<const uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(out) = packed;
        } else {
            const float v[4] = {acc.x, acc.y, acc.z, acc.w};
            for (int e = 0; col + e < n; ++e) out[e] = __float2bfloat16_rn(v[e]);
        }
    }
}

}  // namespace

// ws: [num_splits][panel_rows][ld_ws] FP32 (ld_ws a multiple of 4); d: [m][ldd] BF16 or FP32 (row pitch a multiple of 16 bytes)
int launch_splitk_reduce(const float* ws, void* d, int m, int n, int64_t ld_ws, int64_t panel_rows, int64_t ldd, int num_splits,
                         float alpha, bool d_fp32, cudaStream_t stream) {
    const dim3 grid(ceil_div(ceil_div(n, 4), 256), m);
    const int64_t panel_stride = panel_rows * ld_ws;
    if (d_fp32)
        splitk_reduce_kernel<true><<<grid, 256, 0, stream>>>(ws, d, m, n, ld_ws, panel_stride, ldd, num_splits, alpha);
    else
        splitk_reduce_kernel<false><<<grid, 256, 0, stream>>>(ws, d, m, n, ld_ws, panel_stride, ldd, num_splits, alpha);
    DG_CUDA_RT(cudaGetLastError());
    return DG_OK;
}

}  // namespace dg
