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
    // Launched with programmatic stream serialisation right behind the GEMM that fills the panels: the blocks may
    // already be resident while that GEMM drains, and wait here until it has completed and its stores are visible
    asm volatile("griddepcontrol.wait;" ::: "memory");
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
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = dim3(256);
    config.stream = stream;
    cudaLaunchAttribute attr = {};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attr;
    config.numAttrs = 1;
    if (d_fp32)
        DG_CUDA_RT(cudaLaunchKernelEx(&config, splitk_reduce_kernel<true>, ws, d, m, n, ld_ws, panel_stride, ldd, num_splits, alpha));
    else
        DG_CUDA_RT(cudaLaunchKernelEx(&config, splitk_reduce_kernel<false>, ws, d, m, n, ld_ws, panel_stride, ldd, num_splits, alpha));
    return DG_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// Dense GEMM for callers that must not allocate
// ---------------------------------------------------------------------------------------------------------------
// Some callers run where device allocation at call time is off the table: a real-time serving thread that may not take
// the allocator's locks, a process that handed out its whole memory budget at start-up and forbids cudaMalloc afterwards
// so that its footprint stays fixed, a host application that owns all device memory itself.  The sliced (split-K) dense
// GEMM normally parks its FP32 partial panels in a library-owned buffer that grows on demand; for those callers the
// panels go into this fixed array instead.  It is part of the library image: every GPU that loads the library holds
// these 16 MiB until the process exits.  One array per device, shared by all calls of the entry point below on that
// device (calls that overlap on the GPU race on it); dg_fp8_fp4_gemm never touches it.
constexpr size_t kFixedScratchBytes = 16u << 20;
static __device__ __align__(256) float g_fixed_splitk_scratch[kFixedScratchBytes / sizeof(float)];

int run_dense_gemm_with_fixed_scratch(const dg_gemm_args_t* args, float* scratch, size_t scratch_bytes);   // dg_gemm.cpp

namespace {

// In host code the array's name is only a handle; the device address has to be asked for, once per device, with that
// device current.
int fixed_scratch_address(float** out) {
    constexpr int kMaxDevices = 64;
    static std::mutex mu;
    static float* address[kMaxDevices] = {};
    int device = 0;
    DG_CUDA_RT(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) return fail(DG_ERR_INVALID_ARGUMENT, "device ordinal %d out of range", device);
    std::lock_guard<std::mutex> lock(mu);
    if (address[device] == nullptr) {
        void* ptr = nullptr;
        DG_CUDA_RT(cudaGetSymbolAddress(&ptr, g_fixed_splitk_scratch));
        address[device] = static_cast<float*>(ptr);
    }
    *out = address[device];
    return DG_OK;
}

}  // namespace
}  // namespace dg

extern "C" int dg_fp8_fp4_gemm_noalloc(const dg_gemm_args_t* args) {
    float* scratch = nullptr;
    const int rc = dg::fixed_scratch_address(&scratch);
    if (rc != DG_OK) return rc;
    return dg::run_dense_gemm_with_fixed_scratch(args, scratch, dg::kFixedScratchBytes);
}
