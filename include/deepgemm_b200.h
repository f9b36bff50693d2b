/*
 * C ABI of the B200 (sm_100a) block-scaled FP8 / FP8xFP4 GEMM library.
 *
 * Plain pointers and sizes only.  Every pointer named "device" is a CUDA device pointer of the
 * current device; `stream` is a cudaStream_t / CUstream passed as void*.  All functions return
 * DG_OK (0) or a dg_status_t error code; dg_last_error() gives the message of the last failure on
 * the calling thread.  Nothing here synchronises the host with the device unless it says so.
 *
 * Each entry point names the interface of the reference (DeepGEMM 2.8.1 tree, paths relative to
 * its root) that it stands in for.
 */
#ifndef DEEPGEMM_B200_H_
#define DEEPGEMM_B200_H_

#include <stdint.h>

#if defined(__GNUC__)
#define DG_API __attribute__((visibility("default")))
#else
#define DG_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum dg_status {
    DG_OK = 0,
    DG_ERR_INVALID_ARGUMENT = 1,   /* an assertion of the reference's API layer would have fired */
    DG_ERR_CUDA = 2,               /* a CUDA driver / runtime call failed */
    DG_ERR_JIT = 3,                /* nvcc failed or the kernel image could not be loaded */
    DG_ERR_UNSUPPORTED = 4,        /* valid for the reference, not built here (message says what) */
    DG_ERR_KERNEL = 5              /* a kernel reported a failed bounded wait through the status word */
} dg_status_t;

typedef enum dg_dtype {
    DG_FP8_E4M3 = 0,               /* torch.float8_e4m3fn */
    DG_FP4_E2M1_X2 = 1,            /* two e2m1 codes per byte, even K in the low nibble (torch.int8 in the reference, csrc/utils/math.hpp:11) */
    DG_BF16 = 2,
    DG_FP32 = 3
} dg_dtype_t;

typedef enum dg_major { DG_MAJOR_K = 0, DG_MAJOR_MN = 1 } dg_major_t;

typedef enum dg_gemm_kind {
    DG_GEMM_DENSE = 0,
    DG_GEMM_M_GROUPED_CONTIGUOUS = 1,
    DG_GEMM_M_GROUPED_MASKED = 2,
    DG_GEMM_M_GROUPED_CONTIGUOUS_PSUM = 3,    /* the contiguous layout with use_psum_layout (for dg_get_gemm_config / dg_gemm_precompile) */
    DG_GEMM_K_GROUPED_CONTIGUOUS = 4,
    DG_GEMM_BATCHED = 5
} dg_gemm_kind_t;

DG_API const char* dg_last_error(void);

/* ---- library life cycle and process-wide settings: csrc/apis/config.hpp:9-47 ------------------ */

/* init(library_root_path): where the device headers (csrc/device) and the in-tree kernel cache live.
 * Touches no CUDA context (deep_gemm/__init__.py:122, tests/test_lazy_init.py:18-19). */
DG_API int dg_init(const char* library_root);
/* shutdown(): releases what the library allocated on the devices (split-K panels, the status word); a second call is a
 * no-op; the runtime is not recreated, every later GEMM or setter fails (tests/test_lazy_init.py:78-90). */
DG_API int dg_shutdown(void);
DG_API int dg_is_shut_down(void);                /* 1 after dg_shutdown */
DG_API int dg_set_num_sms(int num_sms);          /* must be even and at most the device's SM count (heuristics/config.hpp:60) */
DG_API int dg_get_num_sms(void);                 /* the override, else the device's SM count, else 148 without a device */
DG_API int dg_set_tc_util(int percent);          /* csrc/runtime/runtime.hpp:88-100; kept for API parity, unused by these kernels */
DG_API int dg_get_tc_util(void);
DG_API int dg_set_pdl(int enabled);              /* programmatic dependent launch attribute on every GEMM launch */
DG_API int dg_get_pdl(void);

/* ---- m-grouped contiguous layout alignment: csrc/apis/layout.hpp:133-141 ----------------------- */
DG_API int dg_set_mk_alignment_for_contiguous_layout(int alignment);        /* unvalidated, like the reference */
DG_API int dg_get_mk_alignment_for_contiguous_layout(void);                 /* default 128 (heuristics/runtime.hpp:12,18) */
DG_API int dg_get_theoretical_mk_alignment_for_contiguous_layout(int expected_m_or_negative);  /* 256 on sm_100 (heuristics/runtime.hpp:57-64) */

/* ---- scaling-factor layout: csrc/apis/layout.hpp:11-58, csrc/jit_kernels/impls/smxx_layout.hpp ---- */

/* get_tma_aligned_size(x, element_size): csrc/utils/math.hpp:23-27.  Returns the aligned size, or -1. */
DG_API int dg_get_tma_aligned_size(int x, int element_size);

/* FP32 power-of-two scales [num_groups, ceil(mn / gran_mn), sf_k] with element strides (in_stride_*)
 * -> packed UE8M0 int32 [num_groups, mn, ceil(sf_k / 4)] with element strides
 * (ceil(sf_k/4) * align(mn,4), 1, align(mn,4)); rows are broadcast along MN by gran_mn.
 * Replaces index_select + get_mn_major_tma_aligned_packed_ue8m0_tensor (csrc/apis/layout.hpp:44-50,
 * smxx_layout.hpp:133-216; kernels deep_gemm/include/deep_gemm/impls/smxx_layout.cuh:78,195).
 * `out` must hold num_groups * ceil(sf_k/4) * align(mn,4) int32 (device). */
DG_API int dg_pack_fp32_into_ue8m0(const float* sf_device, int32_t* out_device,
                            int num_groups, int mn, int sf_k, int gran_mn,
                            int64_t in_stride_group, int64_t in_stride_mn, int64_t in_stride_k,
                            void* stream);

/* The same packing for SFA of an m-grouped contiguous GEMM with a prefix-sum layout
 * (get_mn_major_tma_aligned_packed_ue8m0_tensor(sf, psum_layout), smxx_layout.hpp:133-184): rows that lie in no group
 * (between the end of a group and the next multiple of the contiguous-layout alignment, and after the last group) are
 * not read and get the scale code 0.  `psum_layout_device` holds num_psum_groups int32 row ends (device). */
DG_API int dg_pack_fp32_into_ue8m0_psum(const float* sf_device, int32_t* out_device, int mn, int sf_k,
                                        int64_t in_stride_mn, int64_t in_stride_k,
                                        const int32_t* psum_layout_device, int num_psum_groups, void* stream);

/* K-grouped scales (get_k_grouped_mn_major_tma_aligned_packed_ue8m0_tensor, smxx_layout.hpp:218-283; kernel
 * pack_fp32_into_ue8m0, impls/smxx_layout.cuh:195-267): FP32 [sf_rows, mn] contiguous, one row per gran_k elements of K,
 * the groups one after another, each covering its slice padded to the contiguous-layout alignment -> int32
 * [packed_rows, mn] contiguous: four rows per word, every group starting a new packed row, unused slots zero.
 * `grouped_layout_device` as in dg_k_grouped_fp8_gemm_contiguous.  packed_rows: sum over groups of
 * ceil(padded slice / (4 gran_k)); any larger value is allowed and the extra rows are written as zero. */
DG_API int dg_pack_k_grouped_fp32_into_ue8m0(const float* sf_device, int32_t* out_device, const int32_t* grouped_layout_device,
                                             int num_groups, int mn, int sf_rows, int packed_rows, int gran_k,
                                             int use_psum_layout, void* stream);

/* FP32 scales [num_groups, mn, sf_k] (any strides) -> same values MN-major with pitch align(mn,4):
 * get_mn_major_tma_aligned_tensor (smxx_layout.hpp:60-106; kernel smxx_layout.cuh:13).
 * `out` must hold num_groups * sf_k * align(mn,4) floats (device). */
DG_API int dg_transpose_fp32_mn_major(const float* sf_device, float* out_device,
                               int num_groups, int mn, int sf_k,
                               int64_t in_stride_group, int64_t in_stride_mn, int64_t in_stride_k,
                               void* stream);

/* Per-token (1 x gran_k) cast of BF16 activations [m, k] (row pitch ldx elements) to float8_e4m3 [m, k] or packed
 * float4_e2m1 [m, k/2] (row pitch ldq bytes), with the scales written either as FP32 [m, ceil(k/gran_k)] (row pitch
 * sf_pitch floats) or, with packed_ue8m0 != 0, directly as the packed UE8M0 int32 tensor the GEMMs take
 * ([m, ceil(k/(4 gran_k))], MN contiguous, K pitch sf_pitch >= align(m,4) int32): the "produce pre-transformed SFs in
 * the cast kernel" path of docs/scaling-factor-format.md:123-139.  Same arithmetic as per_token_cast_to_fp8 /
 * per_token_cast_to_fp4 of deep_gemm/utils/math.py:26-49,99-125.  k must be a multiple of 16. */
DG_API int dg_per_token_cast(const void* x_bf16_device, int64_t ldx, void* q_device, int64_t ldq, void* sf_device, int64_t sf_pitch,
                             int m, int k, int out_dtype, int gran_k, int packed_ue8m0, int use_ue8m0, void* stream);

/* ---- GEMMs: csrc/apis/gemm.hpp:78-318 ----------------------------------------------------------- */

typedef struct dg_gemm_args {
    /* operands (device).  SFs are the packed UE8M0 int32 tensors of docs/scaling-factor-format.md:42-63:
     * [groups?, mn, ceil(k / (4 gran_k))], MN contiguous, K pitch = sf*_pitch (>= align(mn,4), % 4 == 0),
     * groups packed tightly (group stride = pitch * ceil(k / (4 gran_k))). */
    const void* a;
    const void* sfa;
    const void* b;
    const void* sfb;
    void* d;
    int32_t m;                 /* dense/contiguous: rows of A; masked: max_m (rows per group) */
    int32_t n;
    int32_t k;                 /* logical K (twice the byte count of a packed FP4 row) */
    int32_t num_groups;        /* 1 for dense */
    int32_t a_dtype;           /* dg_dtype_t: DG_FP8_E4M3 or DG_FP4_E2M1_X2 */
    int32_t b_dtype;
    int32_t d_dtype;           /* DG_BF16, DG_FP32 (dense only) or DG_FP8_E4M3 (dense only, with sfd below) */
    int32_t major_a;           /* dg_major_t; K-major: rows of K contiguous */
    int32_t major_b;
    int64_t lda;               /* pitch between rows (K-major) or between K slices (MN-major), in storage elements (bytes) */
    int64_t ldb;
    int64_t ldd;               /* row pitch of D in elements */
    int64_t sfa_pitch;         /* stride(-1) of SFA in int32 elements */
    int64_t sfb_pitch;
    int32_t gran_k_a;          /* 32 or 128 */
    int32_t gran_k_b;
    int32_t accumulate;        /* non-zero: D += alpha A B^T (the reference's c == d case, gemm.hpp:17-53) */
    int32_t has_alpha;
    float alpha;               /* used when has_alpha != 0 (epilogue Alpha, csrc/jit_kernels/impls/epilogue_class.hpp:111-127) */
    const int32_t* grouped_layout; /* contiguous: int32[m] expert id per row, -1 on padding; masked: int32[num_groups] rows used;
                                    * contiguous with use_psum_layout: int32[num_groups], the row where each group ends */
    int32_t expected_m;        /* masked, and contiguous with use_psum_layout (0 = unknown): heuristic hint only (gemm.hpp:269-318) */
    void* stream;
    /* Contiguous layout only (gemm.hpp:190-192,213-220; docs/scaling-factor-format.md 7.3).  With use_psum_layout group g
     * occupies rows [align(grouped_layout[g-1], mk_alignment), grouped_layout[g]) of A and D (from row 0 for g = 0); the
     * rows in between are padding.  ensure_zero_padding != 0 also writes the padding rows of D up to the next aligned
     * row (zero when A's padding rows are zero, as the reference's assert_psum_zero_padding checks); otherwise no row
     * outside a group is written. */
    int32_t use_psum_layout;
    int32_t ensure_zero_padding;
    /* Dense GEMM with d_dtype == DG_FP8_E4M3: the FP8Quantization epilogue (csrc/jit_kernels/impls/epilogue_class.hpp:69-92,
     * deep_gemm/include/deep_gemm/epilogue/operators.cuh:68-92).  D [m, n] is written as float8_e4m3 (ldd in bytes) and
     * `sfd` receives one UE8M0 scale per row and 32 columns, packed four to an int32 in the layout the GEMMs take for SFA:
     * [m, ceil(n / 128)] int32, MN contiguous, K pitch sfd_pitch (>= align(m, 4)).  Each accumulator is rounded to BF16
     * first, so D and sfd equal a BF16 D followed by dg_per_token_cast(gran_k 32, packed).  Not combined with accumulate
     * or alpha; words of sfd beyond column n keep the bytes they had. */
    void* sfd;
    int64_t sfd_pitch;
    /* dg_fp8_bmm only: distance between consecutive batches of A, B and D in storage elements (any value whose byte
     * count is a multiple of 16: the permuted views of fp8_einsum are expressed this way).  The scale tensors of a
     * batched GEMM are packed tightly: batch stride = sf*_pitch * ceil(k / (4 gran_k)) int32. */
    int64_t batch_stride_a;
    int64_t batch_stride_b;
    int64_t batch_stride_d;
    /* BF16StochasticRounding epilogue (epilogue_class.hpp:94-108, epilogue/operators.cuh:32-63): a BF16 D is rounded
     * stochastically instead of to nearest; the random bits are a hash of the four FP32 accumulators of columns
     * 4q .. 4q+3 and of q (tests/utils.py:53-79 states it), so the result is reproducible.  BF16 output only, not
     * combined with accumulate or alpha; K is never sliced. */
    int32_t stochastic_rounding;
    /* einsum 'bmk,bnk->mn' (csrc/apis/einsum.hpp:22-58, csrc/jit_kernels/impls/sm100_bmk_bnk_mn.hpp): with reduce_batches =
     * S > 1 the dense BF16 GEMM sums over S batches as well, D[m,n] = sum over s of A[s] @ B[s]^T with A [S, M, K] and
     * B [S, N, K] (K-major, batches batch_stride_a / batch_stride_b elements apart, k % 64 == 0): the K loop walks
     * (batch, K-block) pairs, so the reduction is one GEMM with K' = S * K.  dg_fp8_fp4_gemm only; D BF16 or FP32. */
    int32_t reduce_batches;
} dg_gemm_args_t;

/* fp8_fp4_gemm_nt and, through major_a / major_b, nn / tn / tt (gemm.hpp:78-179). */
DG_API int dg_fp8_fp4_gemm(const dg_gemm_args_t* args);
/* m_grouped_fp8_fp4_gemm_nt_contiguous / nn (gemm.hpp:181-267), with either form of grouped_layout. */
DG_API int dg_m_grouped_fp8_fp4_gemm_contiguous(const dg_gemm_args_t* args);
/* m_grouped_fp8_fp4_gemm_nt_masked (gemm.hpp:269-318). */
DG_API int dg_m_grouped_fp8_fp4_gemm_masked(const dg_gemm_args_t* args);
/* k_grouped_fp8_gemm_tn_contiguous (gemm.hpp:320-372; the weight-gradient GEMM of a mixture of experts):
 * D[g] (+)= A[slice g of K]^T B[slice g of K] for g < num_groups, with
 *   a, b : float8_e4m3 [k, m] / [k, n] (major_* = DG_MAJOR_MN, lda = m, the reference's layout) or [m, k] / [n, k]
 *          (DG_MAJOR_K); k = the sum of the (padded) slices; padding rows must be zero;
 *   d    : [num_groups, m, n] BF16 or FP32, row pitch ldd, groups m rows apart; accumulate != 0 adds into it;
 *   grouped_layout : int32[num_groups] on the device: each slice's length, a multiple of the contiguous-layout
 *          alignment, or with use_psum_layout the element where it ends, the next slice starting at the following
 *          multiple of the alignment (docs/scaling-factor-format.md 5.1);
 *   sfa, sfb : packed UE8M0 int32 [rows, m] / [rows, n], MN contiguous (pitch sf*_pitch >= mn, mn % 4 == 0), one row per
 *          4 * gran_k elements of K, every group starting a new row (docs/scaling-factor-format.md 5.2;
 *          dg_pack_k_grouped_fp32_into_ue8m0 produces it); gran_k_a == gran_k_b.
 * An empty slice gives D[g] = 0 (leaves it unchanged when accumulating). */
DG_API int dg_k_grouped_fp8_gemm_contiguous(const dg_gemm_args_t* args);
/* fp8_bmm behind fp8_einsum (csrc/apis/einsum.hpp:183-243): D[b] = C[b] + A[b] B[b]^T for b < num_groups, every operand
 * a [num_groups, rows, K-or-MN] tensor with its own batch stride (batch_stride_* above) and row pitch (lda / ldb / ldd);
 * FP8 operands, K- or MN-major; D BF16, FP32 or, with sfd, e4m3 (then n % 128 == 0 and batch_stride_d == n: sfd is the
 * scale tensor of D viewed as [m, num_groups * n]).  Rows beyond m are clipped per batch. */
DG_API int dg_fp8_bmm(const dg_gemm_args_t* args);

/* Same operation and arguments as dg_fp8_fp4_gemm, for callers that cannot allocate device memory at call time: a
 * serving thread that must never block on the allocator's locks, a process that hands out its whole memory budget at
 * start-up and forbids cudaMalloc afterwards, a plugin host that owns all device memory itself.  It has no counterpart
 * in the reference.  The scratch of the K-sliced path (FP32 partial panels) lives in a 16 MiB array inside the library
 * image, which every GPU that loads the library keeps until exit; the call performs no cudaMalloc / cudaFree /
 * cudaHostAlloc and calls no allocating library routine (with DG_PROFILE set it runs without the tuning counters, which
 * would need a buffer).  A GEMM whose slicing needs more than 16 MiB of panels (num_splits * align(m,128) *
 * align(n,4) * 4 bytes) is rejected with DG_ERR_INVALID_ARGUMENT and nothing is launched.  The first call on a device
 * looks up the array's device address (and, like every entry point, the first call of a tile configuration loads its
 * kernel image): make that first call before any stream capture.  There is one array per device, shared by every call
 * of this entry point on that device, and it keeps the last call's panels; nothing in it has to start at zero (every
 * element that is read is written first by the same call), but two calls of this entry point that overlap on one GPU
 * (from two streams) race on it.  Calls of dg_fp8_fp4_gemm use a different, library-owned buffer, so mixing the two
 * entry points does not race.  Failed bounded waits are reported through the status word only if another entry point
 * has already created it. */
DG_API int dg_fp8_fp4_gemm_noalloc(const dg_gemm_args_t* args);

/* Compile (but do not load or launch) the kernel the call above would use, so that a later call
 * finds it in the cache.  Needs nvcc, not a GPU.  Device pointers in `args` may be null. */
DG_API int dg_gemm_precompile(int kind, const dg_gemm_args_t* args);

/* ---- heuristics: csrc/jit_kernels/heuristics/{common,sm100}.hpp -------------------------------- */

typedef struct dg_gemm_config {
    int32_t block_m, block_n, block_k;
    int32_t num_stages;
    int32_t cluster_size;      /* CTAs per cluster (1 or 2) */
    int32_t raster_group;      /* row blocks per band of the tile order */
    int32_t num_ctas;          /* grid size */
    int32_t smem_bytes;
    int32_t tmem_cols;
    int32_t num_tiles;         /* dense / contiguous: exact; masked: estimated from expected_m */
    int32_t waves_x100;
    int32_t num_splits;        /* slices of K per output tile (dense GEMMs with few tiles); 1 = not split */
    int32_t kb_per_split;      /* K-blocks (128 of K) per slice */
    int32_t split_in_cluster;  /* 1: the slices of a tile are the CTAs of one thread-block cluster, whose first CTA adds the
                                  others' accumulators from their shared memory (no workspace, no second kernel) */
    int32_t swap_ab;           /* 1: dense GEMM with few rows run with the operands' roles exchanged: block_m counts rows of the
                                  caller's B, block_n is the caller's M rounded up to 16, and the epilogue writes D transposed */
    int32_t store_buffers;     /* staging buffers of D per epilogue warpgroup (2; 1 where that buys a third pipeline stage) */
    int32_t a_rows;            /* rows of A a pipeline stage holds: block_m, or fewer (16/32/64) when the whole GEMM has no more rows,
                                  which leaves room for more stages */
} dg_gemm_config_t;

/* get_best_config<SM100ArchSpec> (heuristics/common.hpp:17-56, sm100.hpp:30-301).  Host only. */
DG_API int dg_get_gemm_config(int kind, const dg_gemm_args_t* args, dg_gemm_config_t* config);

/* Host model of the device tile scheduler (scheduler/gemm.cuh:108-263 in the reference): lists the
 * tiles CTA `cta` of `num_ctas` visits, four uint32 per tile {m_block, n_block, group, valid_rows}
 * (prefix-sum layout: m_block counts from row 0 of A; k-grouped: the fourth word is the slice's K-block count).
 * `layout` is a HOST pointer here.  Returns the number of tiles (may exceed max_tiles; only
 * max_tiles are written) or a negative dg_status_t. */
DG_API int dg_enumerate_tiles(int kind, int block_n, int raster_group, int shape_m, int shape_n, int num_groups,
                       const int32_t* layout_host, int cta, int num_ctas, uint32_t* out, int max_tiles);

/* ---- JIT runtime: csrc/runtime/jit.hpp + third-party/deep_jit (README.md:164-191) --------------- */

typedef struct dg_kernel* dg_kernel_t;

/* Compile `source` (CUDA C++, entry point `entry`, extern "C") to an sm_100a cubin, or find it in the
 * cache (key: source + flags + compiler version).  Cache: $DG_JIT_CACHE_DIR, else <library_root>/_jit_cache
 * if writable, else $HOME/.deepgemm_b200.  Honours DG_JIT_DEBUG, DG_JIT_PRINT_COMPILER_COMMAND,
 * DG_JIT_PTXAS_VERBOSE, DG_JIT_WITH_LINEINFO, DG_JIT_NVCC_COMPILER. */
DG_API int dg_jit_compile(const char* name, const char* entry, const char* source, const char* extra_flags, dg_kernel_t* kernel);
/* Path of the cached cubin of a compiled kernel. */
DG_API const char* dg_jit_kernel_path(dg_kernel_t kernel);
/* How many clusters of `cluster_x` CTAs of this kernel (block_x threads, smem_bytes of dynamic shared memory) the
 * current device can hold at once (cuOccupancyMaxActiveClusters).  Loads the kernel image if needed. */
DG_API int dg_jit_max_active_clusters(dg_kernel_t kernel, uint32_t block_x, uint32_t cluster_x, uint32_t smem_bytes,
                                      int* num_clusters);

/* cuLaunchKernelEx on `stream`; loads the module into the current context on first use. */
DG_API int dg_jit_launch(dg_kernel_t kernel, uint32_t grid_x, uint32_t block_x, uint32_t cluster_x,
                  uint32_t smem_bytes, int enable_pdl, void* stream, void** kernel_args);

/* ---- kernel status word ------------------------------------------------------------------------- */
/* Every wait inside the kernels is bounded; a wait that runs out writes a code here and the kernel
 * unwinds.  Returns the word (0 = no failure) WITHOUT synchronising: call after the stream is idle. */
DG_API int dg_kernel_status(void);
DG_API int dg_reset_kernel_status(void);
/* Exercises the expiry path without a fault: a one-CTA kernel built from the kernels' own wait primitive, with the
 * limit lowered to timeout_us (100 .. 1e6), waits on a barrier nobody arrives at, gives up, records its code
 * (role 7, site 3, CTA 0 -> 0x87030000) in the status word and returns normally; a second waiter of the CTA must leave
 * through the abort flag without reporting.  elapsed_ns (optional, two words) receives how long each waited.
 * Synchronises `stream`.  The reference's only bounded wait traps after 60 s instead
 * (deep_gemm/include/deep_gemm/comm/barrier.cuh:11-24). */
DG_API int dg_selftest_bounded_wait(uint32_t timeout_us, void* stream, uint64_t* elapsed_ns);

#ifdef __cplusplus
}
#endif
#endif  /* DEEPGEMM_B200_H_ */
