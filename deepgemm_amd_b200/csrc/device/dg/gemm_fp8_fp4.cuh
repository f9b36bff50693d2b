// Persistent, warp-specialised block-scaled GEMM for sm_100a:
//     D[M,N] (+)= alpha * (SFA . A[M,K]) (SFB . B[N,K])^T
// A, B: float8_e4m3 or packed float4_e2m1, K-major; SFA / SFB: packed UE8M0 (four exponents per
// int32, MN-major) with one scale per 128 or per 32 elements of K; D: bf16 or fp32, row-major.
//
// It serves the same operations as the reference kernel sm100_fp8_fp4_gemm_1d1d_impl
// (deep_gemm/include/deep_gemm/impls/sm100_fp8_fp4_gemm_1d1d.cuh:38) for GemmType Normal,
// MGroupedContiguous and MGroupedMasked, with its own structure:
//
//   warp 0      TMA producer: fills a ring of kNumStages {A, B, SFA, SFB} shared-memory stages
//   warp 1      MMA issuer: one thread issues tcgen05.cp (scales -> tensor memory) and
//               tcgen05.mma.kind::mxf8f6f4.block_scale into one of two accumulators
//   warp 2      allocates tensor memory; rearranges each scale chunk for tcgen05.cp
//   warp 3      idle
//   warps 4-7   epilogue: tcgen05.ld -> alpha -> bf16/fp32 -> swizzled staging -> TMA store, 128 bytes of every
//               row (1, 2 or 4 store boxes) per synchronisation (row-predicated direct stores for ragged tiles
//               of the masked layout)
//   warps 8-11  a second epilogue warpgroup, only with 256-row tiles (DG_M_HALVES == 2)
//
// The configuration arrives as DG_* macros set by the host-side code generator:
//   DG_GEMM_TYPE (0 dense, 1 m-grouped contiguous, 2 m-grouped masked, 3 m-grouped contiguous with a prefix-sum
//   layout; DG_WRITE_PADDING for the latter, 4 k-grouped contiguous; DG_K_PSUM for its prefix-sum form), DG_M_HALVES, DG_BLOCK_N, DG_NUM_STAGES,
//   DG_CLUSTER, DG_A_FP4, DG_B_FP4, DG_MAJOR_A, DG_MAJOR_B (0 K-major, 1 MN-major), DG_GRAN_K_A, DG_GRAN_K_B,
//   DG_D_FP32, DG_D_FP8, DG_ACCUMULATE, DG_RASTER_GROUP, DG_SPLIT_K.
//
// DG_D_FP8 (dense only): the epilogue quantises D on the way out.  Every accumulator is first rounded to BF16, then each
// 32 columns of a row get one UE8M0 scale (amax clamped to 1e-4, / 448, rounded up to a power of two), D is stored as
// float8_e4m3 and the scale bytes go into a packed int32 tensor in the layout the GEMMs take for SFA (four scales per
// word, MN-major): the same bits as a BF16 D followed by the per-token 1 x 32 cast, which is how the reference defines
// its QuantizeToFP8 epilogue (deep_gemm/include/deep_gemm/epilogue/operators.cuh:68-92).
//
// k-grouped (type 4; the reference's sm100_k_grouped_fp8_gemm_1d1d, csrc/jit_kernels/impls/sm100_fp8_fp4_gemm_1d1d.hpp:325-441):
// D[g] (+)= A[slice g of K]^T B[slice g of K] for every group g, A and B being [sum K, M] and [sum K, N] (MN-major) or
// [M, sum K] and [N, sum K] (K-major), D [G, M, N] in FP32 or BF16, the scales one packed row per 4 * gran_k elements of
// K with every group starting a new row.  The slices are read on the device; an empty slice gives a zero D[g]
// (nothing, when accumulating).  Rows of a tile beyond M are stored one by one so that D[g + 1] is not touched.
//
// batched (type 5; the reference's sm100_fp8_bmm behind fp8_einsum): num_groups GEMMs of one shape; every tensor map
// is three-dimensional with the batch outermost, so operands and D may have any batch stride (the permuted views of
// the einsum expressions) and rows beyond M are clipped per batch.
//
// DG_AB_BF16: A and B are bfloat16 and there are no scales (the reference's sm100_bf16_gemm family): a stage row is still
// 128 bytes, now 64 elements of K; the MMA is tcgen05.mma.kind::f16 (16 elements of K per instruction); the scale loads,
// the rearranging warp's work and the scale columns of tensor memory disappear; MN-major atoms are 64 elements wide.
//
// DG_SPLIT_K (dense only, for shapes with too few output tiles to fill the GPU): every output tile becomes
// num_splits work items over slices of K, and the kernel's D is an FP32 workspace of num_splits stacked
// [rows x N] panels: work item (tile, slice) stores its partial tile into panel `slice`.  A separate kernel
// (dg_splitk.cu) then adds the panels in slice order, applies alpha and converts, so the result does not
// depend on which CTA finished first.
//
// DG_SPLIT_CLUSTER = S > 1 (dense only; the form of K slicing used whenever S <= 8 clusters fit the GPU): the S work
// items of an output tile are the CTAs of one thread-block cluster.  Each CTA runs the main loop over its slice of K;
// CTAs 1 .. S-1 then park their FP32 accumulator in their own shared memory (the pipeline stages are free by then),
// the cluster synchronises, and CTA 0 adds the parked tiles to its own accumulator in rank order, reading them through
// distributed shared memory, before the ordinary epilogue.  No workspace, no second kernel, and the same bits as the
// two-kernel form (both add the slices in slice order).
//
// MN-major operands (the nn / tn / tt variants): the tile is staged as [128 of K][128 B of MN] atoms with the
// same 128-byte swizzle (one TMA box per 128 columns of MN), the descriptor's leading-dimension offset steps
// between atoms, and a step of 32 along K is 32 rows = 4096 B.
//
// DG_M_HALVES == 2 gives one CTA a 256 x BLOCK_N tile: a stage holds 256 rows of A, and every K-block is multiplied
// as two 128-row MMAs that read the same B stage, so B leaves shared memory once per 256 rows and a K-block carries
// twice the tensor-core time per byte loaded (the ring of stages stops limiting long-K shapes).  The two halves'
// accumulators fill tensor memory, so a tile's MMAs start only after the epilogue has drained the previous tile.
// In the contiguous layout a 256-row tile whose halves belong to two experts runs over K twice, once per half with
// that half's B.
//
// DG_CLUSTER == 2 pairs two CTAs (a cluster of two SMs) on one 256 x BLOCK_N tile with
// tcgen05.mma.cta_group::2: each CTA loads its own 128 rows of A and one half of the B tile, CTA 0 issues
// the MMAs for both, each CTA keeps the accumulator of its own 128 rows in its tensor memory and runs its
// own epilogue.  B crosses L2 -> shared memory once per pair, and a stage is a third smaller, so the ring is deeper.
// Barriers that gather arrivals from both CTAs (full, tmem_empty) live in CTA 0; the peer reaches them
// through their shared::cluster addresses.
#pragma once

#include <cuda_bf16.h>

#include "gemm_config.hpp"
#include "ptx.cuh"
#include "quant_math.cuh"
#include "tile_scheduler.cuh"

namespace dg {

#ifndef DG_GEMM_TYPE
#error "DG_GEMM_TYPE and the other DG_* configuration macros must be defined by the code generator"
#endif

constexpr uint32_t kGemmType   = DG_GEMM_TYPE;
constexpr uint32_t BLOCK_M     = 128;
constexpr uint32_t BLOCK_N     = DG_BLOCK_N;
constexpr uint32_t BLOCK_K     = DG_BLOCK_K;       // bytes of K per row of a pipeline stage (64, 128 or 256)
constexpr bool     kABIsBF16   = DG_AB_BF16 != 0;
constexpr uint32_t kABElemBytes = kABIsBF16 ? 2 : 1;
#ifndef DG_MXF4
#define DG_MXF4 0
#endif
// FP4 x FP4 through tcgen05.mma.kind::mxf4 (the reference's kIsMXF4, impls/sm100_fp8_fp4_gemm_1d1d.cuh:51-54): the
// operands stay packed in shared memory (two E2M1 values per byte), so a 128-byte stage row is 256 elements of K, an MMA
// covers 64 of them, a stage carries two packed scale words per row (one scale per 32 elements), and the tensor cores run
// at twice the FP8 rate.  Without it FP4 operands are unpacked to one byte per element on the way into shared memory and
// multiplied by kind::mxf8f6f4.
constexpr bool     kMXF4       = DG_MXF4 != 0;
constexpr uint32_t BLOCK_K_ELEMS = BLOCK_K * (kMXF4 ? 2 : 1) / kABElemBytes;         // elements of K per pipeline stage
constexpr bool     kHasSF      = !kABIsBF16;                       // block-scaled operands
constexpr uint32_t kAtomElems  = 128 / kABElemBytes;               // MN-major staging: elements of MN per 128-byte atom row
constexpr uint32_t kNumStages  = DG_NUM_STAGES;
constexpr uint32_t kCluster    = DG_CLUSTER;       // CTAs cooperating on one tile (1 or 2)
constexpr bool     kAIsFP4     = DG_A_FP4 != 0;
constexpr bool     kBIsFP4     = DG_B_FP4 != 0;
constexpr bool     kAMnMajor   = DG_MAJOR_A != 0;
constexpr bool     kBMnMajor   = DG_MAJOR_B != 0;
constexpr uint32_t kGranKA     = DG_GRAN_K_A;
constexpr uint32_t kGranKB     = DG_GRAN_K_B;
constexpr bool     kDIsFP32    = DG_D_FP32 != 0;
constexpr bool     kDIsFP8     = DG_D_FP8 != 0;
constexpr bool     kStochastic = DG_STOCHASTIC_ROUNDING != 0;      // BF16 output rounded stochastically (quant_math.cuh)
constexpr bool     kAccumulate = DG_ACCUMULATE != 0;
constexpr uint32_t kRasterGroup = DG_RASTER_GROUP;
constexpr bool     kSplitK     = DG_SPLIT_K != 0;
#ifndef DG_TRANSPOSED_D
#define DG_TRANSPOSED_D 0
#endif
// The caller's operands are passed swapped (its B, the weight, as the 128-row operand; its few rows of A as the tile's
// columns): the tile is the transpose of the caller's D, and the epilogue writes element (row, column) to D[column][row].
// For GEMMs with few rows a CTA then pulls M x 128 bytes of activations per K-block next to its 128 rows of weights,
// instead of 128 rows of (mostly padding) activations next to a narrow slice of the weights.
constexpr bool kTransposedD = DG_TRANSPOSED_D != 0;
#ifndef DG_BATCH_REDUCE
#define DG_BATCH_REDUCE 0
#endif
// Dense GEMM that also sums over batches: K-block t of the work item is K-block (t mod kb_per_batch) of batch
// (t / kb_per_batch), the batch being the third coordinate of A's and B's tensor maps (D has none)
constexpr bool kBatchReduce = DG_BATCH_REDUCE != 0;
constexpr uint32_t kSplitCluster = DG_SPLIT_CLUSTER;   // CTAs of a cluster sharing one output tile along K (1 = off)

constexpr uint32_t kMHalves    = DG_M_HALVES;      // 128-row MMAs per CTA and K-block (1 or 2)
constexpr uint32_t kL2Hint     = DG_L2_HINT;

constexpr uint32_t UMMA_M = 128 * kCluster, UMMA_N = BLOCK_N, UMMA_K = 32;
constexpr uint32_t LOAD_BLOCK_N = BLOCK_N / kCluster;      // rows of B each CTA loads
constexpr uint32_t CTA_M = BLOCK_M * kMHalves;             // rows of A (and D) per CTA
constexpr uint32_t TILE_M = CTA_M * kCluster;              // rows of D per scheduled tile
// Four role warps and one epilogue warpgroup per 128 rows of the CTA's tile
constexpr uint32_t kNumThreads = 128 + 128 * kMHalves, kNumEpilogueThreads = 128, kEpilogueWarpBase = 4;
// Tensor memory holds two accumulators: two tiles in flight, or the two halves of one
constexpr uint32_t kNumAccumStages = kMHalves == 1 ? 2 : 1;

static_assert(BLOCK_N % 16 == 0 && BLOCK_N >= 16 && BLOCK_N <= (kHasSF ? 240 : 256), "UMMA_N must be a multiple of 16 that leaves room for the scales");
static_assert(!kABIsBF16 || (!kAIsFP4 && !kBIsFP4 && BLOCK_K == 128), "BF16 operands: 128-byte stages");
static_assert(kGranKA == 32 || kGranKA == 128, "one scale per 32 or 128 elements of K");
static_assert(kGranKB == 32 || kGranKB == 128, "one scale per 32 or 128 elements of K");
static_assert(kNumStages >= 2 && kNumStages <= 32, "pipeline depth");
static_assert(BLOCK_K == 128 || BLOCK_K == 256 || (BLOCK_K == 64 && !kAIsFP4 && !kBIsFP4 && !kAMnMajor && !kBMnMajor && !kSplitK),
              "64-element stages are built for K-major FP8 operands and unsliced K");
// A 256-byte stage is two 128-byte swizzle atoms side by side, [atom of K][row][128 bytes]: two copies per operand on one
// barrier and eight MMAs per wait.  Narrow tiles are bound by the MMA warp's walk around its loop (barrier poll, fence,
// commit, re-convergence), not by the MMAs or the loads, and this halves the walks per byte of K.
static_assert(BLOCK_K != 256 || (DG_GEMM_TYPE == 0 && !DG_AB_BF16 && !DG_A_FP4 && !DG_B_FP4 && !DG_MAJOR_A && !DG_MAJOR_B && DG_GRAN_K_A == 128 &&
                                 DG_GRAN_K_B == 128 && DG_CLUSTER == 1 && DG_M_HALVES == 1),
              "256-element stages are built for the dense GEMM of K-major FP8 operands with one scale per 128 elements, one 128-row CTA per tile");
constexpr uint32_t kKAtoms = BLOCK_K > 128 ? BLOCK_K / 128 : 1;      // 128-byte swizzle atoms along K per K-major stage row
constexpr uint32_t kKAtomBytes = BLOCK_K / kKAtoms;                  // width of one (the swizzle span): 64 or 128
static_assert(kCluster == 1 || kCluster == 2, "one CTA or a CTA pair per tile");
static_assert(kMHalves == 1 || kMHalves == 2, "128 or 256 rows per CTA");
static_assert(!(kAIsFP4 && kAMnMajor), "a packed FP4 A must be K-major");
static_assert(!(kBIsFP4 && kBMnMajor) || (!kAIsFP4 && BLOCK_N % 128 == 0 && kCluster == 1),
              "an MN-major packed FP4 B: FP8 x FP4 only; a load of the packed 4-bit type starts on a multiple of 128 elements");
static_assert(!kBMnMajor || (BLOCK_N / kCluster) % 16 == 0, "an MN-major B load must start on a 16-byte boundary");
static_assert(!kSplitK || (kGemmType == 0 && kDIsFP32 && !kAccumulate && kMHalves == 1), "split-K serves the plain dense GEMM and writes FP32 partials");
static_assert(kGemmType != kKGrouped || (BLOCK_K == 128 && kCluster == 1 && kGranKA == kGranKB), "k-grouped: one CTA per tile, 128-element stages, one scale granularity");
static_assert(!kMXF4 || (DG_A_FP4 && DG_B_FP4 && !DG_MAJOR_A && !DG_MAJOR_B && kGranKA == 32 && kGranKB == 32 && BLOCK_K == 128 &&
                         kGemmType != kKGrouped && kGemmType != kBatched && !DG_BATCH_REDUCE),
              "kind::mxf4: K-major packed FP4 on both sides, one scale per 32 elements of K");

// Scales: a packed int32 holds 4 scales, so it spans 4 * gran_k elements of K and is fetched on every
// (4 * gran_k / BLOCK_K)-th K-block: every 4th (8th with 64-element stages) at one scale per 128 K, every (2nd) one
// at one per 32 K.
// (a kind::mxf4 stage holds 256 elements of K: two words per row and K-block, fetched on every K-block)
constexpr uint32_t kSFAPeriod = 4 * kGranKA / BLOCK_K_ELEMS ? 4 * kGranKA / BLOCK_K_ELEMS : 1;
constexpr uint32_t kSFBPeriod = 4 * kGranKB / BLOCK_K_ELEMS ? 4 * kGranKB / BLOCK_K_ELEMS : 1;
constexpr uint32_t SF_BLOCK_M = CTA_M;
constexpr uint32_t SF_BLOCK_N = (BLOCK_N + 127) / 128 * 128;

// Shared memory and tensor memory maps (every operand stage starts on a 1024-byte boundary, as the
// 128-byte swizzle requires); the arithmetic lives in gemm_config.hpp, shared with the host heuristics
constexpr uint32_t kDElemBytes = kDIsFP32 ? 4 : (kDIsFP8 ? 1 : 2);
static_assert(!(kDIsFP32 && kDIsFP8), "one output type");
static_assert(!kStochastic || (!kDIsFP32 && !kDIsFP8 && !kAccumulate), "stochastic rounding writes BF16 directly");
static_assert(!kDIsFP8 || ((kGemmType == kDense || kGemmType == kBatched) && !kAccumulate && !kSplitK && BLOCK_N % 32 == 0),
              "the quantising epilogue serves the dense and batched GEMMs with tiles of whole 32-column scale groups");
static_assert(kGemmType != kBatched || (kCluster == 1 && !kSplitK), "batched: one CTA per tile");
static_assert(!kBatchReduce || (kGemmType == kDense && kABIsBF16 && !kAMnMajor && !kBMnMajor && kCluster == 1),
              "the batch-reduced GEMM takes K-major BF16 operands, one CTA per tile");
static_assert(!kTransposedD || (kGemmType == kDense && (kCluster == 1 || kSplitCluster == 1) && kMHalves == 1 && !kAccumulate && !kDIsFP8 && !kStochastic && !kSplitK),
              "the transposed epilogue serves the plain dense GEMM");
static_assert(kSplitCluster >= 1 && kSplitCluster <= 8, "portable cluster sizes");
static_assert(kSplitCluster == 1 || (kGemmType == kDense && !kSplitK && kCluster == 1 && kMHalves == 1 && !kAccumulate && !kDIsFP8 && !kStochastic),
              "cluster-reduced K slicing serves the plain dense GEMM");
#ifndef DG_STORE_BUFFERS
#define DG_STORE_BUFFERS 2
#endif
// The producer's and the MMA issuer's loops are walked by their whole warp (every lane polls the barriers, lane 0
// issues the copies / the tcgen05 instructions, the warp re-converges every K-block).  A lone lane inside a divergent
// branch ran the same loops measurably slower: 10 % of the kernel time with 128-row CTA pairs, 1-2 % with 256-row
// tiles.  0 restores the single-lane form (kept for comparison).
// L2 eviction hints on the operand loads (0 none; 1 keep A, stream B; 2 keep B, stream A)
#ifndef DG_L2_HINT
#define DG_L2_HINT 0
#endif
#ifndef DG_PRODUCER_WHOLE_WARP
#define DG_PRODUCER_WHOLE_WARP 1
#endif
#ifndef DG_MMA_WHOLE_WARP
#define DG_MMA_WHOLE_WARP 1
#endif
// Nanoseconds an epilogue warp sleeps between polls while it waits for its tile's accumulator (0 = poll continuously)
#ifndef DG_EPILOGUE_BACKOFF_NS
#define DG_EPILOGUE_BACKOFF_NS 0
#endif
#ifndef DG_A_ROWS
#define DG_A_ROWS 0
#endif
constexpr GemmLayout kLayout{CTA_M, BLOCK_N, BLOCK_K, kNumStages, kDElemBytes, kCluster, kBMnMajor ? 1u : 0u, kGranKA, kGranKB,
                             DG_SHORT_K, kABElemBytes, DG_STORE_BUFFERS, kMXF4 ? 1u : 0u, DG_A_ROWS};
static_assert(DG_A_ROWS == 0 || (DG_A_ROWS % 8 == 0 && DG_A_ROWS < 128 && kGemmType == kDense && kCluster == 1 && kMHalves == 1 && !kAMnMajor),
              "a shortened A stage: dense GEMMs with fewer rows than one tile, K-major A, one CTA per tile");
constexpr uint32_t kSFAWords = kHasSF ? kLayout.sfa_words() : 1, kSFBWords = kHasSF ? kLayout.sfb_words() : 1;   // packed words per row and stage
// K coordinate of a K-major load advances by this much per K-block: elements of the tensor map's type (bytes for the
// packed operands of kind::mxf4, whose maps are plain byte maps)
constexpr uint32_t kLoadXPerKBlock = kMXF4 ? BLOCK_K : BLOCK_K_ELEMS;
constexpr uint32_t kNumSFABuffers = kHasSF ? kLayout.sfa_buffers() : 1, kNumSFBBuffers = kHasSF ? kLayout.sfb_buffers() : 1;
static_assert(kSFAPeriod >= 1 && kSFBPeriod >= 1 && kSFAPeriod == kLayout.sfa_period() && kSFBPeriod == kLayout.sfb_period(), "scale fetch period");
constexpr uint32_t kBAtoms = kLayout.b_atoms();            // 128-column atoms of an MN-major B tile
constexpr uint32_t kStoreRowBytes   = kLayout.store_row_bytes();     // row width of the boxes covering the ragged end of a tile row
constexpr uint32_t kStoreCols       = kLayout.store_cols();          // columns of D per such box
constexpr uint32_t kNumStores       = kLayout.num_stores();
constexpr uint32_t kGroupCols       = kLayout.group_cols();          // columns of D drained per epilogue synchronisation
constexpr uint32_t kNumGroups       = kLayout.num_groups();
constexpr uint32_t kNumStoreStages  = kLayout.num_store_stages();
constexpr uint32_t kStoreStageBytes = kLayout.store_stage_bytes();
constexpr uint32_t kSmemD   = kLayout.off_d();
constexpr uint32_t kSmemA   = kLayout.off_a();
// Cluster-reduced K slicing: columns of the tile a CTA owns (whole 8-column chunks, dealt round robin), and the bytes it
// receives for them from the S slices.  The receive area starts where the D staging buffers do.
constexpr uint32_t kRecvCols = (BLOCK_N / 8 + kSplitCluster - 1) / kSplitCluster * 8;
constexpr uint32_t kRecvBytes = kSplitCluster * kRecvCols * 128 * 4;
constexpr bool kRecvOverStages = kRecvBytes > kSmemA;
// Transposed output: rows of D (columns of the tile) staged per TMA store, as many as the D staging buffers hold
constexpr uint32_t kTransposedRows = BLOCK_N * 128 * kDElemBytes <= kSmemA ? BLOCK_N : (kSmemA / (128 * kDElemBytes)) / 16 * 16;
constexpr uint32_t kABytes  = kLayout.a_bytes();
constexpr uint32_t kBBytes  = kLayout.b_bytes();
constexpr uint32_t kSmemB   = kLayout.off_b();
constexpr uint32_t kSFABytes = kLayout.sfa_bytes();
constexpr uint32_t kSFBBytes = kLayout.sfb_bytes();
constexpr uint32_t kSmemSFA = kLayout.off_sfa();
constexpr uint32_t kSmemSFB = kLayout.off_sfb();
constexpr uint32_t kSmemBar = kLayout.off_barriers();   // full, sf_full, empty per stage; tmem_full, tmem_empty per accumulator
constexpr uint32_t kSmemMisc = kLayout.off_misc();      // tensor-memory base address, abort flag
constexpr uint32_t kSmemTotal = kLayout.total_bytes();
static_assert(kABytes % (8 * BLOCK_K) == 0 && kBBytes % (8 * BLOCK_K) == 0, "every stage starts on a swizzle-pattern boundary (eight rows)");
// Bytes between the K atoms of a stage: the rows the stage holds, 128 bytes each
constexpr uint32_t kAAtomStride = kABytes / kKAtoms, kBAtomStride = kBBytes / kKAtoms;
static_assert(kKAtoms == 1 || (kAAtomStride % 1024 == 0 && kBAtomStride % 1024 == 0), "every K atom starts on a swizzle-pattern boundary");
static_assert(kSmemTotal <= kSmemCapacity, "shared memory budget exceeded");
static_assert(kStoreCols % 16 == 0 || kDIsFP32, "a store covers whole 16-column tensor-memory loads");

// Bytes the TMA engine reports per stage, summed over the CTAs of the cluster (packed FP4 counts its
// global-memory bytes)
constexpr uint32_t kTxBytesAB = kCluster * (kABytes / (kAIsFP4 && !kMXF4 ? 2 : 1) + kBBytes / (kBIsFP4 && !kMXF4 ? 2 : 1));

constexpr uint32_t kTmemColSFA = kLayout.tmem_col_sfa();
constexpr uint32_t kTmemColSFB = kLayout.tmem_col_sfb();
constexpr uint32_t kTmemCols = kLayout.tmem_cols_alloc();
static_assert(kLayout.tmem_cols_used() <= kTmemCapacityCols, "tensor memory budget exceeded");

enum Role : uint32_t { kRoleProducer = 1, kRoleMma = 2, kRoleSF = 3, kRoleEpilogue = 4 };

struct GemmParams {
    const int* grouped_layout;   // contiguous: expert id per row (-1 = padding); masked: rows used per group
    void* d;                     // D base pointer (for the direct-store path of ragged masked tiles)
    int* status;                 // host-visible status word, 0 = ok
    uint32_t shape_m;            // dense / contiguous: rows of A;  masked: max_m (rows per group)
    uint32_t shape_n;
    uint32_t shape_k;
    uint32_t num_groups;
    uint32_t ldd;                // row pitch of D in elements
    float alpha;
    unsigned long long* profile; // optional cycle counters (kernels built with DG_PROFILE only), else null
    uint32_t num_splits;         // slices of K per output tile (1 = no split)
    uint32_t kb_per_split;       // K-blocks per slice, a multiple of 512 elements so every slice starts on a packed scale word
    uint32_t split_panel_rows;   // split-K: rows between consecutive slices' panels in the workspace D points to
    uint32_t group_alignment;    // prefix-sum layout: every group starts on a multiple of this many rows
    uint32_t* sfd;               // quantising epilogue: packed UE8M0 scales of D, word (row, column / 128) at sfd[(column / 128) * sfd_pitch + row]
    uint32_t sfd_pitch;
    uint32_t kb_per_batch;       // batch-reduced GEMM: K-blocks in one batch
};

// Wait-time accounting for tuning: with DG_PROFILE defined every role adds the cycles it spent inside each
// of its waits, and in its whole loop, to profile[slot]; without it the calls compile to nothing.
enum ProfileSlot : uint32_t {
    kProfProducerWaitEmpty = 0, kProfProducerTotal = 1, kProfMmaWaitFull = 2, kProfMmaWaitTmemEmpty = 3, kProfMmaTotal = 4,
    kProfSFWait = 5, kProfSFTotal = 6, kProfEpiWaitTmemFull = 7, kProfEpiTotal = 8, kProfEpiStoreWait = 9,
    kProfMmaIssueCp = 10, kProfMmaIssueMma = 11, kProfMmaIssueCommit = 12, kProfMmaFence = 13, kProfMmaTail = 14, kProfNumSlots = 16
};
#if defined(DG_PROFILE) && DG_PROFILE
#define DG_PROF_VAR(name) long long name = 0
#define DG_PROF_BEGIN(var) const long long var = clock64()
#define DG_PROF_ADD(acc, var) acc += clock64() - var
#define DG_PROF_FLUSH(slot, acc) do { if (p.profile != nullptr) atomicAdd(p.profile + (slot), static_cast<unsigned long long>(acc)); } while (0)
// (the segments inside the MMA warp's K loop cost ten clock reads per K-block, enough to make that warp the bottleneck
//  of small tiles: DG_PROFILE=2 leaves them out and keeps the waits and totals)
#if DG_PROFILE == 1
#define DG_PROF_FINE_BEGIN(var) const long long var = clock64()
#define DG_PROF_FINE_ADD(acc, var) acc += clock64() - var
#else
#define DG_PROF_FINE_BEGIN(var) do { } while (0)
#define DG_PROF_FINE_ADD(acc, var) do { } while (0)
#endif
// Timeline of CTA 0 in nanoseconds (globaltimer): slots 16.. hold absolute stamps, first writer wins
#define DG_PROF_STAMP(slot) do { if (p.profile != nullptr && blockIdx.x == 0) atomicCAS(p.profile + 16 + (slot), 0ull, global_timer_ns()); } while (0)
// over all CTAs: the earliest / latest time an event happened anywhere in the grid
#define DG_PROF_STAMP_MIN(slot) do { if (p.profile != nullptr) atomicMin(p.profile + 16 + (slot), global_timer_ns()); } while (0)
#define DG_PROF_STAMP_MAX(slot) do { if (p.profile != nullptr) atomicMax(p.profile + 16 + (slot), global_timer_ns()); } while (0)
#else
#define DG_PROF_STAMP(slot) do { } while (0)
#define DG_PROF_STAMP_MIN(slot) do { } while (0)
#define DG_PROF_STAMP_MAX(slot) do { } while (0)
#define DG_PROF_VAR(name) do { } while (0)
#define DG_PROF_FINE_BEGIN(var) do { } while (0)
#define DG_PROF_FINE_ADD(acc, var) do { } while (0)
#define DG_PROF_BEGIN(var) do { } while (0)
#define DG_PROF_ADD(acc, var) do { } while (0)
#define DG_PROF_FLUSH(slot, acc) do { } while (0)
#endif

}  // namespace dg

extern "C" __global__ void __launch_bounds__(dg::kNumThreads, 1)
dg_gemm_fp8_fp4(const __grid_constant__ CUtensorMap tm_a,
                const __grid_constant__ CUtensorMap tm_b,
                const __grid_constant__ CUtensorMap tm_sfa,
                const __grid_constant__ CUtensorMap tm_sfb,
                const __grid_constant__ CUtensorMap tm_d,
                const __grid_constant__ CUtensorMap tm_d_full,       // D again, with 128-byte-wide store boxes
                const dg::GemmParams p) {
    using namespace dg;
    extern __shared__ __align__(1024) uint8_t smem[];

    const uint32_t warp_idx = __shfl_sync(0xFFFFFFFFu, threadIdx.x / 32, 0);
    const uint32_t lane = lane_id();
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t cta_rank = kCluster == 1 ? 0u : cluster_ctarank();
    const bool is_leader = cta_rank == 0;
    const uint32_t split_rank = kSplitCluster == 1 ? 0u : cluster_ctarank();      // which slice of K this CTA computes

    auto full_bar     = [&](uint32_t s) { return smem_base + kSmemBar + s * 8; };
    auto sf_full_bar  = [&](uint32_t s) { return smem_base + kSmemBar + (kNumStages + s) * 8; };
    auto empty_bar    = [&](uint32_t s) { return smem_base + kSmemBar + (2 * kNumStages + s) * 8; };
    auto tmem_full_bar  = [&](uint32_t a) { return smem_base + kSmemBar + (3 * kNumStages + a) * 8; };
    auto tmem_empty_bar = [&](uint32_t a) { return smem_base + kSmemBar + (3 * kNumStages + 2 + a) * 8; };
    // shared::cluster address of a barrier of CTA 0 (the local address when there is no cluster)
    auto in_leader = [&](uint32_t bar) { return kCluster == 1 ? bar : map_to_cta(bar, 0); };
    volatile uint32_t* tmem_base_slot = reinterpret_cast<volatile uint32_t*>(smem + kSmemMisc);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + kSmemMisc + 4);
    const AbortCtx ctx{abort_flag, p.status};

    // ---- set-up -------------------------------------------------------------------------------
    if (threadIdx.x == 0) {
        DG_PROF_STAMP(0);                                   // kernel entry
        DG_PROF_STAMP_MIN(9);                               // first CTA to enter
        DG_PROF_STAMP_MAX(10);                              // last CTA to enter
        *abort_flag = 0;
        prefetch_tensormap(&tm_a);
        prefetch_tensormap(&tm_b);
        prefetch_tensormap(&tm_sfa);
        prefetch_tensormap(&tm_sfb);
        prefetch_tensormap(&tm_d);
        prefetch_tensormap(&tm_d_full);
    }
    if (warp_idx == 1 && lane == 0) {
        for (uint32_t s = 0; s < kNumStages; ++s) {
            // per CTA of the cluster: the producer's arrive + one arrive of the scale warp (used in CTA 0 only)
            mbar_init(full_bar(s), kCluster * (1 + (kHasSF ? 1 : 0)));
            mbar_init(sf_full_bar(s), 1);
            mbar_init(empty_bar(s), 1);          // tcgen05.commit
        }
        for (uint32_t a = 0; a < 2; ++a) {       // one pair per accumulator: two tiles in flight, or the halves of one
            mbar_init(tmem_full_bar(a), 1);      // tcgen05.commit
            mbar_init(tmem_empty_bar(a), kCluster * kNumEpilogueThreads);   // used in CTA 0 only
        }
        fence_mbar_init();
    }
    __syncwarp();
    if constexpr (kCluster > 1) {
        // Both CTAs must be resident before the paired tensor-memory allocation
        cluster_arrive_relaxed();
        cluster_wait();
    }
    if (warp_idx == 2) {
        tmem_alloc<kCluster>(smem_u32(const_cast<uint32_t*>(tmem_base_slot)), kTmemCols);
        tmem_relinquish<kCluster>();
    }
    tc_fence_before_sync();
    if constexpr (kCluster > 1) {
        // Barriers of both CTAs are initialised before either CTA signals the other
        cluster_arrive();
        cluster_wait();
    } else {
        __syncthreads();
    }
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_base_slot;
    // Cluster-reduced K slicing whose receive area lies outside the pipeline stages: peers may write to this CTA as soon
    // as it runs, which the first half of a split barrier announces here (the epilogue waits for it before sending)
    if constexpr (kSplitCluster > 1 && !kRecvOverStages) cluster_arrive_relaxed();
    if (threadIdx.x == 0) DG_PROF_STAMP(1);                 // set-up done (barriers, tensor memory)
    // Everything above touched no global memory, so with programmatic dependent launch it overlapped the tail of the
    // kernel before this one; from here on its results (and its reads of D) must be complete.  The kernel after
    // this one may begin its own set-up as soon as SMs free up.
    griddep_wait();
    griddep_launch_dependents();

    const uint32_t num_k_blocks = (p.shape_k + BLOCK_K_ELEMS - 1) / BLOCK_K_ELEMS;
    const uint32_t sfa_rows_per_group = (p.shape_k + kGranKA * 4 - 1) / (kGranKA * 4);   // packed K extent of SFA
    const uint32_t sfb_rows_per_group = (p.shape_k + kGranKB * 4 - 1) / (kGranKB * 4);

    // A cluster walks the tile list as one unit
    // (cluster-reduced slicing: a cluster has exactly one tile, so the stride past it ends every role's loop)
    TileScheduler<kGemmType> sched(TILE_M, BLOCK_N, kRasterGroup, p.shape_m, p.shape_n, p.num_groups, p.grouped_layout,
                                   blockIdx.x / (kCluster * kSplitCluster),
                                   kSplitCluster > 1 ? 0x40000000u : gridDim.x / kCluster, kSplitK ? p.num_splits : 1u);
    if constexpr (kGemmType == kMGroupedPsum) {
        sched.group_alignment = p.group_alignment;
        sched.write_padding = DG_WRITE_PADDING;
    }
    if constexpr (kGemmType == kKGrouped) {
        sched.group_alignment = p.group_alignment;
        sched.k_psum = DG_K_PSUM;
        sched.k_per_sf_row = 4 * kGranKA;
        sched.k_per_block = BLOCK_K_ELEMS;
    }
    // K-blocks [kb_begin, kb_end) of a work item: all of K unless the GEMM is split
    auto kb_begin = [&](const Tile& t) { return kSplitK ? t.split * p.kb_per_split : (kSplitCluster > 1 ? split_rank * p.kb_per_split : 0u); };
    auto kb_end = [&](const Tile& t) {
        if constexpr (kGemmType == kKGrouped) return t.num_kb;
        if constexpr (!kSplitK && kSplitCluster == 1) return num_k_blocks;
        const uint32_t e = ((kSplitK ? t.split : split_rank) + 1) * p.kb_per_split;
        return e < num_k_blocks ? e : num_k_blocks;
    };
    // A 256-row tile of the contiguous layout whose halves belong to different experts takes two passes over K:
    // pass h multiplies half h with B of its own expert
    auto num_passes_of = [&](const Tile& t) { return kGemmType == 1 && kMHalves == 2 && t.group1 != t.group ? 2u : 1u; };
    // Every role walks the same sequence of (pass, K-block) steps of a tile, one pipeline stage per step
    struct Step { uint32_t pass, kb; };
    auto step_of = [](uint32_t it, uint32_t kb0, uint32_t num_kb) {
        const uint32_t pass = it >= num_kb ? 1u : 0u;
        return Step{pass, kb0 + it - pass * num_kb};
    };
    // Scale words land in a ring of buffers, one per fetch (see GemmLayout::sf_buffers); every role counts the fetches
    uint32_t sfa_slot = 0, sfb_slot = 0;
    auto sfa_buffer = [&]() { return smem_base + kSmemSFA + sfa_slot * kSFABytes; };
    auto sfb_buffer = [&]() { return smem_base + kSmemSFB + sfb_slot * kSFBBytes; };
    auto advance_sf = [&](uint32_t kb) {
        if (kb % kSFAPeriod == 0) sfa_slot = sfa_slot + 1 == kNumSFABuffers ? 0 : sfa_slot + 1;
        if (kb % kSFBPeriod == 0) sfb_slot = sfb_slot + 1 == kNumSFBBuffers ? 0 : sfb_slot + 1;
    };
    // Tensor-map copies: two-dimensional, or with the batch as third coordinate
    auto tma_in = [&](uint32_t dst, const CUtensorMap* map, uint32_t bar, uint32_t x, uint32_t y, uint32_t batch) {
        if constexpr (kGemmType == kBatched) tma_load_3d(dst, map, bar, static_cast<int32_t>(x), static_cast<int32_t>(y), static_cast<int32_t>(batch));
        else tma_load_2d(dst, map, bar, static_cast<int32_t>(x), static_cast<int32_t>(y));
    };
    auto tma_out = [&](const CUtensorMap* map, uint32_t src, uint32_t x, uint32_t y, uint32_t batch) {
        if constexpr (kGemmType == kBatched) {
            if constexpr (kAccumulate) tma_reduce_add_3d(map, src, static_cast<int32_t>(x), static_cast<int32_t>(y), static_cast<int32_t>(batch));
            else tma_store_3d(map, src, static_cast<int32_t>(x), static_cast<int32_t>(y), static_cast<int32_t>(batch));
        } else {
            if constexpr (kAccumulate) tma_reduce_add_2d(map, src, static_cast<int32_t>(x), static_cast<int32_t>(y));
            else tma_store_2d(map, src, static_cast<int32_t>(x), static_cast<int32_t>(y));
        }
    };
    Tile tile;
    uint32_t stage = 0, phase = 0;
    auto advance_stage = [&]() {
        stage = stage + 1 == kNumStages ? 0 : stage + 1;
        phase ^= (stage == 0);
    };

    // With 256-row tiles the CTA has three warpgroups and the launch gives every thread 168 registers.  The epilogue
    // warpgroups keep whole accumulator rows in registers and the role warps need few, so the latter hand registers
    // over (role + 2 x epilogue = 3 x 168; the contiguous layout's producer tracks two experts per tile and needs more).
    constexpr uint32_t kRoleRegs = kGemmType == 1 ? 88 : 72, kEpilogueRegs = (3 * 168 - kRoleRegs) / 2;
    static_assert(kEpilogueRegs % 8 == 0, "register counts move in units of 8");
    if (warp_idx < kEpilogueWarpBase) {
        if constexpr (kMHalves == 2) warpgroup_reg_dec<kRoleRegs>();
        if (warp_idx == 0) {
            // ================= TMA producer (every CTA loads its own rows of A and its share of B) =================
            // Either lane 0 alone walks the loop, or (DG_PRODUCER_WHOLE_WARP) the whole warp does and lane 0 issues the copies
            constexpr bool kProducerWholeWarp = DG_PRODUCER_WHOLE_WARP != 0;
            if (kProducerWholeWarp || lane == 0) {
                bool ok = true;
                [[maybe_unused]] const uint64_t policy_keep = kL2Hint ? l2_policy_evict_last() : 0, policy_stream = kL2Hint ? l2_policy_evict_first() : 0;
                DG_PROF_VAR(prof_wait);
                DG_PROF_BEGIN(prof_t0);
                while (ok && sched.next(tile)) {
                    // Row coordinates of this CTA's part of the tile in the 2-D views of A, B and the scale tensors
                    const uint32_t a_row = tile.a_row_base + tile.m_block * TILE_M + cta_rank * CTA_M;
                    const uint32_t sfa_mn = tile.sfa_mn_base + tile.m_block * TILE_M + cta_rank * CTA_M;
                    const uint32_t sfa_row0 = kGemmType == kKGrouped ? tile.sf_row_base : tile.sfa_group * sfa_rows_per_group;   // batched: 0
                    const uint32_t k_base = kGemmType == kKGrouped ? tile.k_base : 0u;      // first element of K of this work item
                    const uint32_t kb0 = kb_begin(tile), num_kb = kb_end(tile) - kb0, num_steps = num_passes_of(tile) * num_kb;
                    for (uint32_t it = 0; it < num_steps; ++it, advance_stage()) {
                        const auto [pass, kb] = step_of(it, kb0, num_kb);
                        const uint32_t b_group = pass == 0 ? tile.group : tile.group1;
                        // k-grouped: B is one [N, sum K] (or [sum K, N]) matrix and the group selects the slice of K
                        // (batched: the batch is a coordinate of its own)
                        constexpr bool kOneB = kGemmType == kKGrouped || kGemmType == kBatched;
                        const uint32_t b_row = (kOneB ? 0u : b_group * p.shape_n) + tile.n_block * BLOCK_N + cta_rank * LOAD_BLOCK_N;
                        const uint32_t sfb_row0 = kGemmType == kKGrouped ? tile.sf_row_base : (kOneB ? 0u : b_group * sfb_rows_per_group);
                        const uint32_t b_k_base = kGemmType == kKGrouped ? tile.k_base : (kOneB ? 0u : b_group * p.shape_k);   // MN-major B: row of K
                        DG_PROF_BEGIN(prof_w);
                        if (!mbar_wait(empty_bar(stage), phase ^ 1, ctx, kRoleProducer, 1)) { ok = false; break; }
                        DG_PROF_ADD(prof_wait, prof_w);
                        if constexpr (kProducerWholeWarp) __syncwarp();
                        if (kProducerWholeWarp && lane != 0) { advance_sf(kb); continue; }
                        if constexpr (kHasSF) {
                            uint32_t sf_bytes = 0;
                            if (kb % kSFAPeriod == 0) sf_bytes += kSFABytes;
                            if (kb % kSFBPeriod == 0) sf_bytes += kSFBBytes;
                            mbar_arrive_expect_tx(sf_full_bar(stage), sf_bytes);
                            if (kb % kSFAPeriod == 0)
                                tma_in(sfa_buffer(), &tm_sfa, sf_full_bar(stage), sfa_mn, sfa_row0 + kb / kSFAPeriod * kSFAWords, tile.group);
                            if (kb % kSFBPeriod == 0)
                                tma_in(sfb_buffer(), &tm_sfb, sf_full_bar(stage), tile.n_block * BLOCK_N, sfb_row0 + kb / kSFBPeriod * kSFBWords, tile.group);
                        }
                        // With a cluster the copies land in this CTA and their bytes are counted on CTA 0's barrier,
                        // which expects both CTAs' bytes
                        const uint32_t load_bar = kCluster == 1 ? full_bar(stage) : in_leader(full_bar(stage));
                        if (kCluster == 1 || is_leader) mbar_arrive_expect_tx(full_bar(stage), kTxBytesAB);
                        else mbar_arrive_cluster(load_bar);
                        auto load = [&](uint32_t dst, const CUtensorMap* map, uint32_t x, uint32_t y) {
                            if constexpr (kL2Hint != 0 && kGemmType != kBatched) {
                                // DG_L2_HINT 1: A stays (evict_last), B streams (evict_first); 2: the other way round
                                const uint64_t policy = ((map == &tm_a) == (kL2Hint == 1)) ? policy_keep : policy_stream;
                                if constexpr (kCluster == 1) tma_load_2d_hint(dst, map, load_bar, static_cast<int32_t>(x), static_cast<int32_t>(y), policy);
                                else tma_load_2d_2cta_hint(dst, map, load_bar, static_cast<int32_t>(x), static_cast<int32_t>(y), policy);
                            } else if constexpr (kCluster == 1) {
                                tma_in(dst, map, load_bar, x, y, tile.group);
                            } else {
                                tma_load_2d_2cta(dst, map, load_bar, static_cast<int32_t>(x), static_cast<int32_t>(y));
                            }
                        };
                        // K-major: x = K, y = row.  MN-major: x = row (column of the stored matrix), y = K (+ the group's K offset)
                        if constexpr (kBatchReduce) {
                            const uint32_t batch = kb / p.kb_per_batch, kx = (kb - batch * p.kb_per_batch) * BLOCK_K_ELEMS;
                            tma_load_3d(smem_base + kSmemA + stage * kABytes, &tm_a, load_bar, static_cast<int32_t>(kx),
                                        static_cast<int32_t>(a_row), static_cast<int32_t>(batch));
                            tma_load_3d(smem_base + kSmemB + stage * kBBytes, &tm_b, load_bar, static_cast<int32_t>(kx),
                                        static_cast<int32_t>(b_row), static_cast<int32_t>(batch));
                            advance_sf(kb);
                            continue;
                        }
                        if constexpr (!kAMnMajor) {
                            #pragma unroll
                            for (uint32_t ka = 0; ka < kKAtoms; ++ka)       // one box of the stage's rows per 128 bytes of K
                                load(smem_base + kSmemA + stage * kABytes + ka * kAAtomStride, &tm_a, k_base + kb * kLoadXPerKBlock + ka * 128, a_row);
                        } else {
                            // one box per atom: 128 bytes of M (128 FP8 or 64 BF16 elements) by the stage's rows of K
                            #pragma unroll
                            for (uint32_t i = 0; i < CTA_M / kAtomElems; ++i)
                                load(smem_base + kSmemA + stage * kABytes + i * 128 * BLOCK_K_ELEMS, &tm_a, a_row + i * kAtomElems,
                                     k_base + kb * BLOCK_K_ELEMS);
                        }
                        if constexpr (!kBMnMajor) {
                            #pragma unroll
                            for (uint32_t ka = 0; ka < kKAtoms; ++ka)
                                load(smem_base + kSmemB + stage * kBBytes + ka * kBAtomStride, &tm_b, k_base + kb * kLoadXPerKBlock + ka * 128, b_row);
                        } else {
                            #pragma unroll
                            for (uint32_t i = 0; i < kBAtoms; ++i)
                                load(smem_base + kSmemB + stage * kBBytes + i * 128 * BLOCK_K_ELEMS, &tm_b,
                                     tile.n_block * BLOCK_N + cta_rank * LOAD_BLOCK_N + i * kAtomElems, b_k_base + kb * BLOCK_K_ELEMS);
                        }
                        advance_sf(kb);
                    }
                }
                DG_PROF_VAR(prof_total);
                DG_PROF_ADD(prof_total, prof_t0);
                if (lane == 0) {
                    DG_PROF_FLUSH(kProfProducerWaitEmpty, prof_wait);
                    DG_PROF_FLUSH(kProfProducerTotal, prof_total);
                }
            }
        } else if (warp_idx == 1) {
            // ================= MMA issuer (CTA 0 of the cluster only) =================
            // Either lane 0 alone walks the loop, or (DG_MMA_WHOLE_WARP) the whole warp does and lane 0 issues
            constexpr bool kWholeWarp = DG_MMA_WHOLE_WARP != 0;
            const bool issue_lane = lane == 0;
            if ((kWholeWarp || lane == 0) && is_leader) {
                constexpr uint32_t idesc = kABIsBF16 ? make_instr_desc_bf16(kAMnMajor, kBMnMajor, UMMA_M, UMMA_N)
                                           : kMXF4 ? make_instr_desc_block_scaled(kFmtMxf4E2M1, kFmtMxf4E2M1, 0, 0, UMMA_M, UMMA_N)
                                                     : make_instr_desc_block_scaled(kAIsFP4 ? kFmtE2M1 : kFmtE4M3, kBIsFP4 ? kFmtE2M1 : kFmtE4M3,
                                                                                    kAMnMajor, kBMnMajor, UMMA_M, UMMA_N);
                // K-major: 8-row groups of BLOCK_K-byte rows (SBO 1024 or 512, swizzle span = the row), +32 B per UMMA along K.
                // MN-major: atoms of [128 K][128 B]; SBO 1024 = eight K rows, LBO = one atom, +32 rows (4096 B) per UMMA along K.
                constexpr uint32_t kALbo = kAMnMajor ? 128 * BLOCK_K_ELEMS : 0, kBLbo = kBMnMajor ? 128 * BLOCK_K_ELEMS : 0;
                constexpr uint32_t kASbo = kAMnMajor ? 1024 : 8 * kKAtomBytes, kBSbo = kBMnMajor ? 1024 : 8 * kKAtomBytes;
                constexpr uint64_t kASwizzle = kAMnMajor || kKAtomBytes == 128 ? kSwizzle128B : kSwizzle64B;
                constexpr uint64_t kBSwizzle = kBMnMajor || kKAtomBytes == 128 ? kSwizzle128B : kSwizzle64B;
                // (UMMA_K is 32 bytes of K: 32 FP8 or 16 BF16 elements, i.e. that many rows of an MN-major atom)
                constexpr uint32_t kAStepK = (kAMnMajor ? UMMA_K / kABElemBytes * 128 : UMMA_K) >> 4;
                constexpr uint32_t kBStepK = (kBMnMajor ? UMMA_K / kABElemBytes * 128 : UMMA_K) >> 4;
                // (256-byte stages: MMA j works on atom j / 4 of the stage, 32 (j mod 4) bytes into its rows)
                constexpr uint32_t kMmasPerAtom = kKAtomBytes / UMMA_K;
                auto a_step = [&](uint32_t j) { return kKAtoms == 1 ? j * kAStepK : (j / kMmasPerAtom) * (kAAtomStride >> 4) + (j % kMmasPerAtom) * kAStepK; };
                auto b_step = [&](uint32_t j) { return kKAtoms == 1 ? j * kBStepK : (j / kMmasPerAtom) * (kBAtomStride >> 4) + (j % kMmasPerAtom) * kBStepK; };
                // A commit reaches the barrier at the same offset in every CTA of the cluster
                auto commit_all = [&](uint32_t bar) {
                    if constexpr (kCluster == 1) {
                        tc_commit(bar);
                    } else {
                        tc_commit_2cta_mask(bar, 0x3);          // both CTAs' barriers with one instruction
                    }
                };
                bool ok = true;
                uint32_t tile_iter = 0;
                DG_PROF_VAR(prof_full); DG_PROF_VAR(prof_tmem); DG_PROF_VAR(prof_cp); DG_PROF_VAR(prof_mma); DG_PROF_VAR(prof_commit);
                DG_PROF_VAR(prof_fence); DG_PROF_VAR(prof_tail);
                DG_PROF_BEGIN(prof_t0);
                while (ok && sched.next(tile)) {
                    if (kGemmType == kKGrouped && tile.num_kb == 0) continue;      // an empty group: the epilogue writes zeros
                    // First accumulator (and barrier pair) of this tile: tiles alternate between the two, or the halves of a
                    // 256-row tile own one each
                    const uint32_t accum = tile_iter % kNumAccumStages, accum_phase = (tile_iter / kNumAccumStages) & 1;
                    ++tile_iter;
                    DG_PROF_BEGIN(prof_w0);
                    bool accum_free = true;
                    #pragma unroll
                    for (uint32_t h = 0; h < kMHalves; ++h)
                        accum_free = accum_free && mbar_wait(tmem_empty_bar(accum + h), accum_phase ^ 1, ctx, kRoleMma, 1);
                    if (!accum_free) { ok = false; break; }
                    DG_PROF_ADD(prof_tmem, prof_w0);
                    tc_fence_after_sync();
                    const uint32_t kb0 = kb_begin(tile), num_kb = kb_end(tile) - kb0;
                    const uint32_t num_passes = num_passes_of(tile), num_steps = num_passes * num_kb;
                    for (uint32_t it = 0; it < num_steps; ++it, advance_stage()) {
                        const auto [pass, kb] = step_of(it, kb0, num_kb);
                        DG_PROF_BEGIN(prof_w1);
                        if (!mbar_wait(full_bar(stage), phase, ctx, kRoleMma, 2)) { ok = false; break; }
                        DG_PROF_ADD(prof_full, prof_w1);
                        if (it == 0) DG_PROF_STAMP(2);          // first stage arrived
                        if (it == 0 && tile_iter == 1 && lane == 0) DG_PROF_STAMP_MAX(12);      // ... in the last CTA to see one
                        DG_PROF_FINE_BEGIN(prof_f0);
                        tc_fence_after_sync();
                        DG_PROF_FINE_ADD(prof_fence, prof_f0);
                        if (issue_lane) {
                        // Scales: shared memory (rearranged by warp 2) -> tensor memory, in every CTA of the cluster
                        DG_PROF_FINE_BEGIN(prof_i0);
                        if (kHasSF && kb % kSFAPeriod == 0) {
                            #pragma unroll
                            for (uint32_t i = 0; i < kSFAWords * SF_BLOCK_M / 128; ++i)      // chunk (word w, rows 128 r ..): index w * (rows / 128) + r
                                tc_cp_32x128b_warpx4<kCluster>(tmem_base + kTmemColSFA + i * 4,
                                                               make_smem_desc(sfa_buffer() + i * 512, 0, 128, kSwizzleNone));
                        }
                        if (kHasSF && kb % kSFBPeriod == 0) {
                            #pragma unroll
                            for (uint32_t i = 0; i < kSFBWords * SF_BLOCK_N / 128; ++i)
                                tc_cp_32x128b_warpx4<kCluster>(tmem_base + kTmemColSFB + i * 4,
                                                               make_smem_desc(sfb_buffer() + i * 512, 0, 128, kSwizzleNone));
                        }
                        DG_PROF_FINE_ADD(prof_cp, prof_i0);
                        DG_PROF_FINE_BEGIN(prof_i1);
                        const uint64_t a_desc = make_smem_desc(smem_base + kSmemA + stage * kABytes, kALbo, kASbo, kASwizzle);
                        const uint64_t b_desc = make_smem_desc(smem_base + kSmemB + stage * kBBytes, kBLbo, kBSbo, kBSwizzle);
                        #pragma unroll
                        for (uint32_t h = 0; h < kMHalves; ++h) {
                            // In a two-pass tile (halves of different experts) pass p carries half p's expert
                            if (num_passes == 2 && h != pass) continue;
                            // Half h: rows [128 h, 128 h + 128) of the A stage (128 * BLOCK_K bytes further, in either layout),
                            // its own accumulator and its own four columns of row scales
                            const uint32_t tmem_d = tmem_base + (accum + h) * UMMA_N;
                            #pragma unroll
                            for (uint32_t j = 0; j < BLOCK_K / UMMA_K; ++j) {
                                // Which byte of the packed scale word applies to these 32 elements of K
                                const uint32_t sfa_id = ((kb * BLOCK_K + j * UMMA_K) / kGranKA) % 4;
                                const uint32_t sfb_id = ((kb * BLOCK_K + j * UMMA_K) / kGranKB) % 4;
                                // Advancing K moves the start address: +32 B inside the swizzle atom (K-major) or +32 rows (MN-major)
                                if constexpr (kABIsBF16)
                                    tc_mma_bf16<kCluster>(tmem_d, a_desc + h * ((BLOCK_M * BLOCK_K) >> 4) + a_step(j), b_desc + b_step(j),
                                                          idesc, ((kb - kb0) | j) != 0);
                                else if constexpr (kMXF4)
                                    // 64 elements of K per instruction: word j / 2 of the stage, scale bytes 0-1 or 2-3 of it
                                    tc_mma_mxf4<kCluster>(tmem_d, a_desc + h * ((BLOCK_M * BLOCK_K) >> 4) + a_step(j), b_desc + b_step(j),
                                                          instr_desc_with_sf_ids(idesc, (j % 2) * 2, (j % 2) * 2),
                                                          tmem_base + kTmemColSFA + (j / 2) * (SF_BLOCK_M / 32) + h * 4,
                                                          tmem_base + kTmemColSFB + (j / 2) * (SF_BLOCK_N / 32), ((kb - kb0) | j) != 0);
                                else
                                    tc_mma_mxf8f6f4<kCluster>(tmem_d, a_desc + h * ((BLOCK_M * BLOCK_K) >> 4) + a_step(j), b_desc + b_step(j),
                                                              instr_desc_with_sf_ids(idesc, sfa_id, sfb_id),
                                                              tmem_base + kTmemColSFA + h * 4, tmem_base + kTmemColSFB, ((kb - kb0) | j) != 0);
                            }
                        }
                        DG_PROF_FINE_ADD(prof_mma, prof_i1);
                        DG_PROF_FINE_BEGIN(prof_i2);
                        commit_all(empty_bar(stage));                      // releases the stage once its MMAs have read it
                        if (it + 1 == num_steps) {                         // accumulator(s) complete
                            #pragma unroll
                            for (uint32_t h = 0; h < kMHalves; ++h) commit_all(tmem_full_bar(accum + h));
                        }
                        DG_PROF_FINE_ADD(prof_commit, prof_i2);
                        }
                        DG_PROF_FINE_BEGIN(prof_t1);
                        if constexpr (kWholeWarp) __syncwarp();
                        advance_sf(kb);
                        DG_PROF_FINE_ADD(prof_tail, prof_t1);
                    }
                }
                if (issue_lane) {
                DG_PROF_VAR(prof_total);
                DG_PROF_ADD(prof_total, prof_t0);
                DG_PROF_FLUSH(kProfMmaWaitFull, prof_full);
                DG_PROF_FLUSH(kProfMmaWaitTmemEmpty, prof_tmem);
                DG_PROF_FLUSH(kProfMmaTotal, prof_total);
                DG_PROF_FLUSH(kProfMmaIssueCp, prof_cp);
                DG_PROF_FLUSH(kProfMmaIssueMma, prof_mma);
                DG_PROF_FLUSH(kProfMmaIssueCommit, prof_commit);
                DG_PROF_FLUSH(kProfMmaFence, prof_fence);
                DG_PROF_FLUSH(kProfMmaTail, prof_tail);
                }
            }
        } else if (warp_idx == 2 && kHasSF) {
            // ================= scale rearrangement =================
            // tcgen05.cp reads 32 rows x 16 bytes and writes row r to lane r: the scale word of tile row
            // (c * 32 + r) has to sit at word (r * 4 + c).  TMA delivered the 128 words in row order.
            auto rearrange = [&](uint32_t chunk_addr) {
                uint32_t v[4];
                #pragma unroll
                for (uint32_t c = 0; c < 4; ++c)
                    v[c] = ld_shared_u32(chunk_addr + (c * 32 + lane) * 4);
                __syncwarp();
                st_shared_v4(chunk_addr + lane * 16, v[0], v[1], v[2], v[3]);
            };
            bool ok = true;
            DG_PROF_VAR(prof_wait);
            DG_PROF_BEGIN(prof_t0);
            while (ok && sched.next(tile)) {
                const uint32_t kb0 = kb_begin(tile), num_kb = kb_end(tile) - kb0, num_steps = num_passes_of(tile) * num_kb;
                for (uint32_t it = 0; it < num_steps; ++it, advance_stage()) {
                    const uint32_t kb = step_of(it, kb0, num_kb).kb;
                    DG_PROF_BEGIN(prof_w);
                    if (!mbar_wait(sf_full_bar(stage), phase, ctx, kRoleSF, 1)) { ok = false; break; }
                    DG_PROF_ADD(prof_wait, prof_w);
                    if (kb % kSFAPeriod == 0) {
                        #pragma unroll
                        for (uint32_t i = 0; i < kSFAWords * SF_BLOCK_M / 128; ++i)
                            rearrange(sfa_buffer() + i * 512);
                    }
                    if (kb % kSFBPeriod == 0) {
                        #pragma unroll
                        for (uint32_t i = 0; i < kSFBWords * SF_BLOCK_N / 128; ++i)
                            rearrange(sfb_buffer() + i * 512);
                    }
                    // every lane makes its own writes visible to the async proxy; then one lane signals for the warp
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        if (kCluster == 1 || is_leader) mbar_arrive(full_bar(stage));
                        else mbar_arrive_cluster(in_leader(full_bar(stage)));
                    }
                    advance_sf(kb);
                }
            }
            if (lane == 0) {
                DG_PROF_VAR(prof_total);
                DG_PROF_ADD(prof_total, prof_t0);
                DG_PROF_FLUSH(kProfSFWait, prof_wait);
                DG_PROF_FLUSH(kProfSFTotal, prof_total);
            }
        }
        if constexpr (kSplitCluster > 1) {
            // The role warps have nothing to publish: they only take part in the two cluster-wide barriers of the
            // epilogue ("every CTA may be written to", "every slice has arrived")
            __syncwarp();
            if constexpr (kRecvOverStages) cluster_arrive();
            cluster_wait();
            cluster_arrive();
            cluster_wait();
        }
    } else {
        if constexpr (kMHalves == 2) warpgroup_reg_inc<kEpilogueRegs>();
        // ================= epilogue =================
        // Warpgroup `wg` (four warps) drains the accumulator of rows [128 wg, 128 wg + 128) of this CTA's tile: one
        // warpgroup with 128-row tiles, two working side by side with 256-row tiles.
        const uint32_t wg = (warp_idx - kEpilogueWarpBase) / 4;
        const uint32_t quarter = warp_idx % 4;                        // tensor-memory lanes [32q, 32q+32)
        const uint32_t row_in_tile = quarter * 32 + lane;             // row inside the warpgroup's 128 rows
        const uint32_t epi_tid = threadIdx.x - (kEpilogueWarpBase + 4 * wg) * 32;
        const uint32_t bar_id = 1 + wg;
        const bool prof_thread = epi_tid == 0 && wg == 0;
        // The staging buffers are divided among the warpgroups, two each
        constexpr uint32_t kBuffersPerWG = kNumStoreStages / kMHalves;
        static_assert(kBuffersPerWG == 2 || kBuffersPerWG == 1, "every epilogue warpgroup has one or two staging buffers");
        const uint32_t staging = smem_base + kSmemD + wg * kBuffersPerWG * kStoreStageBytes;
        // 256-row tiles have no spare accumulator, so the next tile's MMAs wait for this one's tensor-memory reads.
        // With BF16 output a thread therefore first moves its whole accumulator row into registers (packed, BLOCK_N / 2
        // of them) and hands tensor memory back before any staging or store.  Otherwise (a spare accumulator, or FP32
        // output, whose rows would need twice the registers) the row is read group by group.
        constexpr bool kRowInRegs = kMHalves == 2 && !kDIsFP32;
        constexpr uint32_t kGroupBytes = kLayout.group_bytes();
        bool ok = true;
        [[maybe_unused]] uint32_t cluster_barriers_done = 0;
        uint32_t tile_iter = 0, store_iter = 0;
        DG_PROF_VAR(prof_wait); DG_PROF_VAR(prof_store);
        DG_PROF_BEGIN(prof_t0);
        while (ok && sched.next(tile)) {
            if (kGemmType == kKGrouped && tile.num_kb == 0) {
                // An empty group contributes nothing: D[g] = 0 unless the GEMM accumulates into D
                if constexpr (!kAccumulate) {
                    const uint32_t d_row = tile.d_row_base + tile.m_block * TILE_M + wg * BLOCK_M + row_in_tile;
                    if (tile.m_block * TILE_M + wg * BLOCK_M + row_in_tile < p.shape_m) {
                        uint8_t* drow = reinterpret_cast<uint8_t*>(p.d) + static_cast<size_t>(d_row) * p.ldd * kDElemBytes;
                        #pragma unroll 4
                        for (uint32_t c = 0; c < BLOCK_N * kDElemBytes / 16; ++c) {
                            constexpr uint32_t kPerChunk = 16 / kDElemBytes;
                            const uint32_t col = tile.n_block * BLOCK_N + c * kPerChunk;
                            if (col + kPerChunk <= p.shape_n) {
                                *reinterpret_cast<uint4*>(drow + static_cast<size_t>(col) * kDElemBytes) = make_uint4(0, 0, 0, 0);
                            } else {
                                for (uint32_t b = col * kDElemBytes; b < p.shape_n * kDElemBytes && b < (col + kPerChunk) * kDElemBytes; ++b) drow[b] = 0;
                            }
                        }
                    }
                }
                continue;
            }
            const uint32_t accum = tile_iter % kNumAccumStages + wg, accum_phase = (tile_iter / kNumAccumStages) & 1;
            ++tile_iter;
            DG_PROF_BEGIN(prof_w);
            if (!mbar_wait(tmem_full_bar(accum), accum_phase, ctx, kRoleEpilogue, 1, DG_EPILOGUE_BACKOFF_NS)) { ok = false; break; }
            DG_PROF_ADD(prof_wait, prof_w);
            tc_fence_after_sync();
            if (prof_thread) DG_PROF_STAMP(3);              // first accumulator complete
            if (epi_tid == 0 && wg == 0 && tile_iter == 1) DG_PROF_STAMP_MAX(13);          // ... in the last CTA to have one

            // Cluster-reduced K slicing.  The CTAs of the cluster share the reduction by columns: CTA r owns the 8-column
            // chunks r, r + S, ... of the tile.  Every CTA sends each column of its FP32 accumulator straight from tensor
            // memory into the owner's shared memory (distributed shared memory stores: posted, so their latency is not
            // waited for), one cluster barrier makes all of it visible, and then every CTA adds the S slices of its own
            // columns out of its OWN shared memory, in slice order, scales, converts and writes them to D.  After that
            // barrier no CTA touches a peer's memory again, so none has to outlive its peers.
            // Receive area of a CTA: [slice][owned column][row] words from the start of dynamic shared memory: the D
            // staging buffers, which this form does not use, and beyond them the drained pipeline stages.
            if constexpr (kSplitCluster > 1) {
                static_assert(kSplitCluster == 1 || kRecvBytes <= kSmemA + kNumStages * (kABytes + kBBytes), "the receive area fits the staging buffers and stages");
                if constexpr (kRecvOverStages) {
                    // Peers write over this CTA's pipeline stages: they may start once every CTA's MMAs have read theirs
                    cluster_arrive();
                    cluster_wait();
                } else {
                    cluster_wait();             // (arrived at set-up) every CTA of the cluster is running
                }
                ++cluster_barriers_done;
                uint32_t owners[kSplitCluster];
                #pragma unroll
                for (uint32_t r = 0; r < kSplitCluster; ++r)
                    owners[r] = map_to_cta(smem_base + kSmemD + (split_rank * kRecvCols * BLOCK_M + row_in_tile) * 4, r);
                #pragma unroll
                for (uint32_t b = 0; b < BLOCK_N / 16; ++b) {
                    uint32_t v[16];
                    tmem_ld_32x32b_x16(tmem_base + ((quarter * 32) << 16) + accum * UMMA_N + b * 16, v);
                    tmem_ld_wait();
                    #pragma unroll
                    for (uint32_t i = 0; i < 16; ++i) {
                        const uint32_t chunk = (b * 16 + i) / 8, owned_col = chunk / kSplitCluster * 8 + i % 8;
                        st_shared_cluster_u32(owners[chunk % kSplitCluster] + owned_col * BLOCK_M * 4, v[i]);
                    }
                }
                tc_fence_before_sync();
                mbar_arrive(tmem_empty_bar(accum));
                if (prof_thread) DG_PROF_STAMP(7);          // accumulator sent
                cluster_arrive();               // release: what this CTA sent is visible to its owners
                cluster_wait();
                ++cluster_barriers_done;
                if (prof_thread) DG_PROF_STAMP(8);          // every slice of the cluster has arrived
                const uint32_t recv = smem_base + kSmemD;

                if constexpr (kTransposedD) {
                    // Work items are (owned column, 8 consecutive rows): 32 contiguous bytes of every slice, 8 consecutive
                    // elements of one row of the caller's D
                    constexpr uint32_t kItems = kRecvCols * (BLOCK_M / 8);
                    #pragma unroll 1
                    for (uint32_t q = epi_tid; q < kItems; q += 128) {
                        const uint32_t oc = q / (BLOCK_M / 8), r8 = q % (BLOCK_M / 8);
                        const uint32_t c = (oc / 8 * kSplitCluster + split_rank) * 8 + oc % 8;      // column of the tile
                        const uint32_t col = tile.n_block * BLOCK_N + c;             // row of the caller's D
                        const uint32_t row = tile.m_block * BLOCK_M + r8 * 8;        // its first column
                        if (c >= BLOCK_N || col >= p.shape_n || row >= p.shape_m) continue;
                        float sum[8];
                        #pragma unroll
                        for (uint32_t i = 0; i < 8; ++i) sum[i] = 0.0f;
                        #pragma unroll
                        for (uint32_t r = 0; r < kSplitCluster; ++r) {
                            const uint4 lo = ld_shared_v4(recv + ((r * kRecvCols + oc) * BLOCK_M + r8 * 8) * 4);
                            const uint4 hi = ld_shared_v4(recv + ((r * kRecvCols + oc) * BLOCK_M + r8 * 8) * 4 + 16);
                            sum[0] += __uint_as_float(lo.x); sum[1] += __uint_as_float(lo.y); sum[2] += __uint_as_float(lo.z); sum[3] += __uint_as_float(lo.w);
                            sum[4] += __uint_as_float(hi.x); sum[5] += __uint_as_float(hi.y); sum[6] += __uint_as_float(hi.z); sum[7] += __uint_as_float(hi.w);
                        }
                        #pragma unroll
                        for (uint32_t i = 0; i < 8; ++i) sum[i] *= p.alpha;
                        const size_t at = static_cast<size_t>(col) * p.ldd + row;
                        if constexpr (kDIsFP32) {
                            float* out = reinterpret_cast<float*>(p.d) + at;
                            if (row + 8 <= p.shape_m) {
                                *reinterpret_cast<float4*>(out) = make_float4(sum[0], sum[1], sum[2], sum[3]);
                                *reinterpret_cast<float4*>(out + 4) = make_float4(sum[4], sum[5], sum[6], sum[7]);
                            } else {
                                #pragma unroll
                                for (uint32_t i = 0; i < 8; ++i)
                                    if (row + i < p.shape_m) out[i] = sum[i];
                            }
                        } else {
                            unsigned short* out = reinterpret_cast<unsigned short*>(p.d) + at;
                            uint32_t w[4];
                            #pragma unroll
                            for (uint32_t i = 0; i < 4; ++i) w[i] = pack_bf16x2(sum[2 * i], sum[2 * i + 1]);
                            if (row + 8 <= p.shape_m) {
                                *reinterpret_cast<uint4*>(out) = make_uint4(w[0], w[1], w[2], w[3]);
                            } else {
                                #pragma unroll
                                for (uint32_t i = 0; i < 8; ++i)
                                    if (row + i < p.shape_m) out[i] = static_cast<unsigned short>(w[i / 2] >> (16 * (i % 2)));
                            }
                        }
                    }
                    continue;
                }
                const uint32_t d_row = tile.m_block * BLOCK_M + row_in_tile;
                if (d_row < p.shape_m) {
                    uint8_t* drow = reinterpret_cast<uint8_t*>(p.d) + static_cast<size_t>(d_row) * p.ldd * kDElemBytes;
                    #pragma unroll
                    for (uint32_t jj = 0; jj < kRecvCols / 8; ++jj) {
                        const uint32_t j = jj * kSplitCluster + split_rank;
                        const uint32_t col = tile.n_block * BLOCK_N + j * 8;
                        if (j < BLOCK_N / 8 && col < p.shape_n) {
                            float sum[8];
                            #pragma unroll
                            for (uint32_t i = 0; i < 8; ++i) {
                                sum[i] = 0.0f;                  // (0 + first slice: the same operations as the two-kernel reduction)
                                #pragma unroll
                                for (uint32_t r = 0; r < kSplitCluster; ++r)
                                    sum[i] += __uint_as_float(ld_shared_u32(recv + ((r * kRecvCols + jj * 8 + i) * BLOCK_M + row_in_tile) * 4));
                                sum[i] *= p.alpha;
                            }
                            if constexpr (kDIsFP32) {
                                float* out = reinterpret_cast<float*>(drow) + col;
                                if (col + 8 <= p.shape_n) {
                                    *reinterpret_cast<float4*>(out) = make_float4(sum[0], sum[1], sum[2], sum[3]);
                                    *reinterpret_cast<float4*>(out + 4) = make_float4(sum[4], sum[5], sum[6], sum[7]);
                                } else {
                                    #pragma unroll
                                    for (uint32_t i = 0; i < 8; ++i)
                                        if (col + i < p.shape_n) out[i] = sum[i];
                                }
                            } else {
                                unsigned short* out = reinterpret_cast<unsigned short*>(drow) + col;
                                uint32_t q[4];
                                #pragma unroll
                                for (uint32_t i = 0; i < 4; ++i) q[i] = pack_bf16x2(sum[2 * i], sum[2 * i + 1]);
                                if (col + 8 <= p.shape_n) {
                                    *reinterpret_cast<uint4*>(out) = make_uint4(q[0], q[1], q[2], q[3]);
                                } else {
                                    #pragma unroll
                                    for (uint32_t i = 0; i < 8; ++i)
                                        if (col + i < p.shape_n) out[i] = static_cast<unsigned short>(q[i / 2] >> (16 * (i % 2)));
                                }
                            }
                        }
                    }
                }
                continue;
            }

            const uint32_t n0 = tile.n_block * BLOCK_N;
            const uint32_t d_row0 = tile.d_row_base + tile.m_block * TILE_M + cta_rank * CTA_M + wg * BLOCK_M +
                                    (kSplitK ? tile.split * p.split_panel_rows : 0u);
            const uint32_t tmem_row_addr = tmem_base + ((quarter * 32) << 16) + accum * UMMA_N;
            // Rows of this 128-row part that may be written
            const uint32_t rows_before = cta_rank * CTA_M + wg * BLOCK_M;
            const uint32_t valid_rows = tile.valid_rows <= rows_before ? 0u :
                                        (tile.valid_rows - rows_before < BLOCK_M ? tile.valid_rows - rows_before : BLOCK_M);
            // (fewer than 128 only in a ragged tile of the masked and prefix-sum layouts: those rows are stored one by one)
            const bool direct = (kGemmType == kMGroupedMasked || kGemmType == kMGroupedPsum || kGemmType == kKGrouped) && valid_rows < BLOCK_M;
            auto release_tmem = [&]() {
                tc_fence_before_sync();
                if (kCluster == 1 || is_leader) mbar_arrive(tmem_empty_bar(accum));
                else mbar_arrive_cluster(in_leader(tmem_empty_bar(accum)));
            };

            if constexpr (kTransposedD) {
                // Thread = one row of the tile = one column of the caller's D.  The tile leaves transposed through shared
                // memory: chunk by chunk of `kTRows` rows of D (= columns of the tile), every thread writes its element of
                // each row (consecutive lanes, consecutive addresses), and one TMA store per chunk takes the
                // [kTRows][128] block to D, which also clips rows beyond the caller's M and columns beyond its N.
                constexpr uint32_t kTRowBytes = 128 * kDElemBytes;
                constexpr uint32_t kTRows = kTransposedRows;
                const uint32_t t_stage = smem_base + kSmemD;
                const uint32_t d_col0 = tile.m_block * TILE_M + cta_rank * CTA_M;       // first column of D this CTA writes
                #pragma unroll
                for (uint32_t c0 = 0; c0 < BLOCK_N; c0 += kTRows) {
                    // the staging block is free once the previous chunk's store has read it
                    if (store_iter > 0) {
                        if (epi_tid == 0) tma_store_wait_read<0>();
                        named_barrier_sync(bar_id, kNumEpilogueThreads);
                    }
                    ++store_iter;
                    #pragma unroll
                    for (uint32_t b = c0 / 16; b < (c0 + kTRows < BLOCK_N ? c0 + kTRows : BLOCK_N) / 16; ++b) {
                        uint32_t v[16];
                        tmem_ld_32x32b_x16(tmem_row_addr + b * 16, v);
                        tmem_ld_wait();
                        if (b + 1 == BLOCK_N / 16) release_tmem();
                        #pragma unroll
                        for (uint32_t i = 0; i < 16; ++i) {
                            const float x = __uint_as_float(v[i]) * p.alpha;
                            const uint32_t at = t_stage + (b * 16 + i - c0) * kTRowBytes + row_in_tile * kDElemBytes;
                            if constexpr (kDIsFP32) st_shared_u32(at, __float_as_uint(x));
                            else st_shared_u16(at, pack_bf16x2(x, 0.0f) & 0xFFFFu);
                        }
                    }
                    fence_proxy_async_smem();
                    named_barrier_sync(bar_id, kNumEpilogueThreads);
                    if (epi_tid == 0) {
                        tma_store_2d(&tm_d, t_stage, static_cast<int32_t>(d_col0), static_cast<int32_t>(n0 + c0));
                        tma_store_commit();
                    }
                }
                continue;
            }

            [[maybe_unused]] uint32_t row[kRowInRegs ? BLOCK_N / 2 : 1];        // BF16 pairs: columns (2i, 2i+1) of the tile row
            if constexpr (kRowInRegs) {
                // 32 columns per round trip to tensor memory (more in flight cost registers the row itself needs:
                // 48 and 64 columns spilled and measured 3-20 % slower)
                constexpr uint32_t kLoadsPerTrip = 2;
                #pragma unroll
                for (uint32_t b = 0; b < BLOCK_N / 16; b += kLoadsPerTrip) {
                    uint32_t v[kLoadsPerTrip][16];
                    #pragma unroll
                    for (uint32_t l = 0; l < kLoadsPerTrip; ++l)
                        if (b + l < BLOCK_N / 16) tmem_ld_32x32b_x16(tmem_row_addr + (b + l) * 16, v[l]);
                    tmem_ld_wait();
                    #pragma unroll
                    for (uint32_t l = 0; l < kLoadsPerTrip; ++l)
                        if (b + l < BLOCK_N / 16) {
                            if constexpr (kStochastic) {
                                #pragma unroll
                                for (uint32_t j = 0; j < 4; ++j)       // quartets are aligned to absolute columns
                                    stochastic_round_quartet(v[l][4 * j], v[l][4 * j + 1], v[l][4 * j + 2], v[l][4 * j + 3],
                                                             (n0 + (b + l) * 16) / 4 + j, row[(b + l) * 8 + 2 * j], row[(b + l) * 8 + 2 * j + 1]);
                            } else {
                                #pragma unroll
                                for (uint32_t i = 0; i < 8; ++i)
                                    row[(b + l) * 8 + i] = pack_bf16x2(__uint_as_float(v[l][2 * i]) * p.alpha,
                                                                       __uint_as_float(v[l][2 * i + 1]) * p.alpha);
                            }
                        }
                }
                release_tmem();
            }

            #pragma unroll
            for (uint32_t g = 0; g < kNumGroups; ++g) {
                // Columns [g * kGroupCols, + kCols) of the tile: one group (or the ragged rest) of every row
                const uint32_t kCols = (g + 1) * kGroupCols <= BLOCK_N ? kGroupCols : BLOCK_N - g * kGroupCols;
                constexpr uint32_t kMaxLoads = (kGroupCols + 15) / 16;
                [[maybe_unused]] uint32_t v[kRowInRegs ? 1 : kMaxLoads][16];
                if constexpr (!kRowInRegs) {
                    #pragma unroll
                    for (uint32_t l = 0; l < kMaxLoads; ++l)
                        if (l * 16 < kCols) tmem_ld_32x32b_x16(tmem_row_addr + g * kGroupCols + l * 16, v[l]);
                    tmem_ld_wait();
                    if (g + 1 == kNumGroups) release_tmem();           // the last of the accumulator is in registers
                    #pragma unroll
                    for (uint32_t l = 0; l < kMaxLoads; ++l)
                        if (l * 16 < kCols) {
                            #pragma unroll
                            for (uint32_t i = 0; i < 16; ++i)
                                v[l][i] = __float_as_uint(__uint_as_float(v[l][i]) * p.alpha);
                        }
                }
                // Quantised output: the group's BF16-rounded values, 32 columns per scale, as e4m3 words; the scale bytes
                // go straight to global memory (one byte per row and 32 columns)
                [[maybe_unused]] uint32_t q8[kDIsFP8 ? kGroupCols / 4 : 1];
                if constexpr (kDIsFP8) {
                    #pragma unroll
                    for (uint32_t t = 0; t < kGroupCols / 32; ++t) {
                        if (t * 32 < kCols) {
                            uint32_t pairs[16];                     // BF16 pairs of the 32 columns
                            #pragma unroll
                            for (uint32_t i = 0; i < 16; ++i) {
                                if constexpr (kRowInRegs) pairs[i] = row[g * (kGroupCols / 2) + t * 16 + i];
                                else pairs[i] = pack_bf16x2(__uint_as_float(v[t * 2 + i / 8][(2 * i) % 16]),
                                                            __uint_as_float(v[t * 2 + i / 8][(2 * i) % 16 + 1]));
                            }
                            float amax = 0.0f;
                            #pragma unroll
                            for (uint32_t i = 0; i < 16; ++i)
                                amax = fmaxf(amax, fmaxf(fabsf(bf16_lo(pairs[i])), fabsf(bf16_hi(pairs[i]))));
                            const float sf = e4m3_block_scale(amax), inv = 1.0f / sf;
                            #pragma unroll
                            for (uint32_t i = 0; i < 8; ++i)
                                q8[t * 8 + i] = pack_e4m3x4(bf16_lo(pairs[2 * i]) * inv, bf16_hi(pairs[2 * i]) * inv,
                                                            bf16_lo(pairs[2 * i + 1]) * inv, bf16_hi(pairs[2 * i + 1]) * inv);
                            // Batched: the scale columns of all batches follow one another, as in D viewed as [m, batches * n]
                            const uint32_t col = n0 + g * kGroupCols + t * 32, d_row = d_row0 + row_in_tile;
                            const uint32_t sf_col = (kGemmType == kBatched ? tile.group * p.shape_n : 0u) + col;
                            if (d_row < p.shape_m && col < p.shape_n)
                                reinterpret_cast<uint8_t*>(p.sfd + static_cast<size_t>(sf_col / 128) * p.sfd_pitch + d_row)[(sf_col / 32) % 4] =
                                    static_cast<uint8_t>(ue8m0_code(sf));
                        }
                    }
                }
                // The four registers of 16-byte chunk c of this group's row: 16 e4m3, 8 BF16 or 4 FP32 values
                constexpr uint32_t kElemsPerChunk = 16 / kDElemBytes;
                auto chunk = [&](uint32_t c, uint32_t (&out)[4]) {
                    if constexpr (kDIsFP8) {
                        #pragma unroll
                        for (uint32_t i = 0; i < 4; ++i) out[i] = q8[c * 4 + i];
                    } else if constexpr (kRowInRegs) {
                        #pragma unroll
                        for (uint32_t i = 0; i < 4; ++i) out[i] = row[g * (kGroupCols / 2) + c * 4 + i];
                    } else if constexpr (!kDIsFP32) {
                        const uint32_t l = (c * 8) / 16, i0 = (c * 8) % 16;
                        if constexpr (kStochastic) {
                            #pragma unroll
                            for (uint32_t j = 0; j < 2; ++j)
                                stochastic_round_quartet(v[l][i0 + 4 * j], v[l][i0 + 4 * j + 1], v[l][i0 + 4 * j + 2], v[l][i0 + 4 * j + 3],
                                                         (n0 + g * kGroupCols + c * 8) / 4 + j, out[2 * j], out[2 * j + 1]);
                        } else {
                            #pragma unroll
                            for (uint32_t i = 0; i < 4; ++i)
                                out[i] = pack_bf16x2(__uint_as_float(v[l][i0 + 2 * i]), __uint_as_float(v[l][i0 + 2 * i + 1]));
                        }
                    } else {
                        const uint32_t l = (c * 4) / 16, i0 = (c * 4) % 16;
                        #pragma unroll
                        for (uint32_t i = 0; i < 4; ++i) out[i] = v[l][i0 + i];
                    }
                };
                const uint32_t col0 = n0 + g * kGroupCols;

                if (!direct) {
                    const uint32_t sb = store_iter % kBuffersPerWG;
                    ++store_iter;
                    // The staging buffer is free once the TMA stores issued from it two groups ago have read it
                    DG_PROF_BEGIN(prof_s);
                    if (epi_tid == 0) tma_store_wait_read<kBuffersPerWG - 1>();
                    named_barrier_sync(bar_id, kNumEpilogueThreads);
                    DG_PROF_ADD(prof_store, prof_s);
                    const uint32_t stage_addr = staging + sb * kStoreStageBytes;
                    // A complete group is one box of kGroupBytes-wide rows; the ragged last group of a tile row is split
                    // into narrower boxes (rows of kStoreRowBytes)
                    const bool full_group = kCols == kGroupCols;
                    const uint32_t row_bytes = full_group ? kGroupBytes : kStoreRowBytes;
                    const uint32_t box_bytes = BLOCK_M * row_bytes;
                    const uint32_t swizzle_mask = row_bytes == 128 ? 7u : (row_bytes == 64 ? 3u : 1u);
                    #pragma unroll
                    for (uint32_t c = 0; c < kGroupCols / kElemsPerChunk; ++c) {
                        if (c * kElemsPerChunk < kCols) {
                            // chunk c of the row lives in store box (c * 16 / row bytes), at swizzled chunk position
                            const uint32_t box = (c * 16) / row_bytes, in_row = (c * 16) % row_bytes;
                            const uint32_t off = row_in_tile * row_bytes + in_row;
                            const uint32_t phys = off ^ (((off >> 7) & swizzle_mask) << 4);
                            uint32_t q[4];
                            chunk(c, q);
                            st_shared_v4(stage_addr + box * box_bytes + phys, q[0], q[1], q[2], q[3]);
                        }
                    }
                    fence_proxy_async_smem();
                    named_barrier_sync(bar_id, kNumEpilogueThreads);
                    if (epi_tid == 0) {
                        const uint32_t cols_per_box = full_group ? kGroupCols : kStoreCols;
                        const CUtensorMap* map = full_group ? &tm_d_full : &tm_d;
                        #pragma unroll
                        for (uint32_t box = 0; box < kGroupCols / kStoreCols; ++box) {
                            if (box * cols_per_box < kCols) {
                                tma_out(map, stage_addr + box * box_bytes, col0 + box * cols_per_box, d_row0, tile.group);
                            }
                        }
                        tma_store_commit();
                    }
                } else if (row_in_tile < valid_rows) {
                    // Ragged tile of a grouped layout: rows at or beyond the group's row count stay untouched (the masked and
                    // prefix-sum layouts never accumulate; the k-grouped GEMM may: every element belongs to one thread of
                    // one tile, so a plain read-add-write does)
                    if constexpr (kDIsFP8) {
                        // not reached: ragged tiles exist only in the grouped layouts
                    } else if constexpr (!kDIsFP32) {
                        unsigned short* drow = reinterpret_cast<unsigned short*>(p.d) + static_cast<size_t>(d_row0 + row_in_tile) * p.ldd;
                        #pragma unroll
                        for (uint32_t c = 0; c < kGroupCols / 8; ++c) {
                            if (c * 8 < kCols) {
                                const uint32_t col = col0 + c * 8;
                                uint32_t q[4];
                                chunk(c, q);
                                if constexpr (kAccumulate) {
                                    #pragma unroll
                                    for (uint32_t e = 0; e < 8; ++e) {
                                        if (col + e < p.shape_n) {
                                            const float sum = __uint_as_float(static_cast<uint32_t>(drow[col + e]) << 16) +
                                                              (e % 2 ? bf16_hi(q[e / 2]) : bf16_lo(q[e / 2]));
                                            drow[col + e] = static_cast<unsigned short>(pack_bf16x2(sum, 0.0f) & 0xFFFFu);
                                        }
                                    }
                                } else if (col + 8 <= p.shape_n) {
                                    *reinterpret_cast<uint4*>(drow + col) = make_uint4(q[0], q[1], q[2], q[3]);
                                } else {
                                    #pragma unroll
                                    for (uint32_t e = 0; e < 8; ++e)
                                        if (col + e < p.shape_n) drow[col + e] = static_cast<unsigned short>(q[e / 2] >> (16 * (e % 2)));
                                }
                            }
                        }
                    } else {
                        float* drow = reinterpret_cast<float*>(p.d) + static_cast<size_t>(d_row0 + row_in_tile) * p.ldd;
                        #pragma unroll
                        for (uint32_t c = 0; c < kGroupCols; ++c)
                            if (c < kCols && col0 + c < p.shape_n)
                                drow[col0 + c] = (kAccumulate ? drow[col0 + c] : 0.0f) + __uint_as_float(v[c / 16][c % 16]);
                    }
                }
            }
        }
        if constexpr (kSplitCluster > 1) {
            // no tile, or a wait ran out: the rest of the cluster must not wait for ever
            if (cluster_barriers_done == 0) {
                if constexpr (kRecvOverStages) cluster_arrive();
                cluster_wait();
                ++cluster_barriers_done;
            }
            if (cluster_barriers_done == 1) {
                cluster_arrive();
                cluster_wait();
            }
        }
        if (prof_thread) {
            DG_PROF_VAR(prof_total);
            DG_PROF_ADD(prof_total, prof_t0);
            DG_PROF_FLUSH(kProfEpiWaitTmemFull, prof_wait);
            DG_PROF_FLUSH(kProfEpiStoreWait, prof_store);
            DG_PROF_FLUSH(kProfEpiTotal, prof_total);
        }
        // Every byte of D must be in global memory before the grid completes
        if (prof_thread) DG_PROF_STAMP(4);                  // last store issued
        if (epi_tid == 0) tma_store_wait<0>();
        if (prof_thread) DG_PROF_STAMP(5);                  // stores complete
    }

    // ---- tear-down ------------------------------------------------------------------------------
    __syncthreads();
    if (*abort_flag != 0) {
        // A wait ran out somewhere in this CTA: give copies that are still in flight time to land
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000) { }
        __syncthreads();
    }
    if constexpr (kCluster > 1) {
        // Neither CTA of a pair may exit (or free tensor memory) while its peer can still signal its barriers or read
        // its shared memory.  (The CTAs of a K-sliced cluster are done with one another after the epilogue's barrier.)
        tc_fence_before_sync();
        cluster_arrive();
        cluster_wait();
    }
    if (warp_idx == 2) {
        tc_fence_after_sync();
        tmem_dealloc<kCluster>(tmem_base, kTmemCols);
    }
    if (threadIdx.x == 0) DG_PROF_STAMP(6);                 // exit
    if (threadIdx.x == 0) DG_PROF_STAMP_MAX(11);            // last CTA to leave
}
