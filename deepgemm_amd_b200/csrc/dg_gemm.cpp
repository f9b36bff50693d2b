// GEMM entry points: argument checks of the reference's API layer (csrc/apis/gemm.hpp:78-318,
// csrc/utils/layout.hpp:101-140), tile-shape heuristics for B200, tensor maps, kernel source
// generation and launch (the work of csrc/jit_kernels/impls/sm100_fp8_fp4_gemm_1d1d.hpp:101-323 and
// csrc/jit_kernels/impls/runtime_utils.hpp:119-159,325-408 in the reference).
#include "dg_common.hpp"

#include <algorithm>
#include <cstring>
#include <array>
#include <atomic>
#include <map>
#include <mutex>
#include <sstream>

#include "device/dg/gemm_config.hpp"
#include "device/dg/tile_scheduler.cuh"

namespace dg {

int launch_splitk_reduce(const float* ws, void* d, int m, int n, int64_t ld_ws, int64_t panel_rows, int64_t ldd, int num_splits,
                         float alpha, bool d_fp32, cudaStream_t stream);      // dg_splitk.cu

namespace {

// Mirror of dg::GemmParams in device/dg/gemm_fp8_fp4.cuh (kernel argument, passed by value)
struct GemmParams {
    const int* grouped_layout;
    void* d;
    int* status;
    uint32_t shape_m, shape_n, shape_k, num_groups, ldd;
    float alpha;
    unsigned long long* profile;
    uint32_t num_splits, kb_per_split, split_panel_rows;
    uint32_t group_alignment;
    uint32_t* sfd;
    uint32_t sfd_pitch;
    uint32_t kb_per_batch;
};

// Split-K scratch: num_splits stacked FP32 [rows x N] panels.  One buffer per device, shared by every stream (a
// captured graph may replay on any stream, so a per-stream buffer would promise nothing): split-K GEMMs that overlap
// on the GPU from different streams would race on it; set DG_FORCE_SPLIT_K=1 to keep such workloads unsplit.  The
// buffer only grows; growing allocates, so the first call of a shape must not be inside a stream capture.
std::mutex g_workspace_mu;
std::map<int, std::pair<float*, size_t>> g_workspaces;

int split_workspace(size_t bytes, float** out) {
    std::mutex& mu = g_workspace_mu;
    auto& per_device = g_workspaces;
    std::lock_guard<std::mutex> lock(mu);
    int device = 0;
    DG_CUDA_RT(cudaGetDevice(&device));
    auto& w = per_device[device];
    if (w.second < bytes) {
        if (w.first != nullptr) DG_CUDA_RT(cudaFree(w.first));
        w = {nullptr, 0};
        const size_t rounded = align_up<size_t>(bytes, 1 << 20);
        DG_CUDA_RT(cudaMalloc(reinterpret_cast<void**>(&w.first), rounded));
        w.second = rounded;
    }
    *out = w.first;
    return DG_OK;
}

// Tuning aid (DG_PROFILE=1): a device buffer of per-role wait-cycle counters and timeline stamps, printed after every launch
unsigned long long* profile_buffer() {
    static unsigned long long* buf = nullptr;
    if (buf == nullptr && cudaMalloc(reinterpret_cast<void**>(&buf), 32 * sizeof(unsigned long long)) != cudaSuccess) buf = nullptr;
    return buf;
}

struct Problem {
    int kind;
    int m, n, k, groups;
    bool a_fp4, b_fp4, ab_bf16, d_fp32, d_fp8, accumulate, a_mn_major, b_mn_major;
    int gran_k_a, gran_k_b;
    int expected_m;
    bool write_padding;      // prefix-sum layout: also write the padding rows of D up to the next aligned row
    bool k_psum;             // k-grouped: grouped_layout holds prefix sums
    bool stochastic;         // BF16 output rounded stochastically
    int reduce_batches;      // dense BF16 GEMM summed over this many batches as well (k is then batches x K of one batch); 0 = no
    bool mxf4;               // FP4 x FP4 through kind::mxf4 (packed operands in shared memory, 256 elements of K per stage)
};

int validate(int kind, const dg_gemm_args_t* a, bool need_pointers, Problem* p) {
    DG_REQUIRE(a != nullptr);
    DG_REQUIRE(kind == DG_GEMM_DENSE || kind == DG_GEMM_M_GROUPED_CONTIGUOUS || kind == DG_GEMM_M_GROUPED_MASKED ||
               kind == DG_GEMM_M_GROUPED_CONTIGUOUS_PSUM || kind == DG_GEMM_K_GROUPED_CONTIGUOUS || kind == DG_GEMM_BATCHED);
    const bool k_grouped = kind == DG_GEMM_K_GROUPED_CONTIGUOUS, batched = kind == DG_GEMM_BATCHED;
    // BF16 operands (no scales): the reference's bf16_gemm_* family, same kernel with the scale path compiled out
    const bool ab_bf16 = a->a_dtype == DG_BF16 && a->b_dtype == DG_BF16;
    DG_REQUIRE(ab_bf16 || a->a_dtype == DG_FP8_E4M3 || a->a_dtype == DG_FP4_E2M1_X2);
    DG_REQUIRE(ab_bf16 || a->b_dtype == DG_FP8_E4M3 || a->b_dtype == DG_FP4_E2M1_X2);
    DG_REQUIRE(a->d_dtype == DG_BF16 || a->d_dtype == DG_FP32 || a->d_dtype == DG_FP8_E4M3);
    if (kind != DG_GEMM_DENSE && !k_grouped && !batched) DG_REQUIRE(a->d_dtype == DG_BF16);            // gemm.hpp:209,299
    if (k_grouped) DG_REQUIRE(a->d_dtype == DG_BF16 || a->d_dtype == DG_FP32);
    if (batched) {
        // einsum.hpp:183-243: [B, M, K] x [B, N, K]^T -> [B, M, N], any batch strides that a tensor map can express
        DG_REQUIRE(a->num_groups > 0 && !a->has_alpha);
        DG_REQUIRE(ab_bf16 || (a->a_dtype == DG_FP8_E4M3 && a->b_dtype == DG_FP8_E4M3));
        DG_REQUIRE((a->batch_stride_a * (ab_bf16 ? 2 : 1)) % 16 == 0 && (a->batch_stride_b * (ab_bf16 ? 2 : 1)) % 16 == 0);
        DG_REQUIRE((a->batch_stride_d * (a->d_dtype == DG_FP32 ? 4 : (a->d_dtype == DG_FP8_E4M3 ? 1 : 2))) % 16 == 0);
        // quantised output: the scale columns of the batches follow one another, so a batch is whole packed words
        if (a->d_dtype == DG_FP8_E4M3) DG_REQUIRE(a->n % 128 == 0 && a->batch_stride_d == a->n);
    }
    if (a->d_dtype == DG_FP8_E4M3) {
        // "FP8 quantization requires a direct E4M3 output" (epilogue_class.hpp:84-87); the epilogues do not compose
        DG_REQUIRE(!a->accumulate && !a->has_alpha);
        if (need_pointers) DG_REQUIRE(a->sfd != nullptr && reinterpret_cast<uintptr_t>(a->sfd) % 4 == 0);
        DG_REQUIRE(a->sfd_pitch >= align_up<int64_t>(a->m, 4));
        DG_REQUIRE(kind == DG_GEMM_DENSE || batched);
    }
    DG_REQUIRE(a->m >= 0 && a->n >= 0 && a->k >= 0);
    if (!ab_bf16) {
        DG_REQUIRE(a->gran_k_a == 32 || a->gran_k_a == 128);
        DG_REQUIRE(a->gran_k_b == 32 || a->gran_k_b == 128);
    }
    if (kind == DG_GEMM_DENSE) {
        DG_REQUIRE(a->num_groups == 1);
    } else if (batched) {
        DG_REQUIRE(a->n > 0 && a->k > 0);
    } else if (k_grouped) {
        // gemm.hpp:320-372: 1-D scales of one granularity, K slices aligned to whole K-blocks, contiguous operands
        DG_REQUIRE(a->num_groups > 0 && (ab_bf16 || a->gran_k_a == a->gran_k_b));
        DG_REQUIRE(state().mk_alignment % 128 == 0);
        DG_REQUIRE(!a->has_alpha);
    } else {
        DG_REQUIRE(a->n > 0 && a->k > 0 && a->num_groups > 0);                // gemm.hpp:208,296
        DG_REQUIRE(a->major_a == DG_MAJOR_K);                                 // gemm.hpp:197,285
        DG_REQUIRE(!a->accumulate);
    }
    if (kind == DG_GEMM_M_GROUPED_MASKED) {
        DG_REQUIRE(a->major_b == DG_MAJOR_K);                                 // gemm.hpp:285
        DG_REQUIRE(a->expected_m > 0 && a->m > 0);                            // gemm.hpp:296
    }
    // FP4 operands on either side go through kind::mxf8f6f4 (E2M1 format, unpacked to one byte per element in shared
    // memory by the tensor map), FP4 x FP4 included: the same results as the reference's kind::mxf4 path
    // (csrc/utils/layout.hpp:42-45) at the FP8 rate rather than twice it.
    DG_REQUIRE((a->major_a == DG_MAJOR_K || a->major_a == DG_MAJOR_MN) && (a->major_b == DG_MAJOR_K || a->major_b == DG_MAJOR_MN));
    // An MN-major packed FP4 B (two columns of N per byte; the weight-gradient and transposed-weight forms of the FP8 x FP4
    // GEMM, csrc/utils/layout.hpp:66-83) is unpacked by the tensor map along N exactly as a K-major one is along K
    if (a->major_a == DG_MAJOR_MN && a->a_dtype == DG_FP4_E2M1_X2)
        return fail(DG_ERR_UNSUPPORTED, "an MN-major packed FP4 A is not built; FP4 on the A side must be K-major");
    if (a->major_b == DG_MAJOR_MN && a->b_dtype == DG_FP4_E2M1_X2) {
        if (a->a_dtype == DG_FP4_E2M1_X2) return fail(DG_ERR_UNSUPPORTED, "FP4 x FP4 takes K-major operands");
        // (the packed 4-bit tensor-map type wants its contiguous extent in multiples of 128 elements, as K is for K-major FP4)
        if (a->n % 128 != 0) return fail(DG_ERR_INVALID_ARGUMENT, "an MN-major packed FP4 B needs n % 128 == 0 (n = %d)", a->n);
    }
    p->reduce_batches = 0;
    if (a->reduce_batches > 1) {
        // einsum.hpp:41-47, sm100_bmk_bnk_mn.hpp:23: contiguous K-major BF16 batches, K a whole number of 64-element blocks
        DG_REQUIRE(kind == DG_GEMM_DENSE && ab_bf16 && a->major_a == DG_MAJOR_K && a->major_b == DG_MAJOR_K);
        DG_REQUIRE(a->k % 64 == 0 && !a->accumulate && !a->has_alpha && a->d_dtype != DG_FP8_E4M3 && !a->stochastic_rounding);
        DG_REQUIRE((a->batch_stride_a * 2) % 16 == 0 && (a->batch_stride_b * 2) % 16 == 0);
        DG_REQUIRE(static_cast<int64_t>(a->k) * a->reduce_batches < (int64_t{1} << 31));
        p->reduce_batches = a->reduce_batches;
    }
    p->kind = kind;
    p->a_mn_major = a->major_a == DG_MAJOR_MN;
    p->b_mn_major = a->major_b == DG_MAJOR_MN;
    p->m = a->m; p->n = a->n; p->k = a->k * std::max(1, p->reduce_batches); p->groups = a->num_groups;
    p->a_fp4 = a->a_dtype == DG_FP4_E2M1_X2;
    p->b_fp4 = a->b_dtype == DG_FP4_E2M1_X2;
    p->ab_bf16 = ab_bf16;
    p->d_fp32 = a->d_dtype == DG_FP32;
    p->d_fp8 = a->d_dtype == DG_FP8_E4M3;
    p->accumulate = a->accumulate != 0;
    p->gran_k_a = ab_bf16 ? 128 : a->gran_k_a; p->gran_k_b = ab_bf16 ? 128 : a->gran_k_b;
    p->expected_m = a->expected_m;
    p->write_padding = kind == DG_GEMM_M_GROUPED_CONTIGUOUS_PSUM && a->ensure_zero_padding != 0;
    p->k_psum = k_grouped && a->use_psum_layout != 0;
    p->stochastic = a->stochastic_rounding != 0;
    // FP4 x FP4 with K-major operands and one scale per 32 elements of K runs through kind::mxf4 at twice the FP8 rate
    // (the reference's is_mxf4_mma, csrc/jit_kernels/impls/sm100_fp8_fp4_gemm_1d1d.hpp:36-39); other FP4 combinations
    // are unpacked to bytes and multiplied by kind::mxf8f6f4.  DG_DISABLE_MXF4=1 sends FP4 x FP4 down that path as well.
    p->mxf4 = p->a_fp4 && p->b_fp4 && !p->a_mn_major && !p->b_mn_major && p->gran_k_a == 32 && p->gran_k_b == 32 &&
              (kind == DG_GEMM_DENSE || kind == DG_GEMM_M_GROUPED_CONTIGUOUS || kind == DG_GEMM_M_GROUPED_MASKED ||
               kind == DG_GEMM_M_GROUPED_CONTIGUOUS_PSUM) && env_int("DISABLE_MXF4") == 0;
    // "Stochastic rounding requires a direct BF16 output" (epilogue_class.hpp:104-107); the epilogues do not compose
    if (p->stochastic) DG_REQUIRE(a->d_dtype == DG_BF16 && !a->accumulate && !a->has_alpha);
    if (a->m == 0 || a->n == 0 || a->k == 0) return DG_OK;                    // handled by the caller (gemm.hpp:17-53)

    // runtime_utils.hpp:133-135: the contiguous extent of a packed FP4 operand is whole 128-element blocks (K when it is
    // K-major; N for the MN-major B, checked above)
    if ((p->a_fp4 && !p->a_mn_major) || (p->b_fp4 && !p->b_mn_major)) DG_REQUIRE(a->k % 128 == 0);
    if (need_pointers) {
        DG_REQUIRE(a->a != nullptr && a->b != nullptr && a->d != nullptr);
        DG_REQUIRE(ab_bf16 || (a->sfa != nullptr && a->sfb != nullptr));
        const auto aligned = [](const void* ptr, uintptr_t al) { return reinterpret_cast<uintptr_t>(ptr) % al == 0; };
        DG_REQUIRE(aligned(a->a, p->a_fp4 ? 32 : 16));                        // runtime_utils.hpp:126
        DG_REQUIRE(aligned(a->b, p->b_fp4 ? 32 : 16));
        DG_REQUIRE(aligned(a->d, 16) && (ab_bf16 || (aligned(a->sfa, 16) && aligned(a->sfb, 16))));
        if (kind != DG_GEMM_DENSE && !batched) DG_REQUIRE(a->grouped_layout != nullptr);
    }
    // Pitch of the non-contiguous dimension: rows of K bytes (K-major) or K-slices of MN bytes (MN-major)
    // (storage elements: bytes for FP8 / packed FP4, bfloat16 elements for BF16)
    const int64_t k_bytes_a = p->a_mn_major ? a->m : (p->a_fp4 ? a->k / 2 : a->k);
    const int64_t k_bytes_b = p->b_mn_major ? (p->b_fp4 ? a->n / 2 : a->n) : (p->b_fp4 ? a->k / 2 : a->k);
    DG_REQUIRE(a->lda >= k_bytes_a && a->lda % (p->a_fp4 ? 32 : (ab_bf16 ? 8 : 16)) == 0);   // TMA: strides are multiples of 16 bytes
    DG_REQUIRE(a->ldb >= k_bytes_b && a->ldb % (p->b_fp4 ? 32 : (ab_bf16 ? 8 : 16)) == 0);
    const int d_elem = p->d_fp32 ? 4 : (p->d_fp8 ? 1 : 2);
    DG_REQUIRE(a->ldd >= a->n && (a->ldd * d_elem) % 16 == 0);
    // Packed scale tensors: csrc/utils/layout.hpp:121-130
    if (!ab_bf16) {
        DG_REQUIRE(a->sfa_pitch >= align_up<int64_t>(a->m, 4) && a->sfa_pitch % 4 == 0);
        DG_REQUIRE(a->sfb_pitch >= align_up<int64_t>(a->n, 4) && a->sfb_pitch % 4 == 0);
    }
    if (kind == DG_GEMM_M_GROUPED_CONTIGUOUS) {
        // Every expert segment is padded to the alignment, which the row blocks must divide
        DG_REQUIRE(state().mk_alignment % 128 == 0);
        DG_REQUIRE(a->m % 128 == 0);
    }
    if (kind == DG_GEMM_M_GROUPED_CONTIGUOUS_PSUM) {
        DG_REQUIRE(state().mk_alignment % 128 == 0);
        DG_REQUIRE(a->expected_m >= 0);
    }
    return DG_OK;
}

// ---- heuristics ------------------------------------------------------------------------------------
// A CTA works on (128 or 256) x block_n x 128 sub-tiles with block_n in 16..240.  With 256 rows it issues two
// 128-row MMAs per K-block on one B stage; with cluster_size 2 a CTA pair shares one tile (tcgen05 cta_group::2) and
// each CTA loads only half of the B tile.  The choice minimises a cycle model of the whole launch:
//     waves x (k_blocks x max(MMA, shared-memory traffic, stage ring) + per-tile overhead) + exposed epilogue + launch
// with per-SM, per-clock figures of B200: 8192 FP8 MACs and ~150 B through shared memory, writes by TMA and reads by
// the tensor core together.  The latter was fitted on this kernel: seven tile widths of the 256-row kernel and the
// 128-row kernel all ran within 5 % of (bytes written + bytes read) / 150 cycles per K-block.  It is why 256-row tiles
// win wherever M allows them: their B stage is written once and read by two MMAs' worth of rows.
// CTA pairs (tcgen05 cta_group::2) are chosen where they measured faster: each CTA then loads half of B, and B is read
// from shared memory once per pair.  Two forms: 128 rows per CTA with two accumulators (the epilogue of a tile overlaps
// the next tile's main loop: best for short K) and 256 rows per CTA (least shared-memory traffic per MMA cycle: best for
// long K).  Dense GEMMs with block-scaled operands, and the contiguous grouped layout when every expert segment is a
// whole number of pair tiles (alignment 256 or 512).
bool cluster_allowed(const Problem& p, int cluster) {
    if (cluster == 1) return true;
    if (p.ab_bf16 || p.reduce_batches > 1 || p.a_mn_major || p.b_mn_major) return false;       // (K-major block-scaled operands: what was measured)
    // (measured at M = 4096; smaller GEMMs keep the one-CTA forms their cost model was fitted on)
    return (p.kind == DG_GEMM_DENSE && p.m >= 1024) || p.kind == DG_GEMM_M_GROUPED_CONTIGUOUS;
}

// Layout of a candidate with the deepest pipeline that fits shared memory.  `item_kb` is the number of K-blocks (of
// block_k elements) one work item walks; fewer than the stage count makes the scale ring one buffer per stage.
GemmLayout fit_stages(GemmLayout lay, int64_t item_kb, int max_stages) {
    GemmLayout best = lay;
    best.num_stages = 0;
    for (int stages = 2; stages <= max_stages; ++stages) {
        lay.num_stages = static_cast<uint32_t>(stages);
        lay.short_k = item_kb < stages ? 1u : 0u;
        if (lay.total_bytes() > kSmemCapacity) break;
        best = lay;
    }
    return best;
}

// How many thread-block clusters of S CTAs (one CTA per SM) run at once.  A cluster lives inside one GPC, so the answer
// is the sum over GPCs of floor(SMs of the GPC / S), which only the driver knows: the table holds what it reported for
// kernels launched so far (cuOccupancyMaxActiveClusters), and until then the numbers of one B200, scaled by the SM count.
std::atomic<int> g_cluster_fit[9];
int clusters_at_once(int size, int num_sms) {
    const int known = g_cluster_fit[size].load(std::memory_order_relaxed);
    if (known > 0) return std::min(known, num_sms / size);
    static const int kOn148[9] = {0, 148, 74, 45, 33, 26, 22, 15, 15};     // what one 148-SM B200 reported
    return std::max(1, kOn148[size] * num_sms / 148);
}

// The same problem with the operands' roles exchanged: the caller's B (the weight) becomes the 128-row operand and its
// few rows of A the tile's columns; the kernel then writes the transpose of its tile (DG_TRANSPOSED_D)
Problem swapped(const Problem& p) {
    Problem q = p;
    std::swap(q.m, q.n);
    std::swap(q.a_fp4, q.b_fp4);
    std::swap(q.a_mn_major, q.b_mn_major);
    std::swap(q.gran_k_a, q.gran_k_b);
    return q;
}

// Whether a dense GEMM may run with its operands swapped (DG_FORCE_SWAP_AB: 1 = whenever this holds, -1 = never)
bool swap_allowed(const Problem& p) {
    return p.kind == DG_GEMM_DENSE && !p.a_mn_major && !p.b_mn_major && !p.accumulate &&
           !p.d_fp8 && !p.stochastic && p.reduce_batches <= 1 && p.m <= 128 && p.n >= 128 && env_int("FORCE_SWAP_AB") >= 0 &&
           env_int("FORCE_BLOCK_M") != 256 && env_int("FORCE_BLOCK_K") != 64;
}

struct Constraints {
    bool allow_cluster_split = true;
    int only_bn = 0;                  // swapped operands: the tile is as wide as the caller's M, rounded up to 16
    bool swapped = false;             // 128-row tiles, K slices only inside a cluster (the transposed epilogue's two forms)
    bool swapped_pairs = false;       // CTA pairs are candidates of the swapped form (each CTA loads half of the activations' tile)
    int block_k = 128;                // bytes of K per stage row when DG_FORCE_BLOCK_K does not say
};

int choose_config_for(const Problem& p, dg_gemm_config_t* cfg, const Constraints& lim, double* cost_out) {
    const bool allow_cluster_split = lim.allow_cluster_split;
    const int num_sms = dg_get_num_sms();
    const int d_elem = p.d_fp32 ? 4 : (p.d_fp8 ? 1 : 2);
    const int ab_elem = p.ab_bf16 ? 2 : 1;
    // bytes of K per operand row in shared memory: one per FP8 / unpacked FP4 element, two per BF16 element, half a byte
    // per element of the packed operands of kind::mxf4
    const int64_t k_row_bytes = p.mxf4 ? static_cast<int64_t>(p.k) / 2 : static_cast<int64_t>(p.k) * ab_elem;
    const int64_t k_blocks = ceil_div<int64_t>(k_row_bytes, 128);   // in units of 128 bytes of K, whatever the stage size
    const int forced_bn = env_int("FORCE_BLOCK_N"), forced_cluster = env_int("FORCE_CLUSTER"), forced_splits = env_int("FORCE_SPLIT_K");
    // DG_FORCE_SPLIT_CLUSTER: 1 = always reduce the slices of K inside a thread-block cluster, -1 = never (two kernels)
    const int forced_split_cluster = env_int("FORCE_SPLIT_CLUSTER");
    const int forced_block_m = env_int("FORCE_BLOCK_M"), forced_block_k = env_int("FORCE_BLOCK_K");
    const int forced_stages = env_int("FORCE_NUM_STAGES");

    struct Candidate {
        double cost = 0;
        int bn = 0, bk = 128, cluster = 1, halves = 1, splits = 1, kb_per_split = 0;
        bool in_cluster = false;
        int64_t tiles = 0;
        GemmLayout lay{};
    } best;
    for (int cluster = 1; cluster <= 2; ++cluster)
    for (int halves = 1; halves <= 2; ++halves)
    for (int bk = 256; bk >= 64; bk /= 2) {
        if (forced_cluster ? cluster != forced_cluster : !cluster_allowed(p, cluster)) continue;
        // (swapped: 128-row CTAs, alone or as a pair that shares the activations' tile; a pair's K is not sliced)
        if (lim.swapped && (halves != 1 || bk < 128)) continue;
        if (lim.swapped && cluster == 2 && !(forced_cluster == 2 || lim.swapped_pairs)) continue;
        // A CTA pair multiplies all its rows with one B: in the contiguous layout every expert segment must then be a
        // whole number of pair tiles
        if (cluster == 2 && (num_sms % 2 != 0 || (p.b_fp4 && p.b_mn_major) || p.kind == DG_GEMM_M_GROUPED_CONTIGUOUS_PSUM || p.kind == DG_GEMM_K_GROUPED_CONTIGUOUS ||
                             p.kind == DG_GEMM_BATCHED ||
                             (p.kind == DG_GEMM_M_GROUPED_CONTIGUOUS && state().mk_alignment % (256 * halves) != 0))) continue;
        // 256 rows per CTA: two 128-row MMAs per K-block on one B stage; K not sliced
        if (forced_block_m ? 128 * halves != forced_block_m : (halves == 2 && p.m <= 128)) continue;
        if (halves == 2 && forced_splits > 1) continue;
        // Stages of 64 elements of K (twice as many, each half the bytes): K-major FP8 operands and unsliced K only.
        // Built and tested, but it measured 0-20 % slower than 128-element stages on every shape tried (the 64-byte
        // rows double the number of L2 requests), so it is used only on request (DG_FORCE_BLOCK_K=64).
        if (bk != (forced_block_k && p.kind != DG_GEMM_K_GROUPED_CONTIGUOUS ? forced_block_k : lim.block_k)) continue;
        if (bk == 64 && (p.a_fp4 || p.b_fp4 || p.ab_bf16 || p.a_mn_major || p.b_mn_major || forced_splits > 1)) continue;
        // Stages of 256 elements of K (two swizzle atoms side by side, eight MMAs per barrier wait): the dense GEMM of
        // K-major FP8 operands with one scale per 128 elements, 128-row CTAs, K a whole number of such stages
        if (bk == 256 && (p.kind != DG_GEMM_DENSE || p.a_fp4 || p.b_fp4 || p.ab_bf16 || p.mxf4 || p.a_mn_major || p.b_mn_major || p.gran_k_a != 128 ||
                          p.gran_k_b != 128 || p.reduce_batches > 1 || cluster != 1 || halves != 1 || p.k % 256 != 0)) continue;
        const int tile_m = 128 * cluster * halves, units = num_sms / cluster;
        // A dense GEMM with at most 64 rows stages only those rows of A (16, 32 or 64; the box of its tensor map): the
        // bytes saved per stage become more stages, i.e. more of B in flight.  DG_FORCE_A_ROWS=128 keeps whole tiles.
        int a_rows = 0;
        if (p.kind == DG_GEMM_DENSE && cluster == 1 && halves == 1 && bk >= 128 && !p.a_mn_major && p.reduce_batches <= 1 && p.m <= 64 &&
            env_int("FORCE_A_ROWS") != 128)
            a_rows = p.m <= 16 ? 16 : (p.m <= 32 ? 32 : 64);
        int64_t m_blocks;
        if (p.kind == DG_GEMM_M_GROUPED_MASKED)
            m_blocks = static_cast<int64_t>(p.groups) * ceil_div(std::min(std::max(p.expected_m, 1), p.m), tile_m);
        else if (p.kind == DG_GEMM_M_GROUPED_CONTIGUOUS_PSUM && p.expected_m > 0)
            m_blocks = static_cast<int64_t>(p.groups) * ceil_div(std::min(p.expected_m, p.m), tile_m);
        else if (p.kind == DG_GEMM_M_GROUPED_CONTIGUOUS_PSUM)   // every group may end with a partly filled tile
            m_blocks = ceil_div(p.m, tile_m) + p.groups / 2;
        else if (p.kind == DG_GEMM_K_GROUPED_CONTIGUOUS)        // every group has the full tile grid and a share of K
            m_blocks = static_cast<int64_t>(p.groups) * ceil_div(p.m, tile_m);
        else if (p.kind == DG_GEMM_BATCHED)
            m_blocks = static_cast<int64_t>(p.groups) * ceil_div(p.m, tile_m);
        else
            m_blocks = ceil_div(p.m, tile_m);
        // Slicing K: dense GEMMs whose output has too few tiles to occupy the GPU.  What matters is the bytes a CTA has
        // to pull in; slicing K lets wide tiles (little re-reading of A) still spread over all SMs.  Slices hold a
        // multiple of 4 K-blocks (one packed scale word); all work items run in one wave; the second pass costs a
        // launch plus S FP32 panels of traffic.
        const bool can_split = p.kind == DG_GEMM_DENSE && !p.accumulate && !p.d_fp8 && !p.stochastic && cluster == 1 && halves == 1 && bk >= 128 &&
                               forced_splits != 1 && k_blocks >= 16;
        for (int bn = 16; bn <= (p.ab_bf16 ? 256 : 240); bn += 16) {
            if (lim.only_bn ? bn != lim.only_bn : (forced_bn && bn != forced_bn)) continue;
            // An MN-major B load starts on a 16-byte boundary of the row; for the packed 4-bit tensor-map type the
            // innermost coordinate must be a multiple of 128 elements (K-major loads start on whole K-blocks anyway)
            if (p.b_mn_major && (bn / cluster) % (p.b_fp4 ? 128 : 16) != 0) continue;
            if (p.d_fp8 && bn % 32 != 0) continue;                        // whole 32-column scale groups per tile
            const int64_t mn_tiles = m_blocks * ceil_div(p.n, bn);
            const int max_splits = can_split ? static_cast<int>(std::min<int64_t>(units / std::max<int64_t>(mn_tiles, 1), k_blocks / 8)) : 1;
            for (int want = 1; want <= std::max(1, max_splits); ++want) {
                if (forced_splits > 1 && want != std::min(forced_splits, std::max(1, max_splits))) continue;
                int splits = 1, kb_per = static_cast<int>(k_blocks);
                if (want > 1) {
                    kb_per = static_cast<int>(align_up<int64_t>(ceil_div<int64_t>(k_blocks, want), 4));
                    splits = static_cast<int>(ceil_div<int64_t>(k_blocks, kb_per));
                    if (splits != want) continue;                          // same slicing as a smaller request
                }
                // The slices of a tile either go to a workspace that a second kernel adds up, or (up to 8 of them) run as
                // the CTAs of one thread-block cluster whose first CTA adds the others' accumulators out of their shared
                // memory: no workspace, no second launch, the same sums in the same order.
                for (int in_cluster = 0; in_cluster <= (splits > 1 ? 1 : 0); ++in_cluster) {
                if (splits > 1 && forced_split_cluster != 0 && in_cluster != (forced_split_cluster > 0 ? 1 : 0)) continue;
                if (in_cluster && (!allow_cluster_split || splits > 8)) continue;
                if (lim.swapped && splits > 1 && !in_cluster) continue;
                const int64_t tiles = mn_tiles * splits;
                // Clusters are placed inside one GPC each, so fewer of them fit than SMs / size suggests
                const int64_t waves = in_cluster ? ceil_div<int64_t>(mn_tiles, clusters_at_once(splits, num_sms)) : ceil_div<int64_t>(tiles, units);
                // The pipeline: as deep as shared memory allows, but no deeper than the K-blocks of two work items
                // (k-grouped: the groups share K; an average slice stands for all of them)
                // (in bytes of K per row)
                const int64_t item_k = p.kind == DG_GEMM_K_GROUPED_CONTIGUOUS ? std::max<int64_t>(128, static_cast<int64_t>(p.k) * ab_elem / p.groups)
                                                                               : std::min<int64_t>(k_row_bytes, static_cast<int64_t>(kb_per) * 128);
                const int64_t item_kb = ceil_div<int64_t>(item_k, bk);
                int max_stages = static_cast<int>(std::max<int64_t>(2, std::min<int64_t>(32, 2 * item_kb)));
                if (forced_stages >= 2) max_stages = std::min(max_stages, forced_stages);
                GemmLayout lay{128u * halves, static_cast<uint32_t>(bn), static_cast<uint32_t>(bk), 2,
                               static_cast<uint32_t>(splits > 1 && !in_cluster ? 4 : d_elem), static_cast<uint32_t>(cluster),
                               p.b_mn_major ? 1u : 0u, static_cast<uint32_t>(p.gran_k_a), static_cast<uint32_t>(p.gran_k_b), 0u,
                               static_cast<uint32_t>(ab_elem), 2u, p.mxf4 ? 1u : 0u, static_cast<uint32_t>(a_rows)};
                const GemmLayout unfitted = lay;
                lay = fit_stages(lay, p.kind == DG_GEMM_K_GROUPED_CONTIGUOUS ? 0 : item_kb, max_stages);   // slices may be one K-block
                if (lay.num_stages <= 2 && env_int("FORCE_STORE_BUFFERS") != 2) {
                    // Two stages leave the load latency exposed: give up the second staging buffer of D if that buys a third
                    GemmLayout single = unfitted;
                    single.store_buffers = 1;
                    single = fit_stages(single, p.kind == DG_GEMM_K_GROUPED_CONTIGUOUS ? 0 : item_kb, max_stages);
                    if (single.num_stages > lay.num_stages) lay = single;
                }
                if (lay.num_stages == 0 || lay.tmem_cols_used() > kTmemCapacityCols) continue;
                // The cost model was fitted on whole-tile A stages: a shortened A stage keeps the model's choice of tile
                // and slicing and only deepens that candidate's pipeline
                uint32_t model_stages = lay.num_stages;
                if (a_rows) {
                    GemmLayout whole = unfitted;
                    whole.a_rows = 0;
                    whole.store_buffers = lay.store_buffers;
                    whole = fit_stages(whole, item_kb, max_stages);
                    if (whole.num_stages == 0) continue;
                    model_stages = whole.num_stages;
                }
                // What a CTA receives from the cluster (S slices of the columns it owns: whole 8-column chunks of 128 FP32 rows)
                // has to fit the D staging buffers and the pipeline stages behind them
                if (in_cluster && static_cast<uint64_t>(splits) * ceil_div(bn / 8, splits) * 8 * 128 * 4 >
                                      lay.off_a() + static_cast<uint64_t>(lay.num_stages) * (lay.a_bytes() + lay.b_bytes())) continue;
                // Cycles per pipeline stage: the MMAs; shared memory, which moved ~150 B per cycle in every configuration
                // measured, TMA writes and tensor-core reads together (a stage is written once, its A rows are read once
                // and its B rows once per 128-row half), and into which no configuration pulled more than ~67 B per cycle
                // from L2; and the ring of stages, `stages` of which complete per (load latency + MMA time).
                const double stage_frac = bk / 128.0;
                const double mma = 2.0 * bn * halves * stage_frac;
                const double stage_bytes = (128.0 * halves + static_cast<double>(bn) / cluster) * bk;
                // (with a CTA pair the peer's tensor core reads this CTA's half of B as well)
                const double read_bytes = (128.0 * halves + halves * static_cast<double>(bn) / cluster * (cluster == 2 ? 2.0 : 1.0)) * bk;
                // (55 B per cycle fitted the cluster-reduced candidates: few-tile shapes whose B is read once, from HBM)
                const double smem_feed = std::max((stage_bytes + read_bytes) / 150.0, stage_bytes / (in_cluster ? 55.0 : 67.0));
                const double ring = (1500.0 + mma) / model_stages;
                // (one epilogue warpgroup drains a 128 x bn accumulator in ~600 + 14 bn cycles, measured on the K = 512 shape
                //  with 128-row CTA pairs, where it is what bounds a tile)
                const double epilogue = cluster == 2 && halves == 1 ? 600.0 + 14.0 * bn
                                                                    : 300.0 + 150.0 * lay.num_groups() + 20.0 * lay.num_stores() + bn * 2.0;
                // The epilogue of a tile overlaps the next tile's main loop; it is exposed once per CTA
                // + ~1500 cycles per tile that do not shrink with K (tile hand-over, first loads of a new tile), measured
                // on the K = 512 and K = 1536 shapes
                // (700 for 128-row CTA pairs, whose tile hand-over was measured on the K = 1536 and K = 2048 shapes)
                const double per_tile = static_cast<double>(item_kb) * std::max(mma, std::max(smem_feed, ring)) + (cluster == 2 && halves == 1 ? 700.0 : 1500.0);
                double cost = static_cast<double>(waves) * std::max(per_tile, epilogue) + epilogue + 2000.0;
                // 256-row tiles have no spare accumulator: the next tile's MMAs start once the epilogue warpgroups have
                // moved their rows from tensor memory into registers (~1400 cycles, measured)
                if (halves == 2) cost = static_cast<double>(waves) * (per_tile + 1400.0) + epilogue + 2000.0;
                if (splits > 1 && !in_cluster)   // second launch + reading S panels and writing D at a few TB/s (~2000 B per SM clock over the GPU)
                    cost += 6000.0 + static_cast<double>(splits + 1) * p.m * p.n * 4.0 / 2000.0;
                if (in_cluster)                  // parking a tile, the cluster barrier, bn loads per thread across the cluster
                    cost += 600.0 * splits + 20.0 * bn;     // (fitted to a sweep over sizes and widths on six decode shapes)
                if (best.bn == 0 || cost < best.cost - 1e-9 || (std::abs(cost - best.cost) <= 1e-9 && bn > best.bn)) {
                    best.cost = cost;
                    best.bn = bn; best.bk = bk; best.cluster = cluster; best.halves = halves;
                    best.tiles = tiles; best.splits = splits; best.kb_per_split = kb_per;
                    best.in_cluster = in_cluster != 0;
                    best.lay = lay;
                }
                }
            }
        }
    }
    if (best.bn == 0 && lim.swapped) return DG_ERR_UNSUPPORTED;
    if (best.bn == 0)
        return fail(DG_ERR_INVALID_ARGUMENT, "no tile configuration: DG_FORCE_BLOCK_N must be a multiple of 16 in [16, 240], "
                                             "DG_FORCE_CLUSTER 1 or 2 (2 needs an even SM count and, for the contiguous layout, expert segments aligned to the pair's rows), "
                                             "DG_FORCE_BLOCK_M 128 or 256 (256 only with K not sliced), "
                                             "DG_FORCE_BLOCK_K 64, 128 or 256 (64 only for K-major FP8 operands and K not sliced; 256 only for dense K-major FP8 GEMMs with "
                                             "one scale per 128 elements and K a multiple of 256)");

    const int units = num_sms / best.cluster;
    cfg->num_splits = best.splits;
    cfg->kb_per_split = best.kb_per_split;
    cfg->block_m = 128 * best.halves;
    cfg->block_n = best.bn;
    cfg->block_k = best.bk;
    cfg->num_stages = static_cast<int>(best.lay.num_stages);
    cfg->cluster_size = best.cluster;
    const int forced_raster = env_int("FORCE_RASTER_GROUP");
    cfg->raster_group = forced_raster > 0 ? forced_raster : std::max(4, 16 / (best.cluster * best.halves));
    cfg->split_in_cluster = best.in_cluster ? 1 : 0;
    cfg->swap_ab = lim.swapped ? 1 : 0;
    if (cost_out != nullptr) *cost_out = best.cost;
    cfg->num_ctas = best.in_cluster ? static_cast<int>(best.tiles) :
                    best.cluster * (p.kind == DG_GEMM_M_GROUPED_MASKED || p.kind == DG_GEMM_M_GROUPED_CONTIGUOUS_PSUM
                                        ? units : static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(units, best.tiles))));
    cfg->store_buffers = static_cast<int>(best.lay.store_buffers);
    cfg->a_rows = static_cast<int>(best.lay.a_stage_rows());
    cfg->smem_bytes = static_cast<int>(best.lay.total_bytes());
    cfg->tmem_cols = static_cast<int>(best.lay.tmem_cols_alloc());
    cfg->num_tiles = static_cast<int>(best.tiles);
    cfg->waves_x100 = static_cast<int>(best.tiles * 100 / units);
    return DG_OK;
}

// The configuration of a problem: the cheaper of the direct form and, for dense GEMMs with few rows, the form with the
// operands swapped.  Sizes in the result are the kernel's (block_m rows of the weight, block_n = the caller's M rounded up).
int choose_config(const Problem& p, dg_gemm_config_t* cfg, bool allow_cluster_split = true) {
    Constraints direct;
    direct.allow_cluster_split = allow_cluster_split;
    double direct_cost = 0;
    const int forced_swap = env_int("FORCE_SWAP_AB");
    const int rc = choose_config_for(p, cfg, direct, &direct_cost);
    if (!swap_allowed(p) || !allow_cluster_split) return rc;
    // Measured on 28 (M, N, K) points: up to 32 rows the swapped form wins wherever the cost model prefers it (by 5-30 %).
    // From 33 to 64 rows the two are closer (the swapped tile carries as many activation bytes as weight bytes per
    // column): there the swapped form has to be modelled 7 % cheaper, which on the six benchmark shapes at M = 64 picks
    // it where it measured 1-7 % faster and not where it measured 3 % slower.  Above 64 rows (up to 128) on request only.
    if (forced_swap <= 0 && p.m > 64) return rc;
    Constraints lim;
    lim.swapped = true;
    lim.only_bn = static_cast<int>(align_up<int64_t>(p.m, 16));
    dg_gemm_config_t other{};
    double other_cost = 0;
    if (choose_config_for(swapped(p), &other, lim, &other_cost) != DG_OK) return rc;
    if (env_int("PRINT_CONFIGS"))
        fprintf(stderr, "[dg] m %d n %d k %d: modelled cycles direct %.0f (block_n %d x%d), operands swapped %.0f (x%d)\n", p.m, p.n, p.k,
                direct_cost, cfg->block_n, cfg->num_splits, other_cost, other.num_splits);
    // (up to 16 rows the swapped form was the faster or an equal one on all 14 shapes timed, also where the model's wave
    // count speaks against its many small tiles)
    if (rc != DG_OK || forced_swap > 0 || p.m <= 16 || other_cost < direct_cost * (p.m > 32 ? 0.93 : 1.0)) {
        *cfg = other;
        // Tiles of 16 or 32 columns spend more time on the MMA warp's walk around its loop than on the MMAs: where a work
        // item has at least 12 K-blocks, stages of 256 elements of K (half as many walks; measured 2-4 % faster on the
        // benchmark shapes, equal or slower with shorter items) replace the 128-element ones, everything else unchanged
        const int item_kb = other.num_splits > 1 ? other.kb_per_split : static_cast<int>(ceil_div<int64_t>(p.k, 128));
        if (p.m <= 32 && item_kb >= 12 && env_int("FORCE_BLOCK_K") == 0) {
            Constraints wide = lim;
            wide.block_k = 256;
            dg_gemm_config_t longer{};
            if (choose_config_for(swapped(p), &longer, wide, nullptr) == DG_OK && longer.num_splits == other.num_splits &&
                longer.split_in_cluster == other.split_in_cluster && longer.num_stages >= 4)
                *cfg = longer;
        }
        return DG_OK;
    }
    return rc;
}

// The layout the kernel of a configuration uses (same arithmetic as choose_config)
GemmLayout layout_of(const Problem& p, const dg_gemm_config_t& cfg) {
    const bool split = cfg.num_splits > 1 && !cfg.split_in_cluster;
    const int64_t ab_elem = p.ab_bf16 ? 2 : 1;
    const int64_t k_row_bytes = p.mxf4 ? p.k / 2 : p.k * ab_elem;
    const int64_t item_kb = p.kind == DG_GEMM_K_GROUPED_CONTIGUOUS ? 0 :
                            ceil_div<int64_t>(std::min<int64_t>(k_row_bytes, static_cast<int64_t>(cfg.kb_per_split) * 128), cfg.block_k);
    GemmLayout lay{static_cast<uint32_t>(cfg.block_m), static_cast<uint32_t>(cfg.block_n), static_cast<uint32_t>(cfg.block_k),
                   static_cast<uint32_t>(cfg.num_stages), static_cast<uint32_t>((p.d_fp32 || split) ? 4 : (p.d_fp8 ? 1 : 2)),
                   static_cast<uint32_t>(cfg.cluster_size), p.b_mn_major ? 1u : 0u,
                   static_cast<uint32_t>(p.gran_k_a), static_cast<uint32_t>(p.gran_k_b),
                   item_kb < cfg.num_stages ? 1u : 0u, static_cast<uint32_t>(ab_elem), static_cast<uint32_t>(cfg.store_buffers),
                   p.mxf4 ? 1u : 0u, cfg.a_rows > 0 && cfg.a_rows < cfg.block_m ? static_cast<uint32_t>(cfg.a_rows) : 0u};
    return lay;
}

std::string generate_source(const Problem& p, const dg_gemm_config_t& cfg) {
    std::ostringstream s;
    s << "// generated: block-scaled GEMM instantiation\n"
      << "#define DG_GEMM_TYPE " << p.kind << "\n"
      << "#define DG_M_HALVES " << cfg.block_m / 128 << "\n"
      << "#define DG_BLOCK_N " << cfg.block_n << "\n"
      << "#define DG_BLOCK_K " << cfg.block_k << "\n"
      << "#define DG_SHORT_K " << layout_of(p, cfg).short_k << "\n"
      << "#define DG_NUM_STAGES " << cfg.num_stages << "\n"
      << "#define DG_CLUSTER " << cfg.cluster_size << "\n"
      << "#define DG_AB_BF16 " << (p.ab_bf16 ? 1 : 0) << "\n"
      << "#define DG_A_FP4 " << (p.a_fp4 ? 1 : 0) << "\n"
      << "#define DG_B_FP4 " << (p.b_fp4 ? 1 : 0) << "\n"
      << "#define DG_MXF4 " << (p.mxf4 ? 1 : 0) << "\n"
      << "#define DG_MAJOR_A " << (p.a_mn_major ? 1 : 0) << "\n"
      << "#define DG_MAJOR_B " << (p.b_mn_major ? 1 : 0) << "\n"
      << "#define DG_GRAN_K_A " << p.gran_k_a << "\n"
      << "#define DG_GRAN_K_B " << p.gran_k_b << "\n"
      << "#define DG_D_FP32 " << ((p.d_fp32 || (cfg.num_splits > 1 && !cfg.split_in_cluster)) ? 1 : 0) << "\n"
      << "#define DG_D_FP8 " << (p.d_fp8 ? 1 : 0) << "\n"
      << "#define DG_STOCHASTIC_ROUNDING " << (p.stochastic ? 1 : 0) << "\n"
      << "#define DG_ACCUMULATE " << (p.accumulate ? 1 : 0) << "\n"
      << "#define DG_RASTER_GROUP " << cfg.raster_group << "\n"
      << "#define DG_SPLIT_K " << (cfg.num_splits > 1 && !cfg.split_in_cluster ? 1 : 0) << "\n"
      << "#define DG_STORE_BUFFERS " << cfg.store_buffers << "\n"
      << "#define DG_A_ROWS " << (cfg.a_rows > 0 && cfg.a_rows < cfg.block_m ? cfg.a_rows : 0) << "\n"
      << "#define DG_TRANSPOSED_D " << (cfg.swap_ab ? 1 : 0) << "\n"
      << "#define DG_BATCH_REDUCE " << (p.reduce_batches > 1 ? 1 : 0) << "\n"
      << "#define DG_SPLIT_CLUSTER " << (cfg.split_in_cluster ? cfg.num_splits : 1) << "\n"
      << "#define DG_WRITE_PADDING " << (p.write_padding ? 1 : 0) << "\n"
      << "#define DG_K_PSUM " << (p.k_psum ? 1 : 0) << "\n"
      << "#define DG_PROFILE " << env_int("PROFILE") << "\n"
      << "#define DG_EPILOGUE_BACKOFF_NS " << env_int("EPILOGUE_BACKOFF_NS", 0) << "\n"
      << "#define DG_MMA_WHOLE_WARP " << env_int("MMA_WHOLE_WARP", 1) << "\n"
      << "#define DG_PRODUCER_WHOLE_WARP " << env_int("PRODUCER_WHOLE_WARP", 1) << "\n"
      << "#define DG_L2_HINT " << env_int("L2_HINT", 0) << "\n"
      << "#include <dg/gemm_fp8_fp4.cuh>\n";
    return s.str();
}

// A tiled tensor map over [outer][inner] elements (row pitch outer_stride_bytes) or, with batches > 0, over
// [batches][outer][inner] with the batches batch_stride_bytes apart and a box one batch deep.
int encode_2d(CUtensorMap* map, CUtensorMapDataType dtype, const void* base, uint64_t inner, uint64_t outer,
              uint64_t outer_stride_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swizzle,
              uint64_t batches = 0, uint64_t batch_stride_bytes = 0) {
    // Encoding costs the driver ~1 us per map and a GEMM needs six; serving loops call with the same buffers over and
    // over, so the last maps are kept per thread (a map depends on nothing but these arguments)
    struct Key {
        const void* base; uint64_t inner, outer, outer_stride, batches, batch_stride; uint32_t box_inner, box_outer; int dtype, swizzle;
        bool operator==(const Key& o) const {
            return base == o.base && inner == o.inner && outer == o.outer && outer_stride == o.outer_stride && batches == o.batches &&
                   batch_stride == o.batch_stride && box_inner == o.box_inner && box_outer == o.box_outer && dtype == o.dtype && swizzle == o.swizzle;
        }
    };
    struct Slot { Key key; CUtensorMap map; bool valid = false; };
    constexpr size_t kSlots = 256;
    thread_local std::array<Slot, kSlots> cache;
    const Key key{base, inner, outer, outer_stride_bytes, batches, batch_stride_bytes, box_inner, box_outer, static_cast<int>(dtype),
                  static_cast<int>(swizzle)};
    const size_t h = (reinterpret_cast<uintptr_t>(base) >> 4) * 0x9E3779B97F4A7C15ull + inner * 31 + outer * 131 + box_inner * 7 + box_outer * 3 +
                     static_cast<size_t>(dtype) * 1009 + static_cast<size_t>(swizzle) * 9176 + outer_stride_bytes + batch_stride_bytes * 17;
    Slot& slot = cache[(h >> 20) % kSlots];
    const bool verbose = env_int("PRINT_CONFIGS") != 0;
    if (slot.valid && slot.key == key && !verbose) {
        *map = slot.map;
        return DG_OK;
    }
    const Driver& drv = driver();
    if (!drv.ok) return fail(DG_ERR_CUDA, "CUDA driver unavailable: %s", drv.why.c_str());
    const cuuint32_t rank = batches > 0 ? 3 : 2;
    const cuuint64_t dims[3] = {inner, outer, batches};
    const cuuint64_t strides[2] = {outer_stride_bytes, batch_stride_bytes};
    const cuuint32_t box[3] = {box_inner, box_outer, 1};
    const cuuint32_t elem_strides[3] = {1, 1, 1};
    if (verbose)
        fprintf(stderr, "[dg] tensor map: dtype %d dims (%llu, %llu, %llu) strides %llu, %llu B box (%u, %u) swizzle %d base %p\n",
                static_cast<int>(dtype), static_cast<unsigned long long>(inner), static_cast<unsigned long long>(outer),
                static_cast<unsigned long long>(batches), static_cast<unsigned long long>(outer_stride_bytes),
                static_cast<unsigned long long>(batch_stride_bytes), box_inner, box_outer, static_cast<int>(swizzle), base);
    const CUresult r = drv.cuTensorMapEncodeTiled(map, dtype, rank, const_cast<void*>(base), dims, strides, box, elem_strides,
                                                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(DG_ERR_CUDA, "cuTensorMapEncodeTiled failed: %s (dims %llu x %llu x %llu, strides %llu, %llu, box %u x %u)",
                    cu_error(r).c_str(), static_cast<unsigned long long>(inner), static_cast<unsigned long long>(outer),
                    static_cast<unsigned long long>(batches), static_cast<unsigned long long>(outer_stride_bytes),
                    static_cast<unsigned long long>(batch_stride_bytes), box_inner, box_outer);
    slot.key = key;
    slot.map = *map;
    slot.valid = true;
    return DG_OK;
}

int get_kernel(const Problem& p, const dg_gemm_config_t& cfg, dg_kernel_t* kernel) {
    static const char* names[6] = {"gemm_fp8_fp4_dense", "gemm_fp8_fp4_m_grouped_contiguous", "gemm_fp8_fp4_m_grouped_masked",
                                   "gemm_fp8_fp4_m_grouped_contiguous_psum", "gemm_fp8_fp4_k_grouped_contiguous", "gemm_fp8_fp4_batched"};
    const std::string src = generate_source(cfg.swap_ab ? swapped(p) : p, cfg);
    return dg_jit_compile(names[p.kind], "dg_gemm_fp8_fp4", src.c_str(), "", kernel);
}

// Choosing a configuration walks a few hundred candidates and finding its kernel hashes the generated source: ~15 us
// together, more than the kernel time of a decode-sized GEMM.  Both depend only on the problem's descriptor and the
// settings, so the pair is remembered per descriptor (bounded: cleared when it grows past a few thousand shapes).
struct Plan {
    dg_gemm_config_t cfg;
    dg_kernel_t kernel;
};

int get_plan(const Problem& p, Plan* plan) {
    static const char* kEnvNames[] = {"FORCE_BLOCK_N", "FORCE_CLUSTER", "FORCE_SPLIT_K", "FORCE_BLOCK_M", "FORCE_BLOCK_K",
                                      "FORCE_NUM_STAGES", "FORCE_RASTER_GROUP", "PROFILE", "FORCE_SPLIT_CLUSTER", "FORCE_SWAP_AB", "FORCE_STORE_BUFFERS", "FORCE_A_ROWS",
                                      "EPILOGUE_BACKOFF_NS", "MMA_WHOLE_WARP", "PRODUCER_WHOLE_WARP", "L2_HINT"};
    const int fields[] = {p.kind, p.m, p.n, p.k, p.groups, static_cast<int>(p.a_fp4), static_cast<int>(p.b_fp4), static_cast<int>(p.ab_bf16),
                          static_cast<int>(p.d_fp32), static_cast<int>(p.d_fp8), static_cast<int>(p.accumulate), static_cast<int>(p.a_mn_major),
                          static_cast<int>(p.b_mn_major), p.gran_k_a, p.gran_k_b, p.expected_m, static_cast<int>(p.write_padding),
                          static_cast<int>(p.k_psum), static_cast<int>(p.stochastic), p.reduce_batches > 1 ? 1 : 0, dg_get_num_sms(), state().mk_alignment,
                          static_cast<int>(p.mxf4)};
    // The key is sized from what goes into it: every field of the descriptor and every setting the choice reads
    constexpr size_t kNumFields = sizeof(fields) / sizeof(fields[0]), kNumEnv = sizeof(kEnvNames) / sizeof(kEnvNames[0]);
    using PlanKey = std::array<int, kNumFields + kNumEnv>;
    PlanKey key{};
    size_t i = 0;
    for (int v : fields) key[i++] = v;
    for (const char* name : kEnvNames) key[i++] = env_int(name, -12345);       // (unset differs from every value)
    static_assert(std::tuple_size<PlanKey>::value == kNumFields + kNumEnv, "one slot per field and setting");
    static std::mutex mu;
    static std::map<PlanKey, Plan> plans;
    {
        std::lock_guard<std::mutex> lock(mu);
        auto it = plans.find(key);
        if (it != plans.end()) {
            *plan = it->second;
            return DG_OK;
        }
    }
    int rc = choose_config(p, &plan->cfg);
    if (rc != DG_OK) return rc;
    if ((rc = get_kernel(p, plan->cfg, &plan->kernel)) != DG_OK) return rc;
    // The slices of a tile as one cluster: ask the driver how many such clusters the device holds at once.  Clusters
    // beyond that simply run later (nothing waits across clusters), but the choice assumed one wave: when the driver's
    // number is smaller than the guess, choose again with the number known (each size is asked once per process).
    for (int attempt = 0; attempt < 8 && plan->cfg.split_in_cluster; ++attempt) {
        const int size = plan->cfg.num_splits;
        if (g_cluster_fit[size].load(std::memory_order_relaxed) > 0) break;
        int fit = 0;
        rc = dg_jit_max_active_clusters(plan->kernel, 128 + plan->cfg.block_m, size, plan->cfg.smem_bytes, &fit);
        if (env_int("PRINT_CONFIGS"))
            fprintf(stderr, "[dg] clusters of %d CTAs that fit at once: %d (status %d)\n", size, fit, rc);
        const bool usable = rc == DG_OK && fit >= 1;
        const int guessed = clusters_at_once(size, dg_get_num_sms());
        if (usable) g_cluster_fit[size].store(fit, std::memory_order_relaxed);
        if (usable && fit >= guessed) break;
        if ((rc = choose_config(p, &plan->cfg, usable)) != DG_OK) return rc;
        if ((rc = get_kernel(p, plan->cfg, &plan->kernel)) != DG_OK) return rc;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (plans.size() > 4096) plans.clear();
    plans[key] = *plan;
    return DG_OK;
}

// `fixed_scratch`, when given, replaces the library-owned split-K workspace with a caller-provided device buffer of
// fixed size and turns off everything else that would allocate (the status word is used only if it already exists).
struct FixedScratch {
    float* ptr;
    size_t bytes;
};

int run_gemm(int kind, const dg_gemm_args_t* a, const FixedScratch* fixed_scratch = nullptr) {
    DG_REQUIRE_ALIVE();
    env_refresh();
    Problem p;
    int rc = validate(kind, a, true, &p);
    if (rc != DG_OK) return rc;
    if (p.m == 0 || p.n == 0) return DG_OK;
    if (p.k == 0) return fail(DG_ERR_INVALID_ARGUMENT, "k == 0 must be handled by the caller (zero or copy D)");

    Plan plan;
    if ((rc = get_plan(p, &plan)) != DG_OK) return rc;
    const dg_gemm_config_t& cfg = plan.cfg;
    dg_kernel_t kernel = plan.kernel;
    // Operands swapped: from here on "A" is the caller's B and the other way round; D stays the caller's, which the
    // kernel writes transposed
    dg_gemm_args_t exchanged;
    if (cfg.swap_ab) {
        exchanged = *a;
        std::swap(exchanged.a, exchanged.b);
        std::swap(exchanged.sfa, exchanged.sfb);
        std::swap(exchanged.m, exchanged.n);
        std::swap(exchanged.a_dtype, exchanged.b_dtype);
        std::swap(exchanged.major_a, exchanged.major_b);
        std::swap(exchanged.lda, exchanged.ldb);
        std::swap(exchanged.sfa_pitch, exchanged.sfb_pitch);
        std::swap(exchanged.gran_k_a, exchanged.gran_k_b);
        a = &exchanged;
        p = swapped(p);
    }
    if (env_int("PRINT_CONFIGS"))
        fprintf(stderr, "[dg] kind %d m %d n %d k %d groups %d -> block_m %d block_n %d block_k %d cluster %d stages %d store_buffers %d a_rows %d ctas %d smem %d tiles %d splits %d x %d%s\n",
                kind, p.m, p.n, p.k, p.groups, cfg.block_m, cfg.block_n, cfg.block_k, cfg.cluster_size, cfg.num_stages, cfg.store_buffers, cfg.a_rows, cfg.num_ctas, cfg.smem_bytes, cfg.num_tiles,
                cfg.num_splits, cfg.kb_per_split, cfg.split_in_cluster ? " (in a cluster)" : "");
    if (fixed_scratch == nullptr && (rc = ensure_status_word()) != DG_OK) return rc;

    const bool split = cfg.num_splits > 1 && !cfg.split_in_cluster;     // through the workspace and a second kernel
    const int launch_cluster = cfg.split_in_cluster ? cfg.num_splits : cfg.cluster_size;
    const bool kernel_d_fp32 = p.d_fp32 || split;
    const GemmLayout lay = layout_of(p, cfg);
    // Split-K: the kernel's D is the workspace, num_splits panels of [align(m, 128)][align(n, 4)] FP32
    float* workspace = nullptr;
    const int64_t panel_rows = align_up<int64_t>(p.m, 128), ld_ws = align_up<int64_t>(p.n, 4);
    const size_t workspace_bytes = split ? static_cast<size_t>(cfg.num_splits) * panel_rows * ld_ws * sizeof(float) : 0;
    if (split && fixed_scratch != nullptr) {
        if (workspace_bytes > fixed_scratch->bytes)
            return fail(DG_ERR_INVALID_ARGUMENT,
                        "this GEMM (m %d, n %d, k %d) is sliced %d ways along K and needs %zu bytes of scratch, more than the %zu bytes "
                        "of the built-in buffer: call dg_fp8_fp4_gemm instead, or set DG_FORCE_SPLIT_K=1 to run it unsliced",
                        p.m, p.n, p.k, cfg.num_splits, workspace_bytes, fixed_scratch->bytes);
        workspace = fixed_scratch->ptr;
    } else if (split && (rc = split_workspace(workspace_bytes, &workspace)) != DG_OK) {
        return rc;
    }
    const bool k_grouped = kind == DG_GEMM_K_GROUPED_CONTIGUOUS;
    const uint64_t a_rows = kind == DG_GEMM_M_GROUPED_MASKED ? static_cast<uint64_t>(p.groups) * p.m : p.m;
    // k-grouped: one B for all groups (the group selects a slice of K); every group starts a new packed scale row
    const bool one_b = k_grouped || kind == DG_GEMM_BATCHED;        // (batched: the batch is a dimension of its own)
    const uint64_t b_rows = one_b ? p.n : static_cast<uint64_t>(p.groups) * p.n;
    const uint64_t b_k_rows = one_b ? p.k : static_cast<uint64_t>(p.groups) * p.k;
    const uint64_t sfa_k = ceil_div(p.k, p.gran_k_a * 4), sfb_k = ceil_div(p.k, p.gran_k_b * 4);
    const uint64_t sfa_rows = kind == DG_GEMM_M_GROUPED_MASKED ? sfa_k * p.groups : (k_grouped ? sfa_k + p.groups : sfa_k);
    const uint64_t sfb_rows = k_grouped ? sfb_k + p.groups : (kind == DG_GEMM_BATCHED ? sfb_k : sfb_k * p.groups);

    // Batched: every map gets the batch as a third dimension (strides in bytes)
    const bool batched = kind == DG_GEMM_BATCHED;
    const bool reduce = p.reduce_batches > 1;               // A and B get the batch as a third coordinate, D does not
    const uint64_t nb = batched ? p.groups : 0;
    const uint64_t nb_ab = reduce ? p.reduce_batches : nb;
    const uint64_t k_inner = reduce ? p.k / p.reduce_batches : p.k;
    const uint64_t d_elem_bytes = p.d_fp32 ? 4 : (p.d_fp8 ? 1 : 2);
    const uint64_t bs_a = batched || reduce ? a->batch_stride_a : 0, bs_b = batched || reduce ? a->batch_stride_b : 0;
    const uint64_t bs_d = batched ? a->batch_stride_d * d_elem_bytes : 0;
    const uint64_t bs_sfa = batched ? a->sfa_pitch * 4 * ceil_div(p.k, p.gran_k_a * 4) : 0;
    const uint64_t bs_sfb = batched ? a->sfb_pitch * 4 * ceil_div(p.k, p.gran_k_b * 4) : 0;
    CUtensorMap tm_a, tm_b, tm_sfa, tm_sfb, tm_d, tm_d_full;
    // K-major A, B: K (elements) x rows; box = one K-block (at most 128 bytes of it) x the tile's rows, swizzled over its width.
    const CUtensorMapSwizzle k_major_swizzle = cfg.block_k >= 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
    // MN-major (FP8 only): MN x (groups x K); box = 128 columns of MN x one K-block.
    // BF16 operands: two bytes per element, so a 128-byte stage row is 64 elements and an MN-major atom 64 columns
    const uint64_t ab_elem = p.ab_bf16 ? 2 : 1;
    // (a 256-byte stage is filled by two boxes of 128)
    const uint32_t box_k = static_cast<uint32_t>(std::min(cfg.block_k, 128) / ab_elem), atom_mn = static_cast<uint32_t>(128 / ab_elem);
    const CUtensorMapDataType a_type = p.ab_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 :
                                       p.a_fp4 ? CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    const CUtensorMapDataType b_type = p.ab_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 :
                                       p.b_fp4 ? CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    if (p.mxf4) {
        // packed operands as plain byte matrices [rows, K / 2]: a 128-byte box row is 256 elements of K
        if ((rc = encode_2d(&tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, a->a, p.k / 2, a_rows, a->lda, 128, lay.a_stage_rows(), CU_TENSOR_MAP_SWIZZLE_128B)) != DG_OK) return rc;
    } else if (!p.a_mn_major) {
        if ((rc = encode_2d(&tm_a, a_type, a->a, k_inner, a_rows, a->lda * ab_elem, box_k, lay.a_stage_rows(), k_major_swizzle,
                            nb_ab, bs_a * ab_elem)) != DG_OK) return rc;
    } else {
        if ((rc = encode_2d(&tm_a, a_type, a->a, p.m, p.k, a->lda * ab_elem, atom_mn, box_k, CU_TENSOR_MAP_SWIZZLE_128B,
                            nb, bs_a * ab_elem)) != DG_OK) return rc;
    }
    if (p.mxf4) {
        if ((rc = encode_2d(&tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, a->b, p.k / 2, b_rows, a->ldb, 128, cfg.block_n / cfg.cluster_size,
                            CU_TENSOR_MAP_SWIZZLE_128B)) != DG_OK) return rc;
    } else if (!p.b_mn_major) {
        if ((rc = encode_2d(&tm_b, b_type, a->b, k_inner, b_rows, a->ldb * ab_elem, box_k, cfg.block_n / cfg.cluster_size, k_major_swizzle,
                            nb_ab, bs_b * ab_elem)) != DG_OK) return rc;
    } else {
        if ((rc = encode_2d(&tm_b, b_type, a->b, p.n, b_k_rows, a->ldb * ab_elem, atom_mn, box_k, CU_TENSOR_MAP_SWIZZLE_128B,
                            nb, bs_b * ab_elem)) != DG_OK) return rc;
    }
    // Scales: MN (int32) x packed-K rows; the MN extent is the true row count, so reads past it are zero-filled
    if (p.ab_bf16) {
        tm_sfa = tm_sfb = tm_a;                  // never used: the BF16 kernel has no scale loads
    } else {
        // (one packed word per row and K-block, two for the 256-element stages of kind::mxf4)
        if ((rc = encode_2d(&tm_sfa, CU_TENSOR_MAP_DATA_TYPE_INT32, a->sfa, p.m, sfa_rows, a->sfa_pitch * 4, cfg.block_m, lay.sfa_words(),
                            CU_TENSOR_MAP_SWIZZLE_NONE, nb, bs_sfa)) != DG_OK) return rc;
        if ((rc = encode_2d(&tm_sfb, CU_TENSOR_MAP_DATA_TYPE_INT32, a->sfb, p.n, sfb_rows, a->sfb_pitch * 4, lay.sf_block_n(), lay.sfb_words(),
                            CU_TENSOR_MAP_SWIZZLE_NONE, nb, bs_sfb)) != DG_OK) return rc;
    }
    const CUtensorMapSwizzle d_swizzle = lay.store_row_bytes() == 128 ? CU_TENSOR_MAP_SWIZZLE_128B :
                                         lay.store_row_bytes() == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
    // Two views of D: boxes as wide as an epilogue group (128 or 64 bytes) for complete groups, narrower boxes for the
    // ragged end of a tile row
    const CUtensorMapDataType d_type = kernel_d_fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 :
                                       p.d_fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    void* d_base = split ? static_cast<void*>(workspace) : a->d;
    const uint64_t d_rows = split ? static_cast<uint64_t>(cfg.num_splits) * panel_rows :
                            (k_grouped ? static_cast<uint64_t>(p.groups) * p.m : a_rows);
    const uint64_t d_pitch_bytes = split ? ld_ws * 4 : a->ldd * (p.d_fp32 ? 4 : (p.d_fp8 ? 1 : 2));
    if (cfg.swap_ab) {
        // The transposed epilogue stages [rows of the caller's D][128 of its columns] blocks (plain row-major, as many rows
        // as the D staging buffers hold) and stores them through this map: the caller's D as it is, N (here p.m) contiguous.
        // K slices reduced inside a cluster write D directly and do not use it.
        const uint64_t d_elem = p.d_fp32 ? 4 : 2;
        const uint32_t t_rows = static_cast<uint64_t>(cfg.block_n) * 128 * d_elem <= lay.off_a()
                                    ? static_cast<uint32_t>(cfg.block_n) : static_cast<uint32_t>(lay.off_a() / (128 * d_elem) / 16 * 16);
        if ((rc = encode_2d(&tm_d, d_type, a->d, p.m, p.n, a->ldd * d_elem, 128, t_rows, CU_TENSOR_MAP_SWIZZLE_NONE)) != DG_OK) return rc;
        tm_d_full = tm_d;
    } else {
        if ((rc = encode_2d(&tm_d, d_type, d_base, p.n, d_rows, d_pitch_bytes, lay.store_cols(), 128, d_swizzle, nb, bs_d)) != DG_OK) return rc;
        if ((rc = encode_2d(&tm_d_full, d_type, d_base, p.n, d_rows, d_pitch_bytes, lay.group_cols(), 128,
                            lay.group_bytes() == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, nb, bs_d)) != DG_OK)
            return rc;
    }

    GemmParams params;
    params.grouped_layout = a->grouped_layout;
    params.d = split ? static_cast<void*>(workspace) : a->d;
    params.status = state().status_device;
    params.shape_m = p.m; params.shape_n = p.n; params.shape_k = p.k;
    params.num_groups = p.groups;
    params.ldd = static_cast<uint32_t>(split ? ld_ws : a->ldd);
    const float alpha = a->has_alpha ? a->alpha : 1.0f;
    params.alpha = split ? 1.0f : alpha;              // split-K applies alpha in the reduction pass
    params.profile = nullptr;
    params.num_splits = split ? cfg.num_splits : 1;
    params.kb_per_split = cfg.block_k > 128 ? cfg.kb_per_split * 128 / cfg.block_k : cfg.kb_per_split;    // the kernel counts stages
    params.split_panel_rows = static_cast<uint32_t>(panel_rows);
    params.group_alignment = static_cast<uint32_t>(state().mk_alignment);
    params.sfd = static_cast<uint32_t*>(a->sfd);
    params.sfd_pitch = static_cast<uint32_t>(a->sfd_pitch);
    params.kb_per_batch = static_cast<uint32_t>(k_inner * ab_elem / cfg.block_k);
    void* kargs[7] = {&tm_a, &tm_b, &tm_sfa, &tm_sfb, &tm_d, &tm_d_full, &params};
    if (env_int("PROFILE") && fixed_scratch == nullptr) {
        // synchronous, printing path for tuning only (it allocates its counters and waits for the stream, so the entry
        // point that must not allocate runs the kernel without counters instead)
        params.profile = profile_buffer();
        if (params.profile == nullptr) return fail(DG_ERR_CUDA, "cannot allocate the profile buffer");
        DG_CUDA_RT(cudaMemsetAsync(params.profile, 0, 32 * sizeof(unsigned long long), static_cast<cudaStream_t>(a->stream)));
        DG_CUDA_RT(cudaMemsetAsync(params.profile + 16 + 9, 0xFF, sizeof(unsigned long long), static_cast<cudaStream_t>(a->stream)));   // (a minimum)
        rc = dg_jit_launch(kernel, cfg.num_ctas, 128 + cfg.block_m, launch_cluster, cfg.smem_bytes, state().pdl, a->stream, kargs);
        if (rc != DG_OK) return rc;
        unsigned long long h[32];
        DG_CUDA_RT(cudaMemcpyAsync(h, params.profile, sizeof(h), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(a->stream)));
        DG_CUDA_RT(cudaStreamSynchronize(static_cast<cudaStream_t>(a->stream)));
        const double ctas = cfg.num_ctas, leaders = ctas / cfg.cluster_size;
        fprintf(stderr, "[dg profile] cycles per CTA: producer wait_empty %.0f / %.0f | mma wait_full %.0f wait_tmem_empty %.0f "
                        "issue cp %.0f mma %.0f commit %.0f fence %.0f tail %.0f / %.0f | sf wait %.0f / %.0f | epilogue wait_tmem_full %.0f store_wait %.0f / %.0f\n",
                h[0] / ctas, h[1] / ctas, h[2] / leaders, h[3] / leaders, h[10] / leaders, h[11] / leaders, h[12] / leaders,
                h[13] / leaders, h[14] / leaders, h[4] / leaders, h[5] / ctas, h[6] / ctas, h[7] / ctas, h[9] / ctas, h[8] / ctas);
        const auto since_entry = [&](int slot) { return h[16 + slot] == 0 ? -1ll : (long long)(h[16 + slot] - h[16]); };
        fprintf(stderr, "[dg profile] CTA 0 timeline (ns after entry): set-up %lld | first stage %lld | first accumulator %lld | "
                        "parked %lld | cluster parked %lld | last store issued %lld | stores complete %lld | exit %lld\n",
                since_entry(1), since_entry(2), since_entry(3), since_entry(7), since_entry(8), since_entry(4), since_entry(5), since_entry(6));
        fprintf(stderr, "[dg profile] all CTAs (ns after the first entered): last entry %lld | last first-stage %lld | last first-accumulator %lld | last exit %lld\n",
                (long long)(h[16 + 10] - h[16 + 9]), (long long)(h[16 + 12] - h[16 + 9]), (long long)(h[16 + 13] - h[16 + 9]), (long long)(h[16 + 11] - h[16 + 9]));
        if (split)
            return launch_splitk_reduce(workspace, a->d, p.m, p.n, ld_ws, panel_rows, a->ldd, cfg.num_splits, alpha, p.d_fp32,
                                        static_cast<cudaStream_t>(a->stream));
        return DG_OK;
    }
    if ((rc = dg_jit_launch(kernel, cfg.num_ctas, 128 + cfg.block_m, launch_cluster, cfg.smem_bytes, state().pdl, a->stream, kargs)) != DG_OK) return rc;
    if (split)
        return launch_splitk_reduce(workspace, a->d, p.m, p.n, ld_ws, panel_rows, a->ldd, cfg.num_splits, alpha, p.d_fp32,
                                    static_cast<cudaStream_t>(a->stream));
    return DG_OK;
}

}  // namespace

void release_split_workspaces() {
    std::lock_guard<std::mutex> lock(g_workspace_mu);
    for (auto& [device, w] : g_workspaces)
        if (w.first != nullptr) cudaFree(w.first);
    g_workspaces.clear();
}

// Called by the no-allocation entry point in dg_splitk.cu, which owns the fixed buffer
int run_dense_gemm_with_fixed_scratch(const dg_gemm_args_t* args, float* scratch, size_t scratch_bytes) {
    const FixedScratch fixed{scratch, scratch_bytes};
    return run_gemm(DG_GEMM_DENSE, args, &fixed);
}

}  // namespace dg

using namespace dg;

extern "C" {

int dg_fp8_fp4_gemm(const dg_gemm_args_t* args) { return run_gemm(DG_GEMM_DENSE, args); }
int dg_m_grouped_fp8_fp4_gemm_contiguous(const dg_gemm_args_t* args) {
    const bool psum = args != nullptr && args->use_psum_layout != 0;
    return run_gemm(psum ? DG_GEMM_M_GROUPED_CONTIGUOUS_PSUM : DG_GEMM_M_GROUPED_CONTIGUOUS, args);
}
int dg_m_grouped_fp8_fp4_gemm_masked(const dg_gemm_args_t* args) { return run_gemm(DG_GEMM_M_GROUPED_MASKED, args); }
int dg_k_grouped_fp8_gemm_contiguous(const dg_gemm_args_t* args) { return run_gemm(DG_GEMM_K_GROUPED_CONTIGUOUS, args); }
int dg_fp8_bmm(const dg_gemm_args_t* args) { return run_gemm(DG_GEMM_BATCHED, args); }

int dg_get_gemm_config(int kind, const dg_gemm_args_t* args, dg_gemm_config_t* config) {
    DG_REQUIRE(config != nullptr);
    env_refresh();
    Problem p;
    const int rc = validate(kind, args, false, &p);
    if (rc != DG_OK) return rc;
    DG_REQUIRE(p.m > 0 && p.n > 0 && p.k > 0);
    return choose_config(p, config);
}

int dg_gemm_precompile(int kind, const dg_gemm_args_t* args) {
    env_refresh();
    Problem p;
    int rc = validate(kind, args, false, &p);
    if (rc != DG_OK) return rc;
    DG_REQUIRE(p.m > 0 && p.n > 0 && p.k > 0);
    dg_gemm_config_t cfg;
    if ((rc = choose_config(p, &cfg)) != DG_OK) return rc;
    dg_kernel_t kernel = nullptr;
    return get_kernel(p, cfg, &kernel);
}

int dg_enumerate_tiles(int kind, int block_n, int raster_group, int shape_m, int shape_n, int num_groups,
                       const int32_t* layout_host, int cta, int num_ctas, uint32_t* out, int max_tiles) {
    if (!(block_n > 0 && raster_group > 0 && num_ctas > 0 && cta >= 0 && cta < num_ctas && shape_m >= 0 && shape_n >= 0)) {
        fail(DG_ERR_INVALID_ARGUMENT, "Assertion error (%s:%d): bad scheduler arguments", __FILE__, __LINE__);
        return -DG_ERR_INVALID_ARGUMENT;
    }
    int count = 0;
    Tile t;
    auto emit = [&]() {
        if (count < max_tiles && out != nullptr) {
            out[4 * count + 0] = t.m_block; out[4 * count + 1] = t.n_block;
            out[4 * count + 2] = t.group;   out[4 * count + 3] = t.valid_rows;
        }
        ++count;
    };
    auto walk = [&](auto sched) { while (sched.next(t)) emit(); };
    const uint32_t bn = block_n, rg = raster_group, sm = shape_m, sn = shape_n, ng = num_groups, c = cta, nc = num_ctas;
    switch (kind) {
        case DG_GEMM_DENSE: walk(TileScheduler<kDense>(128, bn, rg, sm, sn, ng, layout_host, c, nc)); break;
        case DG_GEMM_M_GROUPED_CONTIGUOUS: walk(TileScheduler<kMGroupedContiguous>(128, bn, rg, sm, sn, ng, layout_host, c, nc)); break;
        case DG_GEMM_M_GROUPED_MASKED: walk(TileScheduler<kMGroupedMasked>(128, bn, rg, sm, sn, ng, layout_host, c, nc)); break;
        case DG_GEMM_M_GROUPED_CONTIGUOUS_PSUM: {
            // m_block is reported as the absolute 128-row block of A (groups start on multiples of the alignment)
            TileScheduler<kMGroupedPsum> sched(128, bn, rg, sm, sn, ng, layout_host, c, nc);
            sched.group_alignment = static_cast<uint32_t>(state().mk_alignment);
            while (sched.next(t)) { t.m_block += t.a_row_base / 128; emit(); }
            break;
        }
        case DG_GEMM_K_GROUPED_CONTIGUOUS: {
            // layout: the slices' lengths (multiples of the alignment); the fourth word is the slice's K-block count
            TileScheduler<kKGrouped> sched(128, bn, rg, sm, sn, ng, layout_host, c, nc);
            sched.group_alignment = static_cast<uint32_t>(state().mk_alignment);
            while (sched.next(t)) { t.valid_rows = t.num_kb; emit(); }
            break;
        }
        case DG_GEMM_BATCHED: walk(TileScheduler<kBatched>(128, bn, rg, sm, sn, ng, layout_host, c, nc)); break;
        default: fail(DG_ERR_INVALID_ARGUMENT, "unknown GEMM kind"); return -DG_ERR_INVALID_ARGUMENT;
    }
    return count;
}

}  // extern "C"
