// Thin inline-PTX wrappers for sm_100a: mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (TMEM
// alloc / cp / mma / commit / ld) and the descriptor encodings they take.
//
// Every wait in this file is bounded: a wait that does not complete within kWaitTimeoutNs
// records a code in a status word and returns false so that the caller can unwind, free its
// tensor memory and return.  Nothing here traps.
#pragma once

#include <cuda.h>
#include <cstdint>

namespace dg {

// ------------------------------------------------------------------------------------------
// Small utilities
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t lane_id() {
    uint32_t l;
    asm volatile("mov.u32 %0, %%laneid;" : "=r"(l));
    return l;
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

__device__ __forceinline__ void cluster_arrive_relaxed() {
    asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_arrive() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Address of the same shared-memory variable in another CTA of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t cta_rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta_rank));
    return r;
}

__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void named_barrier_sync(uint32_t id, uint32_t num_threads) {
    asm volatile("bar.sync %0, %1;" :: "r"(id), "r"(num_threads) : "memory");
}

// Programmatic dependent launch.  A kernel launched with programmatic stream serialisation may start while the
// kernel before it in the stream still runs: griddep_wait() returns once that kernel has completed and its writes
// are visible; griddep_launch_dependents() lets the kernel after this one start its own preamble.  Both do nothing
// in a normally launched kernel.
__device__ __forceinline__ void griddep_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void griddep_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Moves registers between the warpgroups of a CTA: every warp of a warpgroup (four consecutive warps) gives up or
// claims registers down / up to kRegs per thread (a multiple of 8)
template <uint32_t kRegs>
__device__ __forceinline__ void warpgroup_reg_dec() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" :: "n"(kRegs));
}
template <uint32_t kRegs>
__device__ __forceinline__ void warpgroup_reg_inc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" :: "n"(kRegs));
}

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* p) {
    asm volatile("prefetch.tensormap [%0];" :: "l"(reinterpret_cast<uint64_t>(p)) : "memory");
}

// ------------------------------------------------------------------------------------------
// Error reporting: first failure wins.  Code layout: [31:24] role, [23:16] site, [15:0] blockIdx.
// ------------------------------------------------------------------------------------------
// 1.5 s; legitimate waits are < 10 ms.  A translation unit may define DG_WAIT_TIMEOUT_NS before including this file
// (the library's self-test of the expiry path does, with a limit of about a millisecond).
#ifndef DG_WAIT_TIMEOUT_NS
#define DG_WAIT_TIMEOUT_NS 1500000000ull
#endif
constexpr uint64_t kWaitTimeoutNs = DG_WAIT_TIMEOUT_NS;

struct AbortCtx {
    volatile uint32_t* flag;   // shared memory word, non-zero once any role of this CTA gave up
    int* status;               // global (host-visible) status word
};

__device__ __forceinline__ void report_failure(const AbortCtx& ctx, uint32_t role, uint32_t site) {
    *ctx.flag = 1;
    if (ctx.status != nullptr)
        atomicCAS(ctx.status, 0, static_cast<int>((role << 24) | (site << 16) | (blockIdx.x & 0xFFFFu) | 0x80000000u));
}

// ------------------------------------------------------------------------------------------
// mbarrier
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}

// Arrive on a barrier that lives in another CTA of the cluster (address from map_to_cta).
// Default (release, CTA scope) semantics on purpose: what crosses CTAs here is only "my asynchronous copies
// were issued / my tensor-memory reads are done"; the data itself moves through the async proxy.  Cluster-scope
// release/acquire on these barriers halved the MMA issue rate when measured.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" :: "r"(cluster_bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false if this CTA is unwinding (another role failed) or the wait ran out.
// The limit is counted in SM clocks (clock64, a register read) rather than read from the nanosecond global timer, whose
// reads are slow enough to delay a role that a barrier was about to release; at most 2 clocks pass per nanosecond on
// this part, so a wait gives up no earlier than kWaitTimeoutNs after it began (later when the clock is throttled).
// `backoff_ns` > 0 makes a waiter that expects to wait long (an epilogue warp during the main loop of its tile) sleep
// between polls instead of competing for issue slots with the role warps that share its scheduler.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const AbortCtx& ctx,
                                          uint32_t role, uint32_t site, uint32_t backoff_ns = 0) {
    auto poll = [&]() { return mbar_try_wait(bar, parity); };
    #pragma unroll 1
    for (int i = 0; i < (backoff_ns ? 4 : 64); ++i)
        if (poll()) return true;
    const long long t0 = clock64();
    constexpr long long kWaitTimeoutClocks = static_cast<long long>(kWaitTimeoutNs) * 2;
    uint32_t spins = 0;
    #pragma unroll 1
    while (!poll()) {
        if (backoff_ns) __nanosleep(backoff_ns);
        if ((++spins & (backoff_ns ? 0xFu : 0xFFu)) == 0) {
            if (*ctx.flag != 0) return false;
            if (clock64() - t0 > kWaitTimeoutClocks) {
                report_failure(ctx, role, site);
                return false;
            }
        }
    }
    return true;
}

// ------------------------------------------------------------------------------------------
// TMA
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar,
                                            int32_t x, int32_t y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        :: "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y) : "memory");
}

// Three-dimensional forms (batched GEMM: the outermost coordinate is the batch; the box is one batch deep)
__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar,
                                            int32_t x, int32_t y, int32_t z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        :: "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z) : "memory");
}

__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t smem_src, int32_t x, int32_t y, int32_t z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
        :: "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_src), "r"(x), "r"(y), "r"(z) : "memory");
}

__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap* map, uint32_t smem_src, int32_t x, int32_t y, int32_t z) {
    asm volatile(
        "cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
        :: "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_src), "r"(x), "r"(y), "r"(z) : "memory");
}

// 2-CTA form: the copy lands in this CTA's shared memory, the bytes are counted on the barrier
// at the same offset in the leader CTA (bar is a shared::cluster address).
__device__ __forceinline__ void tma_load_2d_2cta(uint32_t smem_dst, const CUtensorMap* map, uint32_t cluster_bar,
                                                 int32_t x, int32_t y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        :: "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(x), "r"(y) : "memory");
}

// L2 eviction-priority policies for loads that carry a cache hint: lines fetched with evict_last stay in L2 in
// preference to lines fetched with evict_first (an operand band that the next waves of tiles read again against a panel
// that is streamed through once).
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void tma_load_2d_hint(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar, int32_t x, int32_t y, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
        :: "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "l"(policy) : "memory");
}
__device__ __forceinline__ void tma_load_2d_2cta_hint(uint32_t smem_dst, const CUtensorMap* map, uint32_t cluster_bar, int32_t x, int32_t y,
                                                      uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
        :: "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(x), "r"(y), "l"(policy) : "memory");
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t smem_src, int32_t x, int32_t y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
        :: "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_src), "r"(x), "r"(y) : "memory");
}

__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, uint32_t smem_src, int32_t x, int32_t y) {
    asm volatile(
        "cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
        :: "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_src), "r"(x), "r"(y) : "memory");
}

__device__ __forceinline__ void tma_store_commit() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

template <int kPending>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" :: "n"(kPending) : "memory");
}

template <int kPending>
__device__ __forceinline__ void tma_store_wait() {
    asm volatile("cp.async.bulk.wait_group %0;" :: "n"(kPending) : "memory");
}

// ------------------------------------------------------------------------------------------
// tcgen05: tensor memory management
// ------------------------------------------------------------------------------------------
template <int kCtaGroup>
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result_addr, uint32_t num_cols) {
    if constexpr (kCtaGroup == 1)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_result_addr), "r"(num_cols) : "memory");
    else
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_result_addr), "r"(num_cols) : "memory");
}

template <int kCtaGroup>
__device__ __forceinline__ void tmem_relinquish() {
    if constexpr (kCtaGroup == 1)
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    else
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

template <int kCtaGroup>
__device__ __forceinline__ void tmem_dealloc(uint32_t tmem_addr, uint32_t num_cols) {
    if constexpr (kCtaGroup == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_addr), "r"(num_cols) : "memory");
    else
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" :: "r"(tmem_addr), "r"(num_cols) : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ------------------------------------------------------------------------------------------
// tcgen05: descriptors
// ------------------------------------------------------------------------------------------
// Shared-memory matrix descriptor (64 bit):
//   [0,14)  start address >> 4        [16,30) leading-dimension byte offset >> 4
//   [32,46) stride-dimension byte offset >> 4     [46,48) descriptor version (1 on sm_100)
//   [49,52) base offset               [52]    LBO mode          [61,64) swizzle mode
enum : uint64_t { kSwizzleNone = 0, kSwizzle128B = 2, kSwizzle64B = 4, kSwizzle32B = 6 };

__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   uint64_t swizzle) {
    return static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4)
         | (static_cast<uint64_t>(lbo_bytes >> 4) << 16)
         | (static_cast<uint64_t>(sbo_bytes >> 4) << 32)
         | (1ull << 46)
         | (swizzle << 61);
}

// Instruction descriptor of the block-scaled MMA kinds (32 bit):
//   [4,6)  B scale-factor byte id     [7,10) A format    [10,13) B format
//   [15]   A is MN-major              [16]   B is MN-major
//   [17,23) N >> 3                    [23]   scale format (1 = UE8M0)
//   [24,29) M >> 4                    [29,31) A scale-factor byte id
// (kind::mxf8f6f4 formats; kind::mxf4 has its own numbering, in which E2M1 is 1)
enum : uint32_t { kFmtE4M3 = 0, kFmtE2M1 = 5, kFmtMxf4E2M1 = 1 };

__host__ __device__ constexpr uint32_t make_instr_desc_block_scaled(uint32_t a_fmt, uint32_t b_fmt,
                                                                     uint32_t a_mn_major, uint32_t b_mn_major,
                                                                     uint32_t umma_m, uint32_t umma_n) {
    return (a_fmt << 7) | (b_fmt << 10) | (a_mn_major << 15) | (b_mn_major << 16)
         | ((umma_n >> 3) << 17) | (1u << 23) | ((umma_m >> 4) << 24);
}

// Instruction descriptor of kind::f16 (BF16 inputs, FP32 accumulation):
//   [4,6) D format (1 = F32)   [7,10) A format (1 = BF16)   [10,13) B format   [15] / [16] A / B MN-major
//   [17,23) N >> 3             [24,29) M >> 4
__host__ __device__ constexpr uint32_t make_instr_desc_bf16(uint32_t a_mn_major, uint32_t b_mn_major, uint32_t umma_m, uint32_t umma_n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (a_mn_major << 15) | (b_mn_major << 16) | ((umma_n >> 3) << 17) | ((umma_m >> 4) << 24);
}

__device__ __forceinline__ uint32_t instr_desc_with_sf_ids(uint32_t idesc, uint32_t sfa_id, uint32_t sfb_id) {
    return idesc | (sfb_id << 4) | (sfa_id << 29);
}

// ------------------------------------------------------------------------------------------
// tcgen05: data movement and math
// ------------------------------------------------------------------------------------------
// 32 rows x 128 bit from shared memory into 32 lanes x 4 columns, replicated in all four
// 32-lane quarters of tensor memory (the layout the block-scaled MMA reads its scales from).
template <int kCtaGroup>
__device__ __forceinline__ void tc_cp_32x128b_warpx4(uint32_t tmem_addr, uint64_t smem_desc) {
    if constexpr (kCtaGroup == 1)
        asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" :: "r"(tmem_addr), "l"(smem_desc) : "memory");
    else
        asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" :: "r"(tmem_addr), "l"(smem_desc) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem] with per-32-K UE8M0 scales in tensor memory (FP8/FP6/FP4 inputs, K = 32).
template <int kCtaGroup>
__device__ __forceinline__ void tc_mma_mxf8f6f4(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
    if constexpr (kCtaGroup == 1)
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
            :: "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb) : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
            :: "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem] for packed FP4 inputs (two E2M1 values per byte, K = 64 elements = 32 bytes per
// instruction) with one UE8M0 scale per 32 elements of K: two scale bytes of the word in tensor memory per instruction,
// bytes 0-1 or 2-3 as the scale-factor id (0 or 2) of the instruction descriptor says.  Twice the FP8 rate.
template <int kCtaGroup>
__device__ __forceinline__ void tc_mma_mxf4(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
    if constexpr (kCtaGroup == 1)
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
            :: "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb) : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
            :: "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem] for BF16 inputs (K = 16 elements per instruction), no scales.
template <int kCtaGroup>
__device__ __forceinline__ void tc_mma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    if constexpr (kCtaGroup == 1)
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            :: "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            :: "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}

// Make an mbarrier track completion of every tcgen05 operation this thread issued so far.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar) : "memory");
}
// 2-CTA form; cluster_bar is a shared::cluster address (own or peer CTA).
__device__ __forceinline__ void tc_commit_2cta(uint32_t cluster_bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(cluster_bar) : "memory");
}
// 2-CTA form that signals the barrier at the same shared-memory offset in every CTA of `cta_mask` with ONE instruction
// (a commit costs the issuing thread ~100 cycles, and a pipeline stage of a CTA pair must be released in both CTAs).
// This is an mbarrier arrive, not a copy: no data moves between the CTAs.
__device__ __forceinline__ void tc_commit_2cta_mask(uint32_t bar, uint16_t cta_mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 :: "r"(bar), "h"(cta_mask) : "memory");
}

// One warp reads its 32 lanes x 16 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t tmem_addr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(tmem_addr) : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ------------------------------------------------------------------------------------------
// Misc data helpers
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" :: "r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// A 32-bit word of another CTA's shared memory (distributed shared memory; the address comes from map_to_cta)
__device__ __forceinline__ uint32_t ld_shared_cluster_u32(uint32_t cluster_addr) {
    uint32_t v;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(cluster_addr) : "memory");
    return v;
}

// Four consecutive words (16-byte aligned) of another CTA's shared memory
__device__ __forceinline__ uint4 ld_shared_cluster_v4(uint32_t cluster_addr) {
    uint4 v;
    asm volatile("ld.shared::cluster.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(cluster_addr) : "memory");
    return v;
}

// Store into another CTA's shared memory (or this one's, through the same window); posted: nothing waits for it
__device__ __forceinline__ void st_shared_cluster_u32(uint32_t cluster_addr, uint32_t v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" :: "r"(cluster_addr), "r"(v) : "memory");
}

__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}

__device__ __forceinline__ void st_shared_u32(uint32_t addr, uint32_t v) {
    asm volatile("st.shared.u32 [%0], %1;" :: "r"(addr), "r"(v) : "memory");
}

__device__ __forceinline__ void st_shared_u16(uint32_t addr, uint32_t v) {
    asm volatile("st.shared.u16 [%0], %1;" :: "r"(addr), "h"(static_cast<unsigned short>(v)) : "memory");
}

__device__ __forceinline__ uint32_t ld_shared_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}

}  // namespace dg
