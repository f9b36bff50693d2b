// Shared-memory and tensor-memory budget of the GEMM kernel as constexpr arithmetic, included by the
// device code (with the DG_* macros as arguments) and by the host heuristics (with candidate values),
// so the two can never disagree about a byte offset.
#pragma once

#include <cstdint>

#if defined(__CUDACC__)
#define DG_HDC __host__ __device__ constexpr
#else
#define DG_HDC constexpr
#endif

namespace dg {

constexpr uint32_t kSmemCapacity = 232448;      // largest dynamic shared memory per CTA on sm_100 (227 KB)
constexpr uint32_t kTmemCapacityCols = 512;

struct GemmLayout {
    uint32_t block_m, block_n, block_k, num_stages, d_elem_bytes;   // block_m: rows of A per CTA and stage (128 or 256); D: 4, 2 or 1 byte
    uint32_t cluster = 1;                          // CTAs sharing one B tile (each loads block_n / cluster rows of B)
    uint32_t b_mn_major = 0;                       // B stored with N contiguous: staged as 128-column atoms of [128 K][128 B]
    uint32_t gran_k_a = 128, gran_k_b = 128;       // elements of K per scale (a packed scale word holds four scales)
    uint32_t short_k = 0;                          // a work item has fewer K-blocks than there are stages
    uint32_t ab_elem_bytes = 1;                    // 1: FP8 / FP4 operands with block scales; 2: BF16 operands, no scales
                                                   // (block_k stays the byte width of a K-major stage row)
    uint32_t store_buffers = 2;                    // staging buffers of D per epilogue warpgroup: 2, or 1 where the 8-16 KB
                                                   // saved buy another pipeline stage (MN-major operands: whole 128-byte atoms)
    uint32_t mxf4 = 0;                             // FP4 x FP4 through kind::mxf4: operands stay packed in shared memory (two
                                                   // elements per byte), so a 128-byte stage row holds 256 elements of K
    uint32_t a_rows = 0;                           // rows of A a stage holds when the whole GEMM has fewer than block_m (0: block_m).
                                                   // The MMA still reads 128 rows: the rest is whatever follows in shared
                                                   // memory and lands in accumulator rows that are never stored

    // A packed scale word covers 4 * gran_k elements of K: it is fetched on every `period`-th K-block of a work item,
    // into the next of a ring of buffers.  A buffer may be refilled once the fetch it held is no longer among the
    // last num_stages pipeline steps (the producer is never further ahead of the MMAs).  num_stages consecutive steps
    // span at most two work items when every item has at least num_stages K-blocks, and then hold at most
    // ceil(num_stages / period) + 1 fetches; with shorter items every step may fetch.
    // (a stage that holds more than 4 * gran_k elements fetches several words per K-block instead: sf_words)
    DG_HDC uint32_t k_elems() const { return block_k * (mxf4 ? 2 : 1) / ab_elem_bytes; }      // elements of K per pipeline stage
    DG_HDC uint32_t sf_period(uint32_t gran) const { return 4 * gran / k_elems() ? 4 * gran / k_elems() : 1; }
    DG_HDC uint32_t sf_words(uint32_t gran) const { return k_elems() / (4 * gran) ? k_elems() / (4 * gran) : 1; }
    DG_HDC uint32_t sfa_period() const { return sf_period(gran_k_a); }
    DG_HDC uint32_t sfb_period() const { return sf_period(gran_k_b); }
    DG_HDC uint32_t sfa_words() const { return sf_words(gran_k_a); }
    DG_HDC uint32_t sfb_words() const { return sf_words(gran_k_b); }
    DG_HDC uint32_t sf_buffers(uint32_t period) const {
        if (ab_elem_bytes != 1) return 0;
        const uint32_t n = (num_stages + period - 1) / period + 1;
        return short_k || n > num_stages ? num_stages : n;
    }
    DG_HDC uint32_t sfa_buffers() const { return sf_buffers(sfa_period()); }
    DG_HDC uint32_t sfb_buffers() const { return sf_buffers(sfb_period()); }

    DG_HDC uint32_t sf_block_n() const { return (block_n + 127) / 128 * 128; }
    // D leaves through TMA store boxes of 128 rows.  The epilogue drains one "group" of every D row per synchronisation:
    // 128 bytes with 128-row CTA tiles, 64 bytes with 256-row tiles (whose two epilogue warpgroups each double-buffer
    // their staging inside the same 32 KB) and with one-byte (quantised FP8) output, so a group is never more than 64 columns.  Complete groups use a box as wide as the group; the remainder of the tile
    // row (when block_n * element size is not a multiple of the group) uses boxes of the widest swizzle span dividing it.
    DG_HDC uint32_t group_bytes() const { return block_m == 256 || d_elem_bytes == 1 ? 64 : 128; }
    DG_HDC uint32_t tail_bytes() const { return (block_n * d_elem_bytes) % group_bytes(); }
    DG_HDC uint32_t store_row_bytes() const {          // row width of the boxes that cover the tail (the group width when there is none)
        return tail_bytes() == 0 ? group_bytes() : (tail_bytes() % 64 == 0 ? 64 : 32);
    }
    DG_HDC uint32_t store_cols() const { return store_row_bytes() / d_elem_bytes; }
    DG_HDC uint32_t num_stores() const { return block_n * d_elem_bytes / group_bytes() + tail_bytes() / store_row_bytes(); }
    DG_HDC uint32_t group_cols() const { return group_bytes() / d_elem_bytes; }
    DG_HDC uint32_t num_groups() const { return (block_n + group_cols() - 1) / group_cols(); }
    DG_HDC uint32_t store_stage_bytes() const { return 128 * group_bytes(); }      // staging holds 128 rows of one group
    DG_HDC uint32_t num_store_stages() const { return store_buffers * (block_m / 128); }

    DG_HDC uint32_t a_stage_rows() const { return a_rows ? a_rows : block_m; }
    DG_HDC uint32_t a_bytes() const { return a_stage_rows() * block_k; }  // one byte per element (FP8, or FP4 in 16-byte containers)
    DG_HDC uint32_t load_block_n() const { return block_n / cluster; }
    // MN-major only: atoms of [block_k / ab_elem_bytes rows of K][128 bytes of N]
    DG_HDC uint32_t b_atoms() const { return (load_block_n() * ab_elem_bytes + 127) / 128; }
    DG_HDC uint32_t b_bytes() const { return b_mn_major ? b_atoms() * 128 * (block_k / ab_elem_bytes) : load_block_n() * block_k; }
    DG_HDC uint32_t sfa_bytes() const { return block_m * 4 * sfa_words(); }          // [word of K][row] int32
    DG_HDC uint32_t sfb_bytes() const { return sf_block_n() * 4 * sfb_words(); }

    DG_HDC uint32_t off_d() const { return 0; }
    DG_HDC uint32_t off_a() const { return (num_store_stages() * store_stage_bytes() + 1023) / 1024 * 1024; }
    DG_HDC uint32_t off_b() const { return off_a() + num_stages * a_bytes(); }
    DG_HDC uint32_t off_sfa() const { return off_b() + num_stages * b_bytes(); }
    DG_HDC uint32_t off_sfb() const { return off_sfa() + sfa_buffers() * sfa_bytes(); }
    DG_HDC uint32_t off_barriers() const { return off_sfb() + sfb_buffers() * sfb_bytes(); }
    DG_HDC uint32_t num_barriers() const { return 3 * num_stages + 2 * 2; }
    DG_HDC uint32_t off_misc() const { return off_barriers() + num_barriers() * 8; }
    // (tensor-memory base, abort flag).  With shortened A stages the MMA of the last stage still reads block_m rows from
    // that stage's base: the allocation reaches at least that far, so the read stays inside this CTA's shared memory
    DG_HDC uint32_t total_bytes() const {
        const uint32_t used = off_misc() + 16, a_read_end = off_a() + (num_stages - 1) * a_bytes() + block_m * block_k;
        return a_rows && a_read_end > used ? a_read_end : used;
    }

    // Tensor memory: two accumulators of block_n columns (two tiles in flight when block_m is 128, the two 128-row
    // halves of one tile when it is 256), then SFA (4 columns per 128 rows) and SFB (4 columns per 128 columns of the tile)
    DG_HDC uint32_t tmem_col_sfa() const { return 2 * block_n; }
    // (per packed word of a stage: kind::mxf4 stages hold two)
    DG_HDC uint32_t tmem_col_sfb() const { return tmem_col_sfa() + block_m / 32 * sfa_words(); }
    DG_HDC uint32_t tmem_cols_used() const { return ab_elem_bytes != 1 ? 2 * block_n : tmem_col_sfb() + sf_block_n() / 32 * sfb_words(); }
    DG_HDC uint32_t tmem_cols_alloc() const {
        const uint32_t u = tmem_cols_used();
        return u <= 32 ? 32 : u <= 64 ? 64 : u <= 128 ? 128 : u <= 256 ? 256 : 512;
    }
};

}  // namespace dg
