// Persistent tile scheduler shared by every warp role of the GEMM kernel and by the host-side
// model that the CPU tests walk.  CTA c processes tiles c, c + num_ctas, c + 2 num_ctas, ...
// of one global tile order:
//
//   dense / m-grouped contiguous : the (m_blocks x n_blocks) grid, rasterised in bands of
//       `raster_group` row blocks (n outer, m inner inside a band) so that the tiles a wave runs
//       together share A rows and B rows in L2.  For the contiguous layout the expert of a row
//       block is grouped_layout[first row of the block] (-1, a padding row, maps to expert 0 as in
//       deep_gemm/include/deep_gemm/scheduler/gemm.cuh:151-153).
//   m-grouped masked : groups in order; group g contributes ceil(masked_m[g] / 128) row blocks,
//       read on the device (no host synchronisation, so a captured graph follows new counts);
//       same contract as scheduler/gemm.cuh:188-204.
//   m-grouped contiguous with a prefix-sum layout : layout[g] is the row where group g ends; group g
//       starts at layout[g - 1] rounded up to the contiguous-layout alignment (row 0 for g = 0), so
//       the rows in between are padding.  Walked on the device like the masked layout; same
//       contract as scheduler/gemm.cuh:205-225.
//   k-grouped contiguous (the weight-gradient GEMM of a mixture of experts): every group g owns a slice
//       of K and its own [shape_m x shape_n] output D[g] = A[slice]^T B[slice]; all groups have the same
//       (m_blocks x n_blocks) tile grid, and a tile carries the slice's first element of K, its length in
//       K-blocks and the first packed scale row of the group.  layout[g] is the slice's length (a multiple
//       of the alignment) or, in the prefix-sum form, the element where it ends, the next slice starting
//       at the following multiple of the alignment (scheduler/gemm.cuh:226-250 of the reference).
//   batched : num_groups independent GEMMs of one shape; tile_id = batch * tiles_per_batch + tile, the
//       batch being the third tensor-map coordinate of every operand (scheduler/gemm.cuh:251-263).
#pragma once

#include <cstdint>

#if defined(__CUDACC__)
#define DG_HD __host__ __device__ __forceinline__
#else
#define DG_HD inline
#endif

namespace dg {

enum GemmKind : uint32_t { kDense = 0, kMGroupedContiguous = 1, kMGroupedMasked = 2, kMGroupedPsum = 3, kKGrouped = 4, kBatched = 5 };

struct Tile {
    uint32_t m_block;       // row block inside the group (masked) or inside A (dense / contiguous)
    uint32_t n_block;
    uint32_t group;         // which B[g] / SFB[g] this tile multiplies with
    uint32_t group1;        // contiguous layout with 256-row tiles: the expert of the tile's second 128 rows
    uint32_t a_row_base;    // first row of the group in the 2-D view of A
    uint32_t d_row_base;    // first row of the group in the 2-D view of D
    uint32_t sfa_mn_base;   // first row of the group along the MN axis of SFA
    uint32_t sfa_group;     // group index along the packed-K axis of SFA
    uint32_t valid_rows;    // rows of this tile that may be written (128 unless a ragged masked tile)
    uint32_t split;         // which slice of K this work item covers (0 unless the GEMM is split along K)
    uint32_t mn_index;      // linear index of the output tile (slot of its split-K partials and counter)
    // k-grouped only
    uint32_t k_base;        // first element of K of the group's slice
    uint32_t num_kb;        // K-blocks (pipeline stages) in the slice (0: an empty group)
    uint32_t sf_row_base;   // first packed scale row of the group
};

// Tile sizes are constructor arguments (literal constants in the kernel, which the compiler folds;
// run-time values in the host model).
template <uint32_t kKind>
struct TileScheduler {
    uint32_t kBlockM, kRasterGroup;
    uint32_t shape_m, num_groups;
    uint32_t num_m_blocks, num_n_blocks;
    const int* layout;
    uint32_t cta, num_ctas, iter;
    uint32_t num_splits;    // dense only: every output tile is computed as num_splits work items over slices of K
    // masked and prefix-sum layouts only
    uint32_t cur_group, group_first_tile;
    // prefix-sum layout only: first row of the current group, the alignment of group starts, and whether the
    // padding rows up to the next aligned row count as writable (they are written as the product of zero rows)
    uint32_t group_start, group_alignment, write_padding;
    // k-grouped only: first element of K and first packed scale row of the current group; whether layout holds
    // prefix sums; elements of K per packed scale row (4 scales)
    uint32_t k_start, sf_row_start, k_psum, k_per_sf_row, k_per_block;     // k_per_block: elements of K per pipeline stage

    DG_HD TileScheduler(uint32_t block_m_, uint32_t block_n_, uint32_t raster_group_,
                        uint32_t shape_m_, uint32_t shape_n_, uint32_t num_groups_, const int* layout_,
                        uint32_t cta_, uint32_t num_ctas_, uint32_t num_splits_ = 1)
        : kBlockM(block_m_), kRasterGroup(raster_group_), shape_m(shape_m_), num_groups(num_groups_),
          num_m_blocks((shape_m_ + block_m_ - 1) / block_m_), num_n_blocks((shape_n_ + block_n_ - 1) / block_n_),
          layout(layout_), cta(cta_), num_ctas(num_ctas_), iter(0), num_splits(num_splits_ == 0 ? 1 : num_splits_),
          cur_group(0), group_first_tile(0), group_start(0), group_alignment(128), write_padding(0),
          k_start(0), sf_row_start(0), k_psum(0), k_per_sf_row(512), k_per_block(128) {}

    // Linear index inside an (mb x num_n_blocks) grid -> (m, n)
    DG_HD void rasterise(uint32_t idx, uint32_t mb, uint32_t& m, uint32_t& n) const {
        const uint32_t per_band = kRasterGroup * num_n_blocks;
        const uint32_t band = idx / per_band;
        const uint32_t first_m = band * kRasterGroup;
        const uint32_t rem = idx - band * per_band;
        const uint32_t rows = mb - first_m < kRasterGroup ? mb - first_m : kRasterGroup;
        m = first_m + rem % rows;
        n = rem / rows;
    }

    DG_HD bool next(Tile& t) {
        const uint32_t tile_id = iter * num_ctas + cta;
        ++iter;
        if constexpr (kKind == kMGroupedMasked) {
            uint32_t mb = 0, rows = 0;
            while (true) {
                if (cur_group >= num_groups) return false;
                const int r = layout[cur_group];
                rows = r < 0 ? 0u : (static_cast<uint32_t>(r) > shape_m ? shape_m : static_cast<uint32_t>(r));
                mb = (rows + kBlockM - 1) / kBlockM;
                if (tile_id < group_first_tile + mb * num_n_blocks) break;
                group_first_tile += mb * num_n_blocks;
                ++cur_group;
            }
            rasterise(tile_id - group_first_tile, mb, t.m_block, t.n_block);
            t.group = t.group1 = cur_group;
            t.a_row_base = t.d_row_base = cur_group * shape_m;
            t.sfa_mn_base = 0;
            t.sfa_group = cur_group;
            const uint32_t left = rows - t.m_block * kBlockM;
            t.valid_rows = left < kBlockM ? left : kBlockM;
            t.split = 0;
            t.mn_index = tile_id;
            return true;
        } else if constexpr (kKind == kBatched) {
            const uint32_t blocks = num_m_blocks * num_n_blocks;
            const uint32_t batch = tile_id / blocks;
            if (batch >= num_groups) return false;
            rasterise(tile_id - batch * blocks, num_m_blocks, t.m_block, t.n_block);
            t.group = t.group1 = batch;
            t.a_row_base = t.d_row_base = t.sfa_mn_base = t.sfa_group = 0;
            t.valid_rows = kBlockM;              // the batch's own extent in the tensor map clips rows beyond M
            t.split = 0;
            t.mn_index = tile_id;
            return true;
        } else if constexpr (kKind == kKGrouped) {
            const uint32_t blocks = num_m_blocks * num_n_blocks;
            // Length of the current group's slice, and the length it occupies in A / B and in the scale tensor
            auto slice = [&](uint32_t& len, uint32_t& padded) {
                const int v = layout[cur_group];
                const uint32_t u = v < 0 ? 0u : static_cast<uint32_t>(v);
                len = k_psum ? (u > k_start ? u - k_start : 0u) : u;
                padded = (len + group_alignment - 1) / group_alignment * group_alignment;
            };
            uint32_t len = 0, padded = 0;
            while (true) {
                if (cur_group >= num_groups) return false;
                slice(len, padded);
                if (tile_id < (cur_group + 1) * blocks) break;
                k_start += padded;
                sf_row_start += (padded + k_per_sf_row - 1) / k_per_sf_row;
                ++cur_group;
            }
            rasterise(tile_id - cur_group * blocks, num_m_blocks, t.m_block, t.n_block);
            t.group = t.group1 = cur_group;
            t.a_row_base = t.sfa_mn_base = t.sfa_group = 0;
            t.d_row_base = cur_group * shape_m;
            const uint32_t left = shape_m - t.m_block * kBlockM;
            t.valid_rows = left < kBlockM ? left : kBlockM;
            t.split = 0;
            t.mn_index = tile_id;
            t.k_base = k_start;
            t.num_kb = (len + k_per_block - 1) / k_per_block;
            t.sf_row_base = sf_row_start;
            return true;
        } else if constexpr (kKind == kMGroupedPsum) {
            uint32_t mb = 0, rows = 0;
            while (true) {
                if (cur_group >= num_groups) return false;
                const int e = layout[cur_group];
                uint32_t end = e < 0 ? 0u : (static_cast<uint32_t>(e) > shape_m ? shape_m : static_cast<uint32_t>(e));
                if (end < group_start) end = group_start;
                rows = end - group_start;
                // With the padding written too, the tiles cover the group up to its aligned end (the alignment may exceed
                // a tile: rows past the last real one are products of the zero rows the layout requires there)
                if (write_padding) {
                    const uint32_t aligned_end = (end + group_alignment - 1) / group_alignment * group_alignment;
                    const uint32_t cap = aligned_end > shape_m ? shape_m : aligned_end;
                    rows = cap > group_start ? cap - group_start : 0u;
                }
                mb = (rows + kBlockM - 1) / kBlockM;
                if (tile_id < group_first_tile + mb * num_n_blocks) break;
                group_first_tile += mb * num_n_blocks;
                group_start = (end + group_alignment - 1) / group_alignment * group_alignment;
                ++cur_group;
            }
            rasterise(tile_id - group_first_tile, mb, t.m_block, t.n_block);
            t.group = t.group1 = cur_group;
            t.a_row_base = t.d_row_base = t.sfa_mn_base = group_start;
            t.sfa_group = 0;
            const uint32_t left = rows - t.m_block * kBlockM;            // (rows already reach the aligned end when the padding is written)
            t.valid_rows = left < kBlockM ? left : kBlockM;
            t.split = 0;
            t.mn_index = tile_id;
            return true;
        } else {
            // Work items of one output tile are consecutive, so CTAs that share a tile run at the same time
            const uint32_t mn = kKind == kDense ? tile_id / num_splits : tile_id;
            if (mn >= num_m_blocks * num_n_blocks) return false;
            rasterise(mn, num_m_blocks, t.m_block, t.n_block);
            t.split = kKind == kDense ? tile_id - mn * num_splits : 0;
            t.mn_index = mn;
            t.group = t.group1 = 0;
            if constexpr (kKind == kMGroupedContiguous) {
                const int g = layout[t.m_block * kBlockM];
                t.group = t.group1 = g < 0 ? 0u : static_cast<uint32_t>(g);
                // Expert segments are multiples of 128 rows, so a 256-row tile can end one expert and start the next
                if (kBlockM == 256 && t.m_block * kBlockM + 128 < shape_m) {
                    const int g1 = layout[t.m_block * kBlockM + 128];
                    t.group1 = g1 < 0 ? t.group : static_cast<uint32_t>(g1);
                }
            }
            t.a_row_base = t.d_row_base = t.sfa_mn_base = t.sfa_group = 0;
            t.valid_rows = kBlockM;
            return true;
        }
    }
};

}  // namespace dg
