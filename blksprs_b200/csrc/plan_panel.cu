// Panel plans: the metadata of the wide-N tcgen05 kernel.
//
// A panel is a group of up to G output blocks that are consecutive in the output LUT (the caller
// chooses the boundaries; the binding takes every G blocks).  Blocks of a panel that lie in the same
// (batch, row) of the output layout contract against the same A blocks (the A operand is indexed
// by (batch, row, t) in all three products), so one staged A block serves them all and their B
// blocks can be placed side by side in shared memory and multiplied by one wide MMA.  Where a
// panel runs across the end of a row, its blocks are walked row by row: the steps of the first
// row's blocks come first, then those of the next row's, each with its own A block.
//
// A step of a panel is one inner index t of one of its rows for which the A block exists and at
// least one B block of the panel's columns in that row exists.  Step record (8 x int32):
//   [0]     a_block
//   [1..4]  b_block of panel column q (or -1)
//   [5]     control word: bits 0-3 present mask, bits 4-7 "first" mask (columns whose
//           accumulator this step touches for the first time), bit 8 last step of the panel,
//           bits 12-14 number of output blocks in the panel
//   [6..7]  zero
#include "common.cuh"

namespace bsp {

static constexpr int kPanelMaxG = 4;

template <bool FILL>
__global__ void __launch_bounds__(256)
panel_walk_kernel(const int64_t* __restrict__ lut_out, const int32_t* __restrict__ panel_first,
                  int64_t n_panels, const int64_t* __restrict__ packed_a, int64_t a_sb, int64_t a_sr,
                  int64_t a_st, const int64_t* __restrict__ packed_b, int64_t b_sb, int64_t b_st,
                  int64_t b_sc, int64_t T, int32_t* __restrict__ counts, int32_t* __restrict__ touched_out,
                  unsigned long long* __restrict__ stats, int32_t* __restrict__ block_counts,
                  const int32_t* __restrict__ step_off, int32_t* __restrict__ steps) {
    const int lane = threadIdx.x & 31;
    const unsigned lt_mask = (1u << lane) - 1u;
    const int64_t warps_total = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t p = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); p < n_panels;
         p += warps_total) {
        const int64_t first = panel_first[p];
        int g = (int)(panel_first[p + 1] - first);
        if (g > kPanelMaxG) g = kPanelMaxG;
        // (batch, row) and the B column of every block of the panel
        int64_t blk_b[kPanelMaxG], blk_r[kPanelMaxG];
        const int64_t* pb[kPanelMaxG];
#pragma unroll
        for (int q = 0; q < kPanelMaxG; ++q) {
            const int64_t e = first + (q < g ? q : 0);
            blk_b[q] = lut_out[e * 3 + 0];
            blk_r[q] = lut_out[e * 3 + 1];
            pb[q] = packed_b + blk_b[q] * b_sb + lut_out[e * 3 + 2] * b_sc;
        }
        int32_t n = 0;
        int32_t n_hits = 0;    // (A block, B block) pairs the steps stand for
        int32_t n_col[kPanelMaxG] = {0, 0, 0, 0};  // the same per block of the panel
        unsigned touched = 0;  // columns hit by earlier steps
        const int32_t base = FILL ? step_off[p] : 0;
        const int32_t last = FILL ? step_off[p + 1] - 1 : -1;
        // runs of blocks in the same (batch, row): `group` = the columns of the current run
        unsigned todo = (1u << g) - 1u;
        while (todo) {
            const int lead = __ffs(todo) - 1;
            int64_t gb = 0, gr = 0;
#pragma unroll
            for (int q = 0; q < kPanelMaxG; ++q)
                if (q == lead) { gb = blk_b[q]; gr = blk_r[q]; }
            unsigned group = 0;
#pragma unroll
            for (int q = 0; q < kPanelMaxG; ++q)
                if (((todo >> q) & 1u) && blk_b[q] == gb && blk_r[q] == gr) group |= 1u << q;
            todo &= ~group;
            const int64_t* pa = packed_a + gb * a_sb + gr * a_sr;
            for (int64_t t0 = 0; t0 < T; t0 += 32) {
                const int64_t t = t0 + lane;
                int64_t ia = -1;
                int64_t ib[kPanelMaxG];
                unsigned mask = 0;
                if (t < T) ia = pa[t * a_st];
#pragma unroll
                for (int q = 0; q < kPanelMaxG; ++q) {
                    ib[q] = (ia >= 0 && ((group >> q) & 1u)) ? pb[q][t * b_st] : -1;
                    if (ib[q] >= 0) mask |= 1u << q;
                }
                const bool hit = mask != 0;
                const unsigned votes = __ballot_sync(0xffffffffu, hit);
                // inclusive OR-scan of the masks over the lanes
                unsigned inc = mask;
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                    const unsigned o = __shfl_up_sync(0xffffffffu, inc, d);
                    if (lane >= d) inc |= o;
                }
                unsigned before = __shfl_up_sync(0xffffffffu, inc, 1);
                if (lane == 0) before = 0;
                before |= touched;
                if (FILL && hit) {
                    const int32_t pos = base + n + __popc(votes & lt_mask);
                    int32_t* rec = steps + (int64_t)pos * 8;
                    rec[0] = (int32_t)ia;
#pragma unroll
                    for (int q = 0; q < kPanelMaxG; ++q) rec[1 + q] = (int32_t)ib[q];
                    rec[5] = (int32_t)(mask | ((mask & ~before) << 4) | (pos == last ? 0x100u : 0u) |
                                       ((unsigned)g << 12));
                    rec[6] = 0;
                    rec[7] = 0;
                }
                touched |= __shfl_sync(0xffffffffu, inc, 31);
                n += __popc(votes);
                if (!FILL) {
                    n_hits += __popc(mask);
                    if (block_counts) {
#pragma unroll
                        for (int q = 0; q < kPanelMaxG; ++q)
                            n_col[q] += __popc(__ballot_sync(0xffffffffu, (mask >> q) & 1u));
                    }
                }
            }
        }
        if (!FILL) {
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) n_hits += __shfl_xor_sync(0xffffffffu, n_hits, d);
            if (lane == 0) {
                counts[p] = n;
                touched_out[p] = (int32_t)touched;
                if (stats) {
                    atomicMax(stats + 0, (unsigned long long)n);
                    atomicAdd(stats + 1, (unsigned long long)n_hits);
                }
                if (block_counts) {
                    int32_t most = 0;
#pragma unroll
                    for (int q = 0; q < kPanelMaxG; ++q) {
                        if (q < g) {
                            block_counts[first + q] = n_col[q];
                            most = n_col[q] > most ? n_col[q] : most;
                        }
                    }
                    if (stats) atomicMax(stats + 2, (unsigned long long)most);
                }
            }
        }
    }
}

}  // namespace bsp

using namespace bsp;

static inline unsigned panel_grid(int64_t n) {
    int64_t blocks = ceil_div(n, 8);
    return (unsigned)(blocks > 148 * 32 ? 148 * 32 : (blocks < 1 ? 1 : blocks));
}

extern "C" int bsp_panel_count(const int64_t* lut_out, const int32_t* panel_first, int64_t n_panels,
                               const int64_t* packed_a, int64_t a_sb, int64_t a_sr, int64_t a_st,
                               const int64_t* packed_b, int64_t b_sb, int64_t b_st, int64_t b_sc, int64_t T,
                               int32_t* counts_out, int32_t* touched_out, int64_t* stats,
                               int32_t* block_counts_out, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (n_panels < 0 || T < 0) return BSP_ERR_INVALID_ARG;
    if (n_panels == 0) return BSP_OK;
    if (!lut_out || !panel_first || !counts_out || !touched_out || (T > 0 && (!packed_a || !packed_b)))
        return BSP_ERR_INVALID_ARG;
    panel_walk_kernel<false><<<panel_grid(n_panels), 256, 0, stream>>>(
        lut_out, panel_first, n_panels, packed_a, a_sb, a_sr, a_st, packed_b, b_sb, b_st, b_sc, T,
        counts_out, touched_out, (unsigned long long*)stats, block_counts_out, nullptr, nullptr);
    BSP_LAUNCH_CHECK();
    return BSP_OK;
}

extern "C" int bsp_panel_fill(const int64_t* lut_out, const int32_t* panel_first, int64_t n_panels,
                              const int64_t* packed_a, int64_t a_sb, int64_t a_sr, int64_t a_st,
                              const int64_t* packed_b, int64_t b_sb, int64_t b_st, int64_t b_sc, int64_t T,
                              const int32_t* step_offsets, int32_t* steps_out, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (n_panels < 0 || T < 0) return BSP_ERR_INVALID_ARG;
    if (n_panels == 0 || T == 0) return BSP_OK;
    if (!lut_out || !panel_first || !step_offsets || !packed_a || !packed_b) return BSP_ERR_INVALID_ARG;
    panel_walk_kernel<true><<<panel_grid(n_panels), 256, 0, stream>>>(
        lut_out, panel_first, n_panels, packed_a, a_sb, a_sr, a_st, packed_b, b_sb, b_st, b_sc, T, nullptr,
        nullptr, nullptr, nullptr, step_offsets, steps_out);
    BSP_LAUNCH_CHECK();
    return BSP_OK;
}
