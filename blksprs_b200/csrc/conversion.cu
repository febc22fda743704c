// Dense <-> compressed conversion (blksprs/ops/conversion.py: to_sparse_kernel :236-276,
// to_dense_kernel :513-557).  Pure data movement: every byte is read once and written once with
// the widest vector access the pointers and row pitches allow (16 bytes normally), in a
// grid-stride loop sized to the SM count.
#include <string.h>

#include "common.cuh"

namespace bsp {

template <int V> struct VecOf;
template <> struct VecOf<16> { using type = uint4; };
template <> struct VecOf<8> { using type = uint2; };
template <> struct VecOf<4> { using type = uint32_t; };
template <> struct VecOf<2> { using type = uint16_t; };
template <> struct VecOf<1> { using type = uint8_t; };

// out[p] = dense[b, r*bs : (r+1)*bs, c*bs : (c+1)*bs] for the p-th LUT row (b, r, c).
// A group of GS threads copies one block: a whole CTA for large blocks, one warp for small ones
// (so that 16 x 16 blocks of 512 bytes still fill the machine).  The writes of a group are
// contiguous, the reads are bs-element row pieces.
template <int V, int GS>
__global__ void __launch_bounds__(256)
to_sparse_kernel(const unsigned char* __restrict__ dense, int64_t rows, int64_t cols,
                 const int64_t* __restrict__ lut, int64_t n, int bs, int elem_bytes,
                 unsigned char* __restrict__ out) {
    using Vec = typename VecOf<V>::type;
    const int64_t row_bytes = (int64_t)bs * elem_bytes;       // one block row
    const int vecs_per_row = (int)(row_bytes / V);
    const int64_t vecs_per_block = (int64_t)bs * vecs_per_row;
    const int64_t pitch = cols * elem_bytes;                   // one dense row
    const int lane = threadIdx.x % GS;
    const int64_t groups = (int64_t)gridDim.x * (256 / GS);
    for (int64_t p = (int64_t)blockIdx.x * (256 / GS) + threadIdx.x / GS; p < n; p += groups) {
        const int64_t b = lut[p * 3 + 0], r = lut[p * 3 + 1], c = lut[p * 3 + 2];
        const unsigned char* src = dense + ((b * rows + r * bs) * cols + c * bs) * elem_bytes;
        unsigned char* dst = out + p * bs * row_bytes;
        for (int64_t i = lane; i < vecs_per_block; i += GS) {
            const int64_t row = i / vecs_per_row, v = i % vecs_per_row;
            *reinterpret_cast<Vec*>(dst + i * V) = *reinterpret_cast<const Vec*>(src + row * pitch + v * V);
        }
    }
}

// dense[b, r*bs.., c*bs..] = x[packed[b, r, c]] where that is >= 0, else the fill value.
// The dense result is cut into tiles of 16 rows x 64 vectors (1 KiB of a row with 16-byte vectors).
// A CTA copies one tile at a time: thread t owns vector column t % 64 and the rows t / 64, +4, +8,
// +12 of the tile.  The four rows of a thread lie in the same block, so one look-up in the reverse
// LUT serves four independent loads; the CTA reads 16 consecutive rows (2 KiB with 64-wide bf16
// blocks) of every block it touches and writes 1 KiB row segments, so both directions reach HBM as
// kilobyte-sized pieces.  Fill value and blocks are written in the same pass.
constexpr int kTileRows = 16, kTileVecs = 64;

template <int V>
__global__ void __launch_bounds__(256)
to_dense_kernel(const unsigned char* __restrict__ x, int64_t n_x, const int64_t* __restrict__ packed,
                int64_t n_block_rows, int64_t C, int bs, int elem_bytes,
                typename VecOf<V>::type fill, unsigned char* __restrict__ dense) {
    using Vec = typename VecOf<V>::type;
    const int64_t row_bytes = (int64_t)bs * elem_bytes;        // one block row
    const int vpb_log2 = __ffs((int)(row_bytes / V)) - 1;      // vectors per block row (power of two)
    const int64_t vecs_per_row = C << vpb_log2;                // one dense row
    const int64_t tiles_per_row = (vecs_per_row + kTileVecs - 1) / kTileVecs;
    const int bands_per_block_row = bs / kTileRows;            // bs is a power of two >= 16
    const int64_t n_tiles = n_block_rows * bands_per_block_row * tiles_per_row;
    const int tv = threadIdx.x % kTileVecs, rg = threadIdx.x / kTileVecs;
    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int64_t band = tile / tiles_per_row;             // 16 dense rows
        const int64_t cv = (tile - band * tiles_per_row) * kTileVecs + tv;
        if (cv >= vecs_per_row) continue;
        const int64_t br = band / bands_per_block_row;         // block row (b * R + r)
        const int row0 = (int)(band - br * bands_per_block_row) * kTileRows + rg;  // row inside the blocks
        const int64_t c = cv >> vpb_log2;
        const int v = (int)(cv & (((int64_t)1 << vpb_log2) - 1));
        const int64_t blk = packed[br * C + c];
        Vec val[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) val[k] = fill;
        if (blk >= 0 && blk < n_x) {
            const unsigned char* src = x + blk * bs * row_bytes + (int64_t)v * V;
#pragma unroll
            for (int k = 0; k < 4; ++k)
                val[k] = *reinterpret_cast<const Vec*>(src + (int64_t)(row0 + 4 * k) * row_bytes);
        }
        unsigned char* dst = dense + ((br * bs + row0) * vecs_per_row + cv) * V;
#pragma unroll
        for (int k = 0; k < 4; ++k)
            *reinterpret_cast<Vec*>(dst + (int64_t)(4 * k) * vecs_per_row * V) = val[k];
    }
}

static int pick_vector(uintptr_t a, uintptr_t b, int64_t pitch_a, int64_t pitch_b) {
    for (int v = 16; v > 1; v >>= 1)
        if (a % v == 0 && b % v == 0 && pitch_a % v == 0 && pitch_b % v == 0) return v;
    return 1;
}

static unsigned copy_grid(int64_t items) {
    const int64_t cap = 148 * 32;
    return (unsigned)(items < cap ? (items < 1 ? 1 : items) : cap);
}

// `fill_bits` replicated to a vector of V bytes (elem_bytes <= V).
template <int V>
static typename VecOf<V>::type make_fill(uint64_t fill_bits, int elem_bytes) {
    unsigned char buf[16];
    for (int i = 0; i < V; ++i) buf[i] = (unsigned char)(fill_bits >> (8 * (i % elem_bytes)));
    typename VecOf<V>::type out;
    memcpy(&out, buf, V);
    return out;
}

}  // namespace bsp

using namespace bsp;

extern "C" int bsp_to_sparse(const void* dense, int64_t B, int64_t rows, int64_t cols, const int64_t* lut,
                             int64_t n, int bs, int elem_bytes, void* out, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (B < 0 || rows < 0 || cols < 0 || n < 0 || bs < 16 || (bs & (bs - 1))) return BSP_ERR_INVALID_ARG;
    if (elem_bytes != 1 && elem_bytes != 2 && elem_bytes != 4 && elem_bytes != 8) return BSP_ERR_UNSUPPORTED;
    if (rows % bs || cols % bs) return BSP_ERR_INVALID_ARG;
    if (n == 0) return BSP_OK;
    if (!dense || !lut || !out) return BSP_ERR_INVALID_ARG;
    const int64_t row_bytes = (int64_t)bs * elem_bytes;
    const int v = pick_vector((uintptr_t)dense, (uintptr_t)out, cols * elem_bytes, row_bytes);
    const bool big = (int64_t)bs * (row_bytes / v) >= 256;   // vectors per block
    const unsigned grid = copy_grid(big ? n : (n + 7) / 8);
    auto src = (const unsigned char*)dense;
    auto dst = (unsigned char*)out;
#define BSP_TO_SPARSE(VV)                                                                                      \
    if (big) to_sparse_kernel<VV, 256><<<grid, 256, 0, stream>>>(src, rows, cols, lut, n, bs, elem_bytes, dst); \
    else to_sparse_kernel<VV, 32><<<grid, 256, 0, stream>>>(src, rows, cols, lut, n, bs, elem_bytes, dst)
    switch (v) {
        case 16: BSP_TO_SPARSE(16); break;
        case 8: BSP_TO_SPARSE(8); break;
        case 4: BSP_TO_SPARSE(4); break;
        case 2: BSP_TO_SPARSE(2); break;
        default: BSP_TO_SPARSE(1); break;
    }
#undef BSP_TO_SPARSE
    BSP_LAUNCH_CHECK();
    return BSP_OK;
}

extern "C" int bsp_to_dense(const void* x, int64_t n_x, const int64_t* packed, int64_t B, int64_t R, int64_t C,
                            int bs, int elem_bytes, uint64_t fill_bits, void* dense, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (B < 0 || R < 0 || C < 0 || n_x < 0 || bs < 16 || (bs & (bs - 1))) return BSP_ERR_INVALID_ARG;
    if (elem_bytes != 1 && elem_bytes != 2 && elem_bytes != 4 && elem_bytes != 8) return BSP_ERR_UNSUPPORTED;
    const int64_t n_cells = B * R * C;
    if (n_cells == 0) return BSP_OK;
    if (!packed || !dense || (n_x > 0 && !x)) return BSP_ERR_INVALID_ARG;
    const int64_t row_bytes = (int64_t)bs * elem_bytes;
    int v = pick_vector(n_x > 0 ? (uintptr_t)x : 0, (uintptr_t)dense, row_bytes, C * row_bytes);
    if (v < elem_bytes) v = elem_bytes;  // pointers are at least element aligned
    const int64_t tiles = B * R * (bs / kTileRows) * ceil_div(C * (row_bytes / v), kTileVecs);
    const unsigned grid = copy_grid(tiles);
    auto src = (const unsigned char*)x;
    auto dst = (unsigned char*)dense;
#define BSP_TO_DENSE(VV)                                                                          \
    to_dense_kernel<VV><<<grid, 256, 0, stream>>>(src, n_x, packed, B * R, C, bs, elem_bytes,      \
                                                  make_fill<VV>(fill_bits, elem_bytes), dst)
    switch (v) {
        case 16: BSP_TO_DENSE(16); break;
        case 8: BSP_TO_DENSE(8); break;
        case 4: BSP_TO_DENSE(4); break;
        case 2: BSP_TO_DENSE(2); break;
        default: BSP_TO_DENSE(1); break;
    }
#undef BSP_TO_DENSE
    BSP_LAUNCH_CHECK();
    return BSP_OK;
}
