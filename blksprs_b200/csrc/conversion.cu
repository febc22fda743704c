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
// Threads walk the dense result in memory order (whole rows, fully coalesced writes); each
// vector looks up the block its column range belongs to.  Four vectors per thread are in flight
// at once; the index arithmetic is 32-bit when the tensor allows it (IDX) and uses shifts for the
// power-of-two block geometry.
template <int V, typename IDX>
__global__ void __launch_bounds__(256)
to_dense_kernel(const unsigned char* __restrict__ x, int64_t n_x, const int64_t* __restrict__ packed,
                int64_t n_cells, int64_t R, int64_t C, int bs, int elem_bytes,
                typename VecOf<V>::type fill, unsigned char* __restrict__ dense) {
    using Vec = typename VecOf<V>::type;
    constexpr int UNROLL = 4;
    const int64_t row_bytes = (int64_t)bs * elem_bytes;        // one block row
    const int vpb_log2 = __ffs((int)(row_bytes / V)) - 1;      // vectors per block row (power of two)
    const int bs_log2 = __ffs(bs) - 1;
    const IDX vecs_per_row = (IDX)(C << vpb_log2);             // one dense row
    const IDX total = (IDX)((n_cells / C) << bs_log2) * vecs_per_row;
    const IDX stride = (IDX)gridDim.x * blockDim.x;
    for (IDX g0 = (IDX)blockIdx.x * blockDim.x + threadIdx.x; g0 < total; g0 += stride * UNROLL) {
        int64_t src_blk[UNROLL];
        IDX off[UNROLL];
#pragma unroll
        for (int k = 0; k < UNROLL; ++k) {
            const IDX g = g0 + (IDX)k * stride;
            src_blk[k] = -1;
            if (g < total) {
                const IDX drow = g / vecs_per_row, cv = g - drow * vecs_per_row;
                const IDX c = cv >> vpb_log2, v = cv & (((IDX)1 << vpb_log2) - 1);
                const IDX br = drow >> bs_log2, row = drow & (IDX)(bs - 1);
                src_blk[k] = packed[(int64_t)br * C + c];
                off[k] = (row << vpb_log2) + v;                // vector index inside the block
            }
        }
        Vec val[UNROLL];
#pragma unroll
        for (int k = 0; k < UNROLL; ++k) {
            val[k] = fill;
            if (src_blk[k] >= 0 && src_blk[k] < n_x)
                val[k] = *reinterpret_cast<const Vec*>(x + (src_blk[k] * bs * row_bytes) + (int64_t)off[k] * V);
        }
#pragma unroll
        for (int k = 0; k < UNROLL; ++k) {
            const IDX g = g0 + (IDX)k * stride;
            if (g < total) *reinterpret_cast<Vec*>(dense + (int64_t)g * V) = val[k];
        }
    }
    (void)R;
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
    const int64_t total_vecs = B * R * bs * (C * row_bytes / v);
    const unsigned grid = copy_grid((total_vecs + 1023) / 1024);
    auto src = (const unsigned char*)x;
    auto dst = (unsigned char*)dense;
    const bool small = total_vecs < 0x7fffffffLL;
#define BSP_TO_DENSE(VV)                                                                                         \
    if (small)                                                                                                   \
        to_dense_kernel<VV, uint32_t><<<grid, 256, 0, stream>>>(src, n_x, packed, n_cells, R, C, bs, elem_bytes,  \
                                                                make_fill<VV>(fill_bits, elem_bytes), dst);       \
    else                                                                                                         \
        to_dense_kernel<VV, int64_t><<<grid, 256, 0, stream>>>(src, n_x, packed, n_cells, R, C, bs, elem_bytes,   \
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
