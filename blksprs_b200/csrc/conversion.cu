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
template <int V>
__global__ void __launch_bounds__(256)
to_sparse_kernel(const unsigned char* __restrict__ dense, int64_t rows, int64_t cols,
                 const int64_t* __restrict__ lut, int64_t n, int bs, int elem_bytes,
                 unsigned char* __restrict__ out) {
    using Vec = typename VecOf<V>::type;
    const int64_t row_bytes = (int64_t)bs * elem_bytes;       // one block row
    const int vecs_per_row = (int)(row_bytes / V);
    const int64_t vecs_per_block = (int64_t)bs * vecs_per_row;
    const int64_t pitch = cols * elem_bytes;                   // one dense row
    for (int64_t p = blockIdx.x; p < n; p += gridDim.x) {
        const int64_t b = lut[p * 3 + 0], r = lut[p * 3 + 1], c = lut[p * 3 + 2];
        const unsigned char* src = dense + ((b * rows + r * bs) * cols + c * bs) * elem_bytes;
        unsigned char* dst = out + p * bs * row_bytes;
        for (int64_t i = threadIdx.x; i < vecs_per_block; i += blockDim.x) {
            const int64_t row = i / vecs_per_row, v = i % vecs_per_row;
            *reinterpret_cast<Vec*>(dst + row * row_bytes + v * V) =
                *reinterpret_cast<const Vec*>(src + row * pitch + v * V);
        }
    }
}

// dense[b, r*bs.., c*bs..] = x[packed[b, r, c]] where that is >= 0, else the fill value.
template <int V>
__global__ void __launch_bounds__(256)
to_dense_kernel(const unsigned char* __restrict__ x, int64_t n_x, const int64_t* __restrict__ packed,
                int64_t n_cells, int64_t R, int64_t C, int bs, int elem_bytes,
                typename VecOf<V>::type fill, unsigned char* __restrict__ dense) {
    using Vec = typename VecOf<V>::type;
    const int64_t row_bytes = (int64_t)bs * elem_bytes;
    const int vecs_per_row = (int)(row_bytes / V);
    const int64_t vecs_per_block = (int64_t)bs * vecs_per_row;
    const int64_t pitch = C * row_bytes;
    for (int64_t cell = blockIdx.x; cell < n_cells; cell += gridDim.x) {
        const int64_t c = cell % C, br = cell / C;  // br = b * R + r
        const int64_t src_blk = packed[cell];
        unsigned char* dst = dense + (br * bs) * pitch + c * row_bytes;
        if (src_blk >= 0 && src_blk < n_x) {
            const unsigned char* src = x + src_blk * bs * row_bytes;
            for (int64_t i = threadIdx.x; i < vecs_per_block; i += blockDim.x) {
                const int64_t row = i / vecs_per_row, v = i % vecs_per_row;
                *reinterpret_cast<Vec*>(dst + row * pitch + v * V) =
                    *reinterpret_cast<const Vec*>(src + row * row_bytes + v * V);
            }
        } else {
            for (int64_t i = threadIdx.x; i < vecs_per_block; i += blockDim.x) {
                const int64_t row = i / vecs_per_row, v = i % vecs_per_row;
                *reinterpret_cast<Vec*>(dst + row * pitch + v * V) = fill;
            }
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
    const int64_t cap = 148 * 16;
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
    const unsigned grid = copy_grid(n);
    auto src = (const unsigned char*)dense;
    auto dst = (unsigned char*)out;
    switch (v) {
        case 16: to_sparse_kernel<16><<<grid, 256, 0, stream>>>(src, rows, cols, lut, n, bs, elem_bytes, dst); break;
        case 8: to_sparse_kernel<8><<<grid, 256, 0, stream>>>(src, rows, cols, lut, n, bs, elem_bytes, dst); break;
        case 4: to_sparse_kernel<4><<<grid, 256, 0, stream>>>(src, rows, cols, lut, n, bs, elem_bytes, dst); break;
        case 2: to_sparse_kernel<2><<<grid, 256, 0, stream>>>(src, rows, cols, lut, n, bs, elem_bytes, dst); break;
        default: to_sparse_kernel<1><<<grid, 256, 0, stream>>>(src, rows, cols, lut, n, bs, elem_bytes, dst); break;
    }
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
    const unsigned grid = copy_grid(n_cells);
    auto src = (const unsigned char*)x;
    auto dst = (unsigned char*)dense;
    switch (v) {
        case 16: to_dense_kernel<16><<<grid, 256, 0, stream>>>(src, n_x, packed, n_cells, R, C, bs, elem_bytes, make_fill<16>(fill_bits, elem_bytes), dst); break;
        case 8: to_dense_kernel<8><<<grid, 256, 0, stream>>>(src, n_x, packed, n_cells, R, C, bs, elem_bytes, make_fill<8>(fill_bits, elem_bytes), dst); break;
        case 4: to_dense_kernel<4><<<grid, 256, 0, stream>>>(src, n_x, packed, n_cells, R, C, bs, elem_bytes, make_fill<4>(fill_bits, elem_bytes), dst); break;
        case 2: to_dense_kernel<2><<<grid, 256, 0, stream>>>(src, n_x, packed, n_cells, R, C, bs, elem_bytes, make_fill<2>(fill_bits, elem_bytes), dst); break;
        default: to_dense_kernel<1><<<grid, 256, 0, stream>>>(src, n_x, packed, n_cells, R, C, bs, elem_bytes, make_fill<1>(fill_bits, elem_bytes), dst); break;
    }
    BSP_LAUNCH_CHECK();
    return BSP_OK;
}
