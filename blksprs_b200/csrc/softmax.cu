// Row-wise block-sparse softmax, forward and backward, fp32 (blksprs/ops/softmax.py: the regular
// path :93-144 / :157-208 and the fused path :438-520 compute the same function; the reference
// makes up to five passes with intermediate tensors, here one kernel per direction).
//
// One warp per matrix row (batch b, block row r, row i inside the blocks): its lanes walk the row's
// active blocks through the reverse LUT, 128-byte pieces at a time.  Inactive blocks do not take
// part (they count as -inf).  Three sweeps over the row (max, sum of exp, normalise); a row is at
// most a few tens of KiB and the second and third sweep hit L1/L2, so HBM sees each element once
// in and once out.
#include <float.h>

#include "common.cuh"

namespace bsp {

__device__ inline float warp_max(float v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, d));
    return v;
}
__device__ inline float warp_sum(float v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}

// Calls f(element offset in the compressed tensor) for every element of the row that this lane
// owns: lanes split each block row (bs floats) among themselves in float4 pieces.
template <typename F>
__device__ inline void for_row_elements(const int64_t* __restrict__ packed_row, int64_t C, int64_t n_x, int bs,
                                        int row, int lane, F&& f) {
    const int vecs = bs / 4;  // float4 per block row
    for (int64_t c = 0; c < C; ++c) {
        const int64_t blk = packed_row[c];
        if (blk < 0 || blk >= n_x) continue;
        const int64_t base = (blk * bs + row) * bs;
        for (int v = lane; v < vecs; v += 32) f(base + 4 * v);
    }
}

__global__ void __launch_bounds__(256)
softmax_fwd_kernel(const float* __restrict__ x, int64_t n_x, const int64_t* __restrict__ packed, int64_t n_rows,
                   int64_t C, int bs, float* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t w = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); w < n_rows; w += warps) {
        const int64_t br = w / bs;  // b * R + r
        const int row = (int)(w % bs);
        const int64_t* prow = packed + br * C;
        float m = -FLT_MAX;
        for_row_elements(prow, C, n_x, bs, row, lane, [&](int64_t off) {
            const float4 v = *reinterpret_cast<const float4*>(x + off);
            m = fmaxf(fmaxf(m, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
        });
        m = warp_max(m);
        float s = 0.f;
        for_row_elements(prow, C, n_x, bs, row, lane, [&](int64_t off) {
            const float4 v = *reinterpret_cast<const float4*>(x + off);
            s += expf(v.x - m) + expf(v.y - m) + expf(v.z - m) + expf(v.w - m);
        });
        s = warp_sum(s);
        const float inv = 1.f / s;
        for_row_elements(prow, C, n_x, bs, row, lane, [&](int64_t off) {
            const float4 v = *reinterpret_cast<const float4*>(x + off);
            float4 o;
            o.x = expf(v.x - m) * inv;
            o.y = expf(v.y - m) * inv;
            o.z = expf(v.z - m) * inv;
            o.w = expf(v.w - m) * inv;
            *reinterpret_cast<float4*>(out + off) = o;
        });
    }
}

// grad_x = o * (g - sum_row(g * o))
__global__ void __launch_bounds__(256)
softmax_bwd_kernel(const float* __restrict__ g, const float* __restrict__ o, int64_t n_x,
                   const int64_t* __restrict__ packed, int64_t n_rows, int64_t C, int bs,
                   float* __restrict__ grad_x) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t w = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); w < n_rows; w += warps) {
        const int64_t br = w / bs;
        const int row = (int)(w % bs);
        const int64_t* prow = packed + br * C;
        float s = 0.f;
        for_row_elements(prow, C, n_x, bs, row, lane, [&](int64_t off) {
            const float4 a = *reinterpret_cast<const float4*>(g + off);
            const float4 b = *reinterpret_cast<const float4*>(o + off);
            s += a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
        });
        s = warp_sum(s);
        for_row_elements(prow, C, n_x, bs, row, lane, [&](int64_t off) {
            const float4 a = *reinterpret_cast<const float4*>(g + off);
            const float4 b = *reinterpret_cast<const float4*>(o + off);
            float4 r;
            r.x = b.x * (a.x - s);
            r.y = b.y * (a.y - s);
            r.z = b.z * (a.z - s);
            r.w = b.w * (a.w - s);
            *reinterpret_cast<float4*>(grad_x + off) = r;
        });
    }
}

static unsigned softmax_grid(int64_t n_rows) {
    const int64_t blocks = ceil_div(n_rows, 8);
    return (unsigned)(blocks > 148 * 16 ? 148 * 16 : (blocks < 1 ? 1 : blocks));
}

}  // namespace bsp

using namespace bsp;

static int check_softmax_args(int64_t n_x, int64_t B, int64_t R, int64_t C, int bs) {
    if (n_x < 0 || B < 0 || R < 0 || C < 0 || bs < 16 || (bs & (bs - 1))) return BSP_ERR_INVALID_ARG;
    return BSP_OK;
}

extern "C" int bsp_softmax_fwd(const float* x, int64_t n_x, const int64_t* packed, int64_t B, int64_t R, int64_t C,
                               int bs, float* out, void* stream_) {
    int st = check_softmax_args(n_x, B, R, C, bs);
    if (st != BSP_OK) return st;
    const int64_t n_rows = B * R * bs;
    if (n_x == 0 || n_rows == 0 || C == 0) return BSP_OK;
    if (!x || !packed || !out) return BSP_ERR_INVALID_ARG;
    if (((uintptr_t)x | (uintptr_t)out) & 15) return BSP_ERR_INVALID_ARG;
    softmax_fwd_kernel<<<softmax_grid(n_rows), 256, 0, (cudaStream_t)stream_>>>(x, n_x, packed, n_rows, C, bs, out);
    BSP_LAUNCH_CHECK();
    return BSP_OK;
}

extern "C" int bsp_softmax_bwd(const float* grad_out, const float* o, int64_t n_x, const int64_t* packed, int64_t B,
                               int64_t R, int64_t C, int bs, float* grad_x, void* stream_) {
    int st = check_softmax_args(n_x, B, R, C, bs);
    if (st != BSP_OK) return st;
    const int64_t n_rows = B * R * bs;
    if (n_x == 0 || n_rows == 0 || C == 0) return BSP_OK;
    if (!grad_out || !o || !packed || !grad_x) return BSP_ERR_INVALID_ARG;
    if (((uintptr_t)grad_out | (uintptr_t)o | (uintptr_t)grad_x) & 15) return BSP_ERR_INVALID_ARG;
    softmax_bwd_kernel<<<softmax_grid(n_rows), 256, 0, (cudaStream_t)stream_>>>(grad_out, o, n_x, packed, n_rows, C,
                                                                                bs, grad_x);
    BSP_LAUNCH_CHECK();
    return BSP_OK;
}
