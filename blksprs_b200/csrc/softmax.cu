// Row-wise block-sparse softmax, forward and backward, fp32 (blksprs/ops/softmax.py: the regular
// path :93-144 / :157-208 and the fused path :438-520 compute the same function; the reference
// makes up to five passes with intermediate tensors, here one kernel per direction).
//
// A CTA takes one block row (batch b, block row r) at a time: it compacts the row's active blocks
// from the reverse LUT into a list in shared memory once, then each of its warps takes matrix rows
// of that block row.  A warp walks a matrix row as one flat sequence of float4 pieces over the
// listed blocks, so all 32 lanes are busy whatever the block size.  The forward pass sweeps a row
// three times (maximum, sum of exp, normalise), the backward pass twice; the repeats hit L1/L2, so
// HBM sees each element once in and once out.  Up to 32 warps per CTA work on consecutive matrix
// rows of the same blocks at the same time, so that HBM is asked for several KiB of a block at once
// (8 warps reached 2.4 TB/s on a 25 % dense 64-block layout, 32 warps 4.3 TB/s).
// Inactive blocks do not take part (they count as -inf).  Block rows with more columns than the
// list holds use the plain kernels at the end of this file (one warp per row walking the LUT).
#include <float.h>
#include <stdint.h>

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

// ---- list-based kernels --------------------------------------------------------------------

// exp through ex2.approx, as the reference's Triton kernels compute it (tl.exp, blksprs/ops/softmax.py:120).
__device__ inline float fast_exp(float v) { return __expf(v); }

constexpr int kListMax = 8192;  // block columns a CTA can list (32 KiB of shared memory)

// Compacts the active blocks of one block row into list[0..n) (column order), by warp 0.
__device__ inline void build_block_list(const int64_t* __restrict__ prow, int64_t C, int64_t n_x,
                                        int32_t* list, int* n_out) {
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        int base = 0;
        for (int64_t c0 = 0; c0 < C; c0 += 32) {
            const int64_t c = c0 + lane;
            const int64_t blk = c < C ? prow[c] : -1;
            const bool ok = blk >= 0 && blk < n_x;
            const unsigned mask = __ballot_sync(0xffffffffu, ok);
            if (ok) list[base + __popc(mask & ((1u << lane) - 1u))] = (int32_t)blk;
            base += __popc(mask);
        }
        if (lane == 0) *n_out = base;
    }
}

// Element offset of float4 piece `idx` of matrix row `row` (pieces numbered through the listed blocks).
__device__ inline int64_t piece_offset(const int32_t* list, int idx, int vpr_log2, int row, int bs) {
    const int blk = list[idx >> vpr_log2];
    const int piece = idx & ((1 << vpr_log2) - 1);
    return ((int64_t)blk * bs + row) * bs + piece * 4;
}

// Four consecutive elements as fp32 (16 bytes of fp32, 8 bytes of a 16-bit type) and back.
template <typename T> __device__ inline float4 load4(const T* p);
template <> __device__ inline float4 load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ inline float4 load4<__half>(const __half* p) {
    const uint2 w = *reinterpret_cast<const uint2*>(p);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&w.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&w.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
template <> __device__ inline float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
    const uint2 w = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
template <typename T> __device__ inline void store4(T* p, float4 v);
template <> __device__ inline void store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ inline void store4<__half>(__half* p, float4 v) {
    const __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}
template <> __device__ inline void store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}

// softmax(scale * x) over the listed blocks of every matrix row; input and output types are free
// (the arithmetic is fp32).  scale = 1 with fp32 in and out is the reference's op.  Two sweeps over a
// row: maximum and sum together (the sum rescaled as the maximum grows), then the result.
template <typename TI, typename TO>
__global__ void __launch_bounds__(1024)
softmax_fwd_list_kernel(const TI* __restrict__ x, int64_t n_x, const int64_t* __restrict__ packed,
                        int64_t n_block_rows, int64_t C, int bs, int vpr_log2, float scale, TO* __restrict__ out) {
    extern __shared__ int32_t list[];
    __shared__ int n_active;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    for (int64_t br = blockIdx.x; br < n_block_rows; br += gridDim.x) {
        __syncthreads();  // the previous block row's readers are done with the list
        build_block_list(packed + br * C, C, n_x, list, &n_active);
        __syncthreads();
        const int total = n_active << vpr_log2;  // pieces of four elements per matrix row
        if (total == 0) continue;
        for (int row = warp; row < bs; row += n_warps) {
            // first sweep: every lane keeps a running maximum and the sum of exp(. - maximum) of its pieces,
            // rescaling the sum whenever the maximum grows; the lanes' pairs are then merged
            float m = -FLT_MAX, s = 0.f;
            for (int idx = lane; idx < total; idx += 32) {
                const float4 v = load4<TI>(x + piece_offset(list, idx, vpr_log2, row, bs));
                const float a = v.x * scale, b = v.y * scale, c = v.z * scale, d = v.w * scale;
                const float mp = fmaxf(fmaxf(a, b), fmaxf(c, d));
                if (mp > m) {
                    s *= fast_exp(m - mp);   // zero on the first piece: exp of a hugely negative number
                    m = mp;
                }
                s += (fast_exp(a - m) + fast_exp(b - m)) + (fast_exp(c - m) + fast_exp(d - m));
            }
            const float m_lane = m;
            m = warp_max(m);
            s = warp_sum(s * fast_exp(m_lane - m));   // lanes without a piece contribute 0 * exp(-huge) = 0
            const float inv = 1.f / s;
            for (int idx = lane; idx < total; idx += 32) {
                const int64_t off = piece_offset(list, idx, vpr_log2, row, bs);
                const float4 v = load4<TI>(x + off);
                float4 o;
                o.x = fast_exp(v.x * scale - m) * inv;
                o.y = fast_exp(v.y * scale - m) * inv;
                o.z = fast_exp(v.z * scale - m) * inv;
                o.w = fast_exp(v.w * scale - m) * inv;
                store4<TO>(out + off, o);
            }
        }
    }
}

// grad_x = scale * o * (g - sum_row(g * o)): the gradient with respect to x of softmax(scale * x), given
// the probabilities o and their gradient g; the three tensors may have different types (fp32 arithmetic).
template <typename TG, typename TP, typename TX>
__global__ void __launch_bounds__(1024)
softmax_bwd_list_kernel(const TG* __restrict__ g, const TP* __restrict__ o, int64_t n_x,
                        const int64_t* __restrict__ packed, int64_t n_block_rows, int64_t C, int bs,
                        int vpr_log2, float scale, TX* __restrict__ grad_x) {
    extern __shared__ int32_t list[];
    __shared__ int n_active;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    for (int64_t br = blockIdx.x; br < n_block_rows; br += gridDim.x) {
        __syncthreads();
        build_block_list(packed + br * C, C, n_x, list, &n_active);
        __syncthreads();
        const int total = n_active << vpr_log2;
        if (total == 0) continue;
        for (int row = warp; row < bs; row += n_warps) {
            float s = 0.f;
            for (int idx = lane; idx < total; idx += 32) {
                const int64_t off = piece_offset(list, idx, vpr_log2, row, bs);
                const float4 a = load4<TG>(g + off);
                const float4 b = load4<TP>(o + off);
                s += (a.x * b.x + a.y * b.y) + (a.z * b.z + a.w * b.w);
            }
            s = warp_sum(s);
            for (int idx = lane; idx < total; idx += 32) {
                const int64_t off = piece_offset(list, idx, vpr_log2, row, bs);
                const float4 a = load4<TG>(g + off);
                const float4 b = load4<TP>(o + off);
                float4 r;
                r.x = b.x * (a.x - s) * scale;
                r.y = b.y * (a.y - s) * scale;
                r.z = b.z * (a.z - s) * scale;
                r.w = b.w * (a.w - s) * scale;
                store4<TX>(grad_x + off, r);
            }
        }
    }
}

// ---- second half of the softmax that is fused into the matmul epilogue -----------------------
// The matmul kernel's softmax epilogue leaves, per output block p and block row r, e = exp(s - m)
// with m = the row's maximum inside that block and l = its sum of e (stats[p][r] = (m, l)).  The
// blocks of one block row of the layout are consecutive in the compressed tensor
// (blocks [row_first[i], row_first[i + 1]) for block row i), so a CTA takes one block row: first the
// row-wide maximum M = max_j m_j and sum L = sum_j l_j exp(m_j - M) of every matrix row, then every
// element once: p = e * exp(m_j - M) / L, converted to the output type.
template <typename T> __device__ inline float to_f32(T v);
template <> __device__ inline float to_f32<float>(float v) { return v; }
template <> __device__ inline float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ inline float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ inline T from_f32(float v);
template <> __device__ inline float from_f32<float>(float v) { return v; }
template <> __device__ inline __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ inline __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
softmax_normalize_kernel(const TI* __restrict__ e, const float2* __restrict__ stats,
                         const int32_t* __restrict__ row_first, int64_t n_block_rows, int bs, int bs_log2,
                         TO* __restrict__ out) {
    extern __shared__ float row_scale[];  // [bs] row maximum M, [bs] 1 / L
    float* row_max = row_scale;
    float* row_inv = row_scale + bs;
    constexpr int V = 8;  // elements per thread and step
    for (int64_t br = blockIdx.x; br < n_block_rows; br += gridDim.x) {
        const int first = row_first[br], n = row_first[br + 1] - first;
        if (n <= 0) continue;
        __syncthreads();  // the previous block row's readers are done with row_scale
        for (int r = threadIdx.x; r < bs; r += blockDim.x) {
            const float2* st = stats + (int64_t)first * bs + r;
            float M = -FLT_MAX;
            for (int j = 0; j < n; ++j) M = fmaxf(M, st[(int64_t)j * bs].x);
            float L = 0.f;
            for (int j = 0; j < n; ++j) {
                const float2 ml = st[(int64_t)j * bs];
                L += ml.y * fast_exp(ml.x - M);
            }
            row_max[r] = M;
            row_inv[r] = 1.f / L;
        }
        __syncthreads();
        const int64_t base = (int64_t)first * bs * bs;
        const int64_t total = (int64_t)n * bs * bs;
        for (int64_t i = (int64_t)threadIdx.x * V; i < total; i += (int64_t)blockDim.x * V) {
            const int64_t row_index = i >> bs_log2;             // (block j, matrix row r) = j * bs + r
            const int r = (int)(row_index & (bs - 1));
            const float f = fast_exp(stats[(int64_t)first * bs + row_index].x - row_max[r]) * row_inv[r];
            TI in[V];
            TO o[V];
            if constexpr (sizeof(TI) == 2) {
                *reinterpret_cast<uint4*>(in) = *reinterpret_cast<const uint4*>(e + base + i);
            } else {
                *reinterpret_cast<uint4*>(in) = *reinterpret_cast<const uint4*>(e + base + i);
                *reinterpret_cast<uint4*>(in + 4) = *reinterpret_cast<const uint4*>(e + base + i + 4);
            }
#pragma unroll
            for (int k = 0; k < V; ++k) o[k] = from_f32<TO>(to_f32<TI>(in[k]) * f);
            if constexpr (sizeof(TO) == 2) {
                *reinterpret_cast<uint4*>(out + base + i) = *reinterpret_cast<const uint4*>(o);
            } else {
                *reinterpret_cast<uint4*>(out + base + i) = *reinterpret_cast<const uint4*>(o);
                *reinterpret_cast<uint4*>(out + base + i + 4) = *reinterpret_cast<const uint4*>(o + 4);
            }
        }
    }
}

template <typename TI>
static int launch_normalize_out(int out_dtype, const void* e, const float* stats, const int32_t* row_first,
                                int64_t n_block_rows, int bs, void* out, cudaStream_t stream) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t cap = (int64_t)sms * 8;
    const unsigned grid = (unsigned)(n_block_rows < cap ? n_block_rows : cap);
    int bs_log2 = 0;
    while ((1 << bs_log2) < bs) ++bs_log2;
    const size_t smem = 2 * (size_t)bs * sizeof(float);
    const float2* st = reinterpret_cast<const float2*>(stats);
    switch (out_dtype) {
        case BSP_F16:
            softmax_normalize_kernel<TI, __half><<<grid, 256, smem, stream>>>((const TI*)e, st, row_first, n_block_rows, bs, bs_log2, (__half*)out);
            break;
        case BSP_BF16:
            softmax_normalize_kernel<TI, __nv_bfloat16><<<grid, 256, smem, stream>>>((const TI*)e, st, row_first, n_block_rows, bs, bs_log2, (__nv_bfloat16*)out);
            break;
        case BSP_F32:
            softmax_normalize_kernel<TI, float><<<grid, 256, smem, stream>>>((const TI*)e, st, row_first, n_block_rows, bs, bs_log2, (float*)out);
            break;
        default: return BSP_ERR_UNSUPPORTED;
    }
    BSP_LAUNCH_CHECK();
    return BSP_OK;
}

// Warps per CTA: enough matrix rows of a block in flight together that HBM sees kilobytes of each
// block at a time (measured: 32 warps for block size >= 64, fewer for the short rows of small blocks).
static int list_warps(int bs) {
    const int w = bs / 2;
    return w < 8 ? 8 : (w > 32 ? 32 : w);
}

static int log2_int(int v) {
    int l = 0;
    while ((1 << l) < v) ++l;
    return l;
}

static unsigned list_grid(int64_t n_block_rows, int warps) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t cap = (int64_t)sms * (64 / warps);  // the CTAs that are resident at once
    return (unsigned)(n_block_rows < cap ? (n_block_rows < 1 ? 1 : n_block_rows) : cap);
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
    if (C <= kListMax && n_x <= INT32_MAX) {
        softmax_fwd_list_kernel<float, float><<<list_grid(B * R, list_warps(bs)), 32 * list_warps(bs), (size_t)C * sizeof(int32_t), (cudaStream_t)stream_>>>(
            x, n_x, packed, B * R, C, bs, log2_int(bs / 4), 1.0f, out);
    } else {
        softmax_fwd_kernel<<<softmax_grid(n_rows), 256, 0, (cudaStream_t)stream_>>>(x, n_x, packed, n_rows, C, bs, out);
    }
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
    if (C <= kListMax && n_x <= INT32_MAX) {
        softmax_bwd_list_kernel<float, float, float><<<list_grid(B * R, list_warps(bs)), 32 * list_warps(bs), (size_t)C * sizeof(int32_t), (cudaStream_t)stream_>>>(
            grad_out, o, n_x, packed, B * R, C, bs, log2_int(bs / 4), 1.0f, grad_x);
    } else {
        softmax_bwd_kernel<<<softmax_grid(n_rows), 256, 0, (cudaStream_t)stream_>>>(grad_out, o, n_x, packed, n_rows,
                                                                                    C, bs, grad_x);
    }
    BSP_LAUNCH_CHECK();
    return BSP_OK;
}

template <typename TI, typename TO>
static int launch_softmax_scaled(const void* x, int64_t n_x, const int64_t* packed, int64_t B, int64_t R, int64_t C,
                                 int bs, float scale, void* out, cudaStream_t stream) {
    softmax_fwd_list_kernel<TI, TO><<<list_grid(B * R, list_warps(bs)), 32 * list_warps(bs), (size_t)C * sizeof(int32_t), stream>>>(
        (const TI*)x, n_x, packed, B * R, C, bs, log2_int(bs / 4), scale, (TO*)out);
    BSP_LAUNCH_CHECK();
    return BSP_OK;
}
template <typename TI>
static int launch_softmax_scaled_out(int out_dtype, const void* x, int64_t n_x, const int64_t* packed, int64_t B,
                                     int64_t R, int64_t C, int bs, float scale, void* out, cudaStream_t stream) {
    switch (out_dtype) {
        case BSP_F16: return launch_softmax_scaled<TI, __half>(x, n_x, packed, B, R, C, bs, scale, out, stream);
        case BSP_BF16: return launch_softmax_scaled<TI, __nv_bfloat16>(x, n_x, packed, B, R, C, bs, scale, out, stream);
        case BSP_F32: return launch_softmax_scaled<TI, float>(x, n_x, packed, B, R, C, bs, scale, out, stream);
        default: return BSP_ERR_UNSUPPORTED;
    }
}

extern "C" int bsp_softmax_fwd_scaled(const void* x, int in_dtype, int64_t n_x, const int64_t* packed, int64_t B,
                                      int64_t R, int64_t C, int bs, float scale, void* out, int out_dtype,
                                      void* stream_) {
    int st = check_softmax_args(n_x, B, R, C, bs);
    if (st != BSP_OK) return st;
    if (n_x == 0 || B * R == 0 || C == 0) return BSP_OK;
    if (!x || !packed || !out) return BSP_ERR_INVALID_ARG;
    if (((uintptr_t)x | (uintptr_t)out) & 15) return BSP_ERR_INVALID_ARG;
    if (C > kListMax || n_x > INT32_MAX) return BSP_ERR_UNSUPPORTED;
    cudaStream_t stream = (cudaStream_t)stream_;
    switch (in_dtype) {
        case BSP_F16: return launch_softmax_scaled_out<__half>(out_dtype, x, n_x, packed, B, R, C, bs, scale, out, stream);
        case BSP_BF16: return launch_softmax_scaled_out<__nv_bfloat16>(out_dtype, x, n_x, packed, B, R, C, bs, scale, out, stream);
        case BSP_F32: return launch_softmax_scaled_out<float>(out_dtype, x, n_x, packed, B, R, C, bs, scale, out, stream);
        default: return BSP_ERR_UNSUPPORTED;
    }
}

template <typename TG, typename TP, typename TX>
static int launch_softmax_bwd_scaled(const void* g, const void* o, int64_t n_x, const int64_t* packed, int64_t B,
                                     int64_t R, int64_t C, int bs, float scale, void* grad_x, cudaStream_t stream) {
    softmax_bwd_list_kernel<TG, TP, TX><<<list_grid(B * R, list_warps(bs)), 32 * list_warps(bs), (size_t)C * sizeof(int32_t), stream>>>(
        (const TG*)g, (const TP*)o, n_x, packed, B * R, C, bs, log2_int(bs / 4), scale, (TX*)grad_x);
    BSP_LAUNCH_CHECK();
    return BSP_OK;
}
template <typename TG, typename TP>
static int launch_softmax_bwd_scaled_x(int x_dtype, const void* g, const void* o, int64_t n_x, const int64_t* packed,
                                       int64_t B, int64_t R, int64_t C, int bs, float scale, void* grad_x,
                                       cudaStream_t stream) {
    switch (x_dtype) {
        case BSP_F16: return launch_softmax_bwd_scaled<TG, TP, __half>(g, o, n_x, packed, B, R, C, bs, scale, grad_x, stream);
        case BSP_BF16: return launch_softmax_bwd_scaled<TG, TP, __nv_bfloat16>(g, o, n_x, packed, B, R, C, bs, scale, grad_x, stream);
        case BSP_F32: return launch_softmax_bwd_scaled<TG, TP, float>(g, o, n_x, packed, B, R, C, bs, scale, grad_x, stream);
        default: return BSP_ERR_UNSUPPORTED;
    }
}
template <typename TG>
static int launch_softmax_bwd_scaled_p(int p_dtype, int x_dtype, const void* g, const void* o, int64_t n_x,
                                       const int64_t* packed, int64_t B, int64_t R, int64_t C, int bs, float scale,
                                       void* grad_x, cudaStream_t stream) {
    switch (p_dtype) {
        case BSP_F16: return launch_softmax_bwd_scaled_x<TG, __half>(x_dtype, g, o, n_x, packed, B, R, C, bs, scale, grad_x, stream);
        case BSP_BF16: return launch_softmax_bwd_scaled_x<TG, __nv_bfloat16>(x_dtype, g, o, n_x, packed, B, R, C, bs, scale, grad_x, stream);
        case BSP_F32: return launch_softmax_bwd_scaled_x<TG, float>(x_dtype, g, o, n_x, packed, B, R, C, bs, scale, grad_x, stream);
        default: return BSP_ERR_UNSUPPORTED;
    }
}

extern "C" int bsp_softmax_bwd_scaled(const void* grad_out, int g_dtype, const void* o, int o_dtype, int64_t n_x,
                                      const int64_t* packed, int64_t B, int64_t R, int64_t C, int bs, float scale,
                                      void* grad_x, int x_dtype, void* stream_) {
    int st = check_softmax_args(n_x, B, R, C, bs);
    if (st != BSP_OK) return st;
    if (n_x == 0 || B * R == 0 || C == 0) return BSP_OK;
    if (!grad_out || !o || !packed || !grad_x) return BSP_ERR_INVALID_ARG;
    if (((uintptr_t)grad_out | (uintptr_t)o | (uintptr_t)grad_x) & 15) return BSP_ERR_INVALID_ARG;
    if (C > kListMax || n_x > INT32_MAX) return BSP_ERR_UNSUPPORTED;
    cudaStream_t stream = (cudaStream_t)stream_;
    switch (g_dtype) {
        case BSP_F16: return launch_softmax_bwd_scaled_p<__half>(o_dtype, x_dtype, grad_out, o, n_x, packed, B, R, C, bs, scale, grad_x, stream);
        case BSP_BF16: return launch_softmax_bwd_scaled_p<__nv_bfloat16>(o_dtype, x_dtype, grad_out, o, n_x, packed, B, R, C, bs, scale, grad_x, stream);
        case BSP_F32: return launch_softmax_bwd_scaled_p<float>(o_dtype, x_dtype, grad_out, o, n_x, packed, B, R, C, bs, scale, grad_x, stream);
        default: return BSP_ERR_UNSUPPORTED;
    }
}

extern "C" int bsp_softmax_normalize(const void* e, int in_dtype, const float* stats, int64_t n_blocks,
                                     const int32_t* row_first, int64_t n_block_rows, int bs, void* out,
                                     int out_dtype, void* stream_) {
    if (n_blocks < 0 || n_block_rows < 0 || bs < 16 || (bs & (bs - 1)) || bs > 4096) return BSP_ERR_INVALID_ARG;
    if (n_blocks == 0 || n_block_rows == 0) return BSP_OK;
    if (!e || !stats || !row_first || !out) return BSP_ERR_INVALID_ARG;
    if (n_blocks > INT32_MAX) return BSP_ERR_UNSUPPORTED;
    if (((uintptr_t)e | (uintptr_t)out) & 15 || ((uintptr_t)stats & 7)) return BSP_ERR_INVALID_ARG;
    cudaStream_t stream = (cudaStream_t)stream_;
    switch (in_dtype) {
        case BSP_F16: return launch_normalize_out<__half>(out_dtype, e, stats, row_first, n_block_rows, bs, out, stream);
        case BSP_BF16: return launch_normalize_out<__nv_bfloat16>(out_dtype, e, stats, row_first, n_block_rows, bs, out, stream);
        case BSP_F32: return launch_normalize_out<float>(out_dtype, e, stats, row_first, n_block_rows, bs, out, stream);
        default: return BSP_ERR_UNSUPPORTED;
    }
}
