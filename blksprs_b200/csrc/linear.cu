// Kernels around the matmul of the sparse linear helper (blksprs/utils/processing.py:26-202):
// the bias of the layer and the reduction of a weight gradient that was computed in chunks.
//
// The reference adds the bias by materialising it once per output block (to_sparse of a repeated
// slice, then `repeat` over the whole output layout, processing.py:72-84) and adding the two
// tensors.  Here the bias stays a vector: one pass reads the product, adds bias[column] and writes
// the result; the gradient of the bias is the column sum of the output gradient, one pass as well.
#include "common.cuh"

namespace bsp {
namespace {

template <typename T> struct Vec;  // 16 bytes of T
template <> struct Vec<float> { static constexpr int N = 4; };
template <> struct Vec<__half> { static constexpr int N = 8; };
template <> struct Vec<__nv_bfloat16> { static constexpr int N = 8; };

template <typename T> __device__ inline float to_f32(T v);
template <> __device__ inline float to_f32<float>(float v) { return v; }
template <> __device__ inline float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ inline float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ inline T from_f32(float v);
template <> __device__ inline float from_f32<float>(float v) { return v; }
template <> __device__ inline __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ inline __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// out[p, r, c] = x[p, r, c] + bias[col(p) * bs + c]; one 16-byte piece per thread and step.
template <typename T>
__global__ void __launch_bounds__(256)
bias_add_kernel(const T* __restrict__ x, const int64_t* __restrict__ lut, int64_t n_blocks, int bs,
                const T* __restrict__ bias, int64_t n_cols, T* __restrict__ out) {
    constexpr int V = Vec<T>::N;
    const int vec_per_row = bs / V;
    const int64_t vec_per_block = (int64_t)bs * vec_per_row;
    const int64_t total = n_blocks * vec_per_block;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t p = i / vec_per_block;
        const int c = (int)(i % vec_per_row) * V;
        const int64_t col = lut[p * 3 + 2] * bs + c;
        uint4 xv = reinterpret_cast<const uint4*>(x)[i];
        uint4 bv = make_uint4(0, 0, 0, 0);
        if (col >= 0 && col + V <= n_cols) bv = *reinterpret_cast<const uint4*>(bias + col);
        T* xe = reinterpret_cast<T*>(&xv);
        const T* be = reinterpret_cast<const T*>(&bv);
#pragma unroll
        for (int e = 0; e < V; ++e) xe[e] = from_f32<T>(to_f32<T>(xe[e]) + to_f32<T>(be[e]));
        reinterpret_cast<uint4*>(out)[i] = xv;
    }
}

// grad_bias[col(p) * bs + c] += sum_r g[p, r, c], fp32.  A CTA takes whole blocks: its threads
// split the rows, every thread sums 16-byte pieces of one column group, shared memory folds the
// row groups, and one atomic per column and block goes to memory.
template <typename T>
__global__ void __launch_bounds__(256)
bias_grad_kernel(const T* __restrict__ g, const int64_t* __restrict__ lut, int64_t n_blocks, int bs,
                 float* __restrict__ grad_bias, int64_t n_cols) {
    constexpr int V = Vec<T>::N;
    __shared__ float part[256 * 8];
    const int vec_per_row = bs / V;              // threads along a row
    const int row_groups = 256 / vec_per_row;    // rows taken per sweep (bs >= 16: at most 128 threads per row)
    const int cg = threadIdx.x % vec_per_row;
    const int rg = threadIdx.x / vec_per_row;
    for (int64_t p = blockIdx.x; p < n_blocks; p += gridDim.x) {
        float acc[V];
#pragma unroll
        for (int e = 0; e < V; ++e) acc[e] = 0.f;
        const T* blk = g + p * bs * bs;
        for (int r = rg; r < bs; r += row_groups) {
            const uint4 v = *reinterpret_cast<const uint4*>(blk + (int64_t)r * bs + cg * V);
            const T* ve = reinterpret_cast<const T*>(&v);
#pragma unroll
            for (int e = 0; e < V; ++e) acc[e] += to_f32<T>(ve[e]);
        }
#pragma unroll
        for (int e = 0; e < V; ++e) part[threadIdx.x * 8 + e] = acc[e];
        __syncthreads();
        // one thread per column folds the row groups
        for (int c = threadIdx.x; c < bs; c += 256) {
            float s = 0.f;
            for (int q = 0; q < row_groups; ++q) s += part[(q * vec_per_row + c / V) * 8 + c % V];
            const int64_t col = lut[p * 3 + 2] * bs + c;
            if (col >= 0 && col < n_cols) atomicAdd(grad_bias + col, s);
        }
        __syncthreads();
    }
}

// out[i] = sum_s parts[s, i] in fp32, rounded once.
template <typename T>
__global__ void __launch_bounds__(256)
sum_chunks_kernel(const T* __restrict__ parts, int64_t n_chunks, int64_t numel, T* __restrict__ out) {
    constexpr int V = Vec<T>::N;
    const int64_t vecs = numel / V;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += stride) {
        float acc[V];
#pragma unroll
        for (int e = 0; e < V; ++e) acc[e] = 0.f;
        for (int64_t s = 0; s < n_chunks; ++s) {
            const uint4 v = reinterpret_cast<const uint4*>(parts + s * numel)[i];
            const T* ve = reinterpret_cast<const T*>(&v);
#pragma unroll
            for (int e = 0; e < V; ++e) acc[e] += to_f32<T>(ve[e]);
        }
        uint4 o;
        T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
        for (int e = 0; e < V; ++e) oe[e] = from_f32<T>(acc[e]);
        reinterpret_cast<uint4*>(out)[i] = o;
    }
}

int grid_for(int64_t work_items) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t want = ceil_div(work_items, 256);
    const int64_t cap = (int64_t)sms * 8;
    return (int)(want < cap ? (want < 1 ? 1 : want) : cap);
}

bool block_size_ok(int bs) { return bs >= 16 && bs <= 1024 && (bs & (bs - 1)) == 0; }

template <typename F>
bool dispatch_data_dtype(int dtype, F&& f) {
    switch (dtype) {
        case BSP_F16: f(__half{}); return true;
        case BSP_BF16: f(__nv_bfloat16{}); return true;
        case BSP_F32: f(float{}); return true;
        default: return false;
    }
}

}  // namespace
}  // namespace bsp

using namespace bsp;

extern "C" int bsp_bias_add(const void* x, const int64_t* lut, int64_t n_blocks, int bs, const void* bias,
                            int64_t n_cols, int dtype, void* out, void* stream_) {
    if (n_blocks < 0 || n_cols < 0 || !block_size_ok(bs)) return BSP_ERR_INVALID_ARG;
    if (n_blocks == 0) return BSP_OK;
    if (!x || !lut || !bias || !out || n_cols % bs) return BSP_ERR_INVALID_ARG;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(bias)) & 15)
        return BSP_ERR_INVALID_ARG;
    cudaStream_t stream = (cudaStream_t)stream_;
    const bool ok = dispatch_data_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        const int64_t vecs = n_blocks * bs * (bs / Vec<T>::N);
        bias_add_kernel<T><<<grid_for(vecs), 256, 0, stream>>>((const T*)x, lut, n_blocks, bs, (const T*)bias, n_cols,
                                                               (T*)out);
    });
    if (!ok) return BSP_ERR_UNSUPPORTED;
    BSP_LAUNCH_CHECK();
    return BSP_OK;
}

extern "C" int bsp_bias_grad(const void* grad_out, const int64_t* lut, int64_t n_blocks, int bs, int dtype,
                             float* grad_bias, int64_t n_cols, void* stream_) {
    if (n_blocks < 0 || n_cols < 0 || !block_size_ok(bs)) return BSP_ERR_INVALID_ARG;
    if (n_blocks == 0) return BSP_OK;
    if (!grad_out || !lut || !grad_bias || n_cols % bs) return BSP_ERR_INVALID_ARG;
    if (reinterpret_cast<uintptr_t>(grad_out) & 15) return BSP_ERR_INVALID_ARG;
    cudaStream_t stream = (cudaStream_t)stream_;
    const bool ok = dispatch_data_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        if (bs / Vec<T>::N > 256) return;  // rows wider than the CTA are not supported (bs <= 1024 for fp32)
        bias_grad_kernel<T><<<grid_for(n_blocks * 256), 256, 0, stream>>>((const T*)grad_out, lut, n_blocks, bs,
                                                                         grad_bias, n_cols);
    });
    if (!ok) return BSP_ERR_UNSUPPORTED;
    BSP_LAUNCH_CHECK();
    return BSP_OK;
}

extern "C" int bsp_sum_chunks(const void* parts, int64_t n_chunks, int64_t numel, int dtype, void* out,
                              void* stream_) {
    if (n_chunks < 1 || numel < 0) return BSP_ERR_INVALID_ARG;
    if (numel == 0) return BSP_OK;
    if (!parts || !out || numel % 8) return BSP_ERR_INVALID_ARG;
    if ((reinterpret_cast<uintptr_t>(parts) | reinterpret_cast<uintptr_t>(out)) & 15) return BSP_ERR_INVALID_ARG;
    cudaStream_t stream = (cudaStream_t)stream_;
    const bool ok = dispatch_data_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        sum_chunks_kernel<T><<<grid_for(numel / Vec<T>::N), 256, 0, stream>>>((const T*)parts, n_chunks, numel,
                                                                             (T*)out);
    });
    if (!ok) return BSP_ERR_UNSUPPORTED;
    BSP_LAUNCH_CHECK();
    return BSP_OK;
}
