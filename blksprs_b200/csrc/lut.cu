// LUT, reverse-LUT, output-layout inference, pair-plan and compressed-transpose
// kernels.  All of this is HBM/latency-bound integer work on arrays of at most
// a few million entries; the kernels are written for coalesced access and a
// three-phase (reduce, scan chunk sums, apply) prefix sum.
#include <limits.h>

#include <mutex>

#include "common.cuh"

namespace bsp {

static constexpr int kScanThreads = 256;
static constexpr int kScanItems = 8;
static constexpr int kScanChunk = kScanThreads * kScanItems;  // 2048 entries per CTA

enum ScanView { kViewI64 = 0, kViewNonzero = 1 };

template <typename T, int VIEW>
__device__ inline int64_t view_value(T v) {
    if (VIEW == kViewI64) return LayoutElem<T>::as_i64(v);
    return LayoutElem<T>::nonzero(v) ? 1 : 0;
}

__device__ inline int64_t warp_inclusive_scan(int64_t v) {
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        int64_t o = __shfl_up_sync(0xffffffffu, v, d);
        if ((threadIdx.x & 31) >= d) v += o;
    }
    return v;
}

// Exclusive scan of one value per thread over a CTA of kScanThreads threads;
// returns the exclusive prefix, writes the CTA total to *total.
__device__ inline int64_t block_exclusive_scan(int64_t v, int64_t* total) {
    __shared__ int64_t warp_sums[kScanThreads / 32];
    __shared__ int64_t block_total;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int64_t inc = warp_inclusive_scan(v);
    if (lane == 31) warp_sums[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int64_t w = lane < kScanThreads / 32 ? warp_sums[lane] : 0;
        int64_t winc = warp_inclusive_scan(w);
        if (lane < kScanThreads / 32) warp_sums[lane] = winc - w;
        if (lane == kScanThreads / 32 - 1) block_total = winc;
    }
    __syncthreads();
    int64_t res = warp_sums[warp] + inc - v;
    *total = block_total;
    __syncthreads();
    return res;
}

// Phase 1: per-chunk sum of the viewed layout values -> chunk_sums[chunk].
template <typename T, int VIEW>
__global__ void __launch_bounds__(kScanThreads)
chunk_reduce_kernel(const T* __restrict__ layout, int64_t numel, int64_t* __restrict__ chunk_sums) {
    const int64_t base = (int64_t)blockIdx.x * kScanChunk;
    int64_t s = 0;
#pragma unroll
    for (int i = 0; i < kScanItems; ++i) {
        int64_t e = base + (int64_t)i * kScanThreads + threadIdx.x;
        if (e < numel) s += view_value<T, VIEW>(layout[e]);
    }
    int64_t total;
    block_exclusive_scan(s, &total);
    if (threadIdx.x == 0) chunk_sums[blockIdx.x] = total;
}

// Phase 2: in-place exclusive scan of the chunk sums by one CTA; the grand
// total goes to chunk_sums[n_chunks] and, if given, to *total_out.
__global__ void __launch_bounds__(kScanThreads)
chunk_scan_kernel(int64_t* __restrict__ chunk_sums, int64_t n_chunks, int64_t* __restrict__ total_out) {
    int64_t carry = 0;
    for (int64_t base = 0; base < n_chunks; base += kScanThreads) {
        int64_t i = base + threadIdx.x;
        int64_t v = i < n_chunks ? chunk_sums[i] : 0;
        int64_t total;
        int64_t ex = block_exclusive_scan(v, &total);
        if (i < n_chunks) chunk_sums[i] = carry + ex;
        carry += total;
    }
    if (threadIdx.x == 0) {
        chunk_sums[n_chunks] = carry;
        if (total_out) *total_out = carry;
    }
}

// Phase 3a: reverse LUT.  Each thread owns kScanItems consecutive entries.
template <typename T>
__global__ void __launch_bounds__(kScanThreads)
packed_apply_kernel(const T* __restrict__ layout, int64_t numel,
                    const int64_t* __restrict__ chunk_offsets, int64_t* __restrict__ packed) {
    const int64_t base = (int64_t)blockIdx.x * kScanChunk + (int64_t)threadIdx.x * kScanItems;
    int64_t v[kScanItems];
    int64_t s = 0;
#pragma unroll
    for (int i = 0; i < kScanItems; ++i) {
        int64_t e = base + i;
        v[i] = e < numel ? LayoutElem<T>::as_i64(layout[e]) : 0;
        s += v[i];
    }
    int64_t total;
    int64_t run = chunk_offsets[blockIdx.x] + block_exclusive_scan(s, &total);
#pragma unroll
    for (int i = 0; i < kScanItems; ++i) {
        int64_t e = base + i;
        run += v[i];  // inclusive cumulative sum at e
        if (e < numel) packed[e] = (v[i] == 1) ? run - 1 : -1;
    }
}

// Phase 3b: LUT rows (batch,row,col) of the non-zero entries in row-major order.
template <typename T>
__global__ void __launch_bounds__(kScanThreads)
lut_apply_kernel(const T* __restrict__ layout, int64_t numel, int64_t R, int64_t C,
                 const int64_t* __restrict__ chunk_offsets, int64_t* __restrict__ lut,
                 int64_t capacity_rows) {
    const int64_t base = (int64_t)blockIdx.x * kScanChunk + (int64_t)threadIdx.x * kScanItems;
    bool nz[kScanItems];
    int64_t s = 0;
#pragma unroll
    for (int i = 0; i < kScanItems; ++i) {
        int64_t e = base + i;
        nz[i] = e < numel ? LayoutElem<T>::nonzero(layout[e]) : false;
        s += nz[i] ? 1 : 0;
    }
    int64_t total;
    int64_t rank = chunk_offsets[blockIdx.x] + block_exclusive_scan(s, &total);
#pragma unroll
    for (int i = 0; i < kScanItems; ++i) {
        if (nz[i]) {
            if (rank < capacity_rows) {
                int64_t e = base + i;
                int64_t c = e % C;
                int64_t br = e / C;
                lut[rank * 3 + 0] = br / R;
                lut[rank * 3 + 1] = br % R;
                lut[rank * 3 + 2] = c;
            }
            ++rank;
        }
    }
}

static inline int64_t scan_chunks(int64_t numel) { return ceil_div(numel, kScanChunk); }

// ---- output-layout inference ------------------------------------------------
template <typename TX, typename TY>
__global__ void layout_matmul_kernel(const TX* __restrict__ lx, const TY* __restrict__ ly,
                                     int64_t B, int64_t R, int64_t K, int64_t C, int mode,
                                     uint8_t* __restrict__ out) {
    const int64_t total = B * R * C;
    for (int64_t o = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; o < total;
         o += (int64_t)gridDim.x * blockDim.x) {
        const int64_t c = o % C;
        const int64_t br = o / C;
        const int64_t b = br / R;
        const TX* xrow = lx + br * K;
        const TY* ycol = ly + b * K * C + c;
        bool res;
        if (mode == BSP_LAYOUT_EXACT) {
            res = false;
            for (int64_t k = 0; k < K; ++k)
                res |= LayoutElem<TX>::nonzero(xrow[k]) && LayoutElem<TY>::nonzero(ycol[k * C]);
        } else {
            bool ax = false, ay = false;
            for (int64_t k = 0; k < K; ++k) {
                ax |= LayoutElem<TX>::nonzero(xrow[k]);
                ay |= LayoutElem<TY>::nonzero(ycol[k * C]);
            }
            res = (mode == BSP_LAYOUT_FAST) ? (ax && ay) : (ax || ay);
        }
        out[o] = res ? 1 : 0;
    }
}

// ---- pair plan ---------------------------------------------------------------
// One warp per output block; lanes stride over the inner index t.
template <bool FILL>
__global__ void __launch_bounds__(256)
plan_walk_kernel(const int64_t* __restrict__ lut_out, int64_t n_out,
                 const int64_t* __restrict__ packed_a, int64_t a_sb, int64_t a_sr, int64_t a_st,
                 const int64_t* __restrict__ packed_b, int64_t b_sb, int64_t b_st, int64_t b_sc,
                 int64_t T, int32_t* __restrict__ counts, const int32_t* __restrict__ offsets,
                 int32_t* __restrict__ pairs) {
    const int lane = threadIdx.x & 31;
    const int64_t warps_total = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t p = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); p < n_out;
         p += warps_total) {
        const int64_t b = lut_out[p * 3 + 0], r = lut_out[p * 3 + 1], c = lut_out[p * 3 + 2];
        const int64_t* pa = packed_a + b * a_sb + r * a_sr;
        const int64_t* pb = packed_b + b * b_sb + c * b_sc;
        int32_t n = 0;
        const int32_t base = FILL ? offsets[p] : 0;
        const int32_t last = FILL ? offsets[p + 1] - 1 : -1;  // position of the block's last pair
        for (int64_t t0 = 0; t0 < T; t0 += 32) {
            const int64_t t = t0 + lane;
            int64_t ia = -1, ib = -1;
            if (t < T) {
                ia = pa[t * a_st];
                ib = pb[t * b_st];
            }
            const bool hit = ia >= 0 && ib >= 0;
            const unsigned m = __ballot_sync(0xffffffffu, hit);
            if (FILL && hit) {
                const int32_t pos = base + n + __popc(m & ((1u << lane) - 1u));
                pairs[2 * (int64_t)pos + 0] = (int32_t)ia | (pos == last ? 0x40000000 : 0);
                pairs[2 * (int64_t)pos + 1] = (int32_t)ib;
            }
            n += __popc(m);
        }
        if (!FILL && lane == 0) counts[p] = n;
    }
}

__global__ void __launch_bounds__(kScanThreads)
count_reduce_kernel(const int32_t* __restrict__ counts, int64_t n, int64_t* __restrict__ chunk_sums) {
    const int64_t base = (int64_t)blockIdx.x * kScanChunk;
    int64_t s = 0;
#pragma unroll
    for (int i = 0; i < kScanItems; ++i) {
        int64_t e = base + (int64_t)i * kScanThreads + threadIdx.x;
        if (e < n) s += counts[e];
    }
    int64_t total;
    block_exclusive_scan(s, &total);
    if (threadIdx.x == 0) chunk_sums[blockIdx.x] = total;
}

__global__ void __launch_bounds__(kScanThreads)
count_apply_kernel(const int32_t* __restrict__ counts, int64_t n,
                   const int64_t* __restrict__ chunk_offsets, int64_t n_chunks,
                   int32_t* __restrict__ offsets) {
    const int64_t base = (int64_t)blockIdx.x * kScanChunk + (int64_t)threadIdx.x * kScanItems;
    int64_t v[kScanItems];
    int64_t s = 0;
#pragma unroll
    for (int i = 0; i < kScanItems; ++i) {
        int64_t e = base + i;
        v[i] = e < n ? counts[e] : 0;
        s += v[i];
    }
    int64_t total;
    int64_t run = chunk_offsets[blockIdx.x] + block_exclusive_scan(s, &total);
#pragma unroll
    for (int i = 0; i < kScanItems; ++i) {
        int64_t e = base + i;
        if (e < n) offsets[e] = (int32_t)run;
        run += v[i];
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) offsets[n] = (int32_t)chunk_offsets[n_chunks];
}

__global__ void total_only_kernel(int32_t* offsets, int64_t* total_out) {
    offsets[0] = 0;
    if (total_out) *total_out = 0;
}

__global__ void plan_schedule_kernel(const int32_t* __restrict__ offsets, int64_t n_out,
                                     int32_t block_cost, int32_t n_chunks,
                                     int32_t* __restrict__ chunk_begin) {
    const int g = blockIdx.x * blockDim.x + threadIdx.x;
    if (g > n_chunks) return;
    if (g == n_chunks) {
        chunk_begin[g] = (int32_t)n_out;
        return;
    }
    // cost of the blocks before p: offsets[p] + block_cost * p (non-decreasing in p)
    const int64_t total = (int64_t)offsets[n_out] + (int64_t)block_cost * n_out;
    const int64_t target = (total * g) / n_chunks;
    int64_t lo = 0, hi = n_out;  // smallest p with cost_before(p) >= target
    while (lo < hi) {
        int64_t mid = (lo + hi) >> 1;
        int64_t cost = (int64_t)offsets[mid] + (int64_t)block_cost * mid;
        if (cost >= target) hi = mid; else lo = mid + 1;
    }
    chunk_begin[g] = (int32_t)lo;
}

// ---- compressed transpose -----------------------------------------------------
// out[p] = x[src[p]]^T, 32x32 (or bs x bs for bs = 16) tiles through shared memory.
template <typename E>
__global__ void __launch_bounds__(256)
transpose_blocks_kernel(const E* __restrict__ x, int64_t n_x, E* __restrict__ out,
                        const int64_t* __restrict__ src_index, int bs) {
    __shared__ E tile[32][33];
    const int ts = bs < 32 ? bs : 32;
    const int tiles = bs / ts;
    const int64_t p = blockIdx.x;
    const int tr = blockIdx.y / tiles, tc = blockIdx.y % tiles;  // output tile coordinates
    const int64_t s = src_index[p];
    E* o = out + p * (int64_t)bs * bs;
    const bool have = s >= 0 && s < n_x;
    const E* xs = x + (have ? s : 0) * (int64_t)bs * bs;
    // the output tile (tr,tc) is the transpose of the source tile (tc,tr)
    for (int i = threadIdx.x; i < ts * ts; i += blockDim.x) {
        int r = i / ts, c = i % ts;
        tile[r][c] = have ? xs[(int64_t)(tc * ts + r) * bs + tr * ts + c] : E(0);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < ts * ts; i += blockDim.x) {
        int r = i / ts, c = i % ts;
        o[(int64_t)(tr * ts + r) * bs + tc * ts + c] = tile[c][r];
    }
}

}  // namespace bsp

using namespace bsp;

extern "C" size_t bsp_lut_workspace_bytes(int64_t numel) {
    if (numel < 0) numel = 0;
    return (size_t)(scan_chunks(numel) + 1) * sizeof(int64_t);
}

extern "C" int bsp_build_packed_indices(const void* layout, int layout_dtype, int64_t numel,
                                        int64_t* packed_out, int64_t* total_out, void* workspace,
                                        size_t workspace_bytes, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (numel < 0 || !workspace || (numel > 0 && (!layout || !packed_out))) return BSP_ERR_INVALID_ARG;
    if (workspace_bytes < bsp_lut_workspace_bytes(numel)) return BSP_ERR_WORKSPACE;
    int64_t* ws = (int64_t*)workspace;
    const int64_t nch = scan_chunks(numel);
    bool ok = dispatch_layout_dtype(layout_dtype, [&](auto tag) {
        using T = decltype(tag);
        if (nch > 0)
            chunk_reduce_kernel<T, kViewI64><<<(unsigned)nch, kScanThreads, 0, stream>>>((const T*)layout, numel, ws);
        chunk_scan_kernel<<<1, kScanThreads, 0, stream>>>(ws, nch, total_out);
        if (nch > 0)
            packed_apply_kernel<T><<<(unsigned)nch, kScanThreads, 0, stream>>>((const T*)layout, numel, ws, packed_out);
    });
    if (!ok) return BSP_ERR_UNSUPPORTED;
    BSP_LAUNCH_CHECK();
    return BSP_OK;
}

extern "C" int bsp_count_nonzero(const void* layout, int layout_dtype, int64_t numel,
                                 int64_t* count_out, void* workspace, size_t workspace_bytes,
                                 void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (numel < 0 || !workspace || (numel > 0 && !layout)) return BSP_ERR_INVALID_ARG;
    if (workspace_bytes < bsp_lut_workspace_bytes(numel)) return BSP_ERR_WORKSPACE;
    int64_t* ws = (int64_t*)workspace;
    const int64_t nch = scan_chunks(numel);
    bool ok = dispatch_layout_dtype(layout_dtype, [&](auto tag) {
        using T = decltype(tag);
        if (nch > 0)
            chunk_reduce_kernel<T, kViewNonzero><<<(unsigned)nch, kScanThreads, 0, stream>>>((const T*)layout, numel, ws);
        chunk_scan_kernel<<<1, kScanThreads, 0, stream>>>(ws, nch, count_out);
    });
    if (!ok) return BSP_ERR_UNSUPPORTED;
    BSP_LAUNCH_CHECK();
    return BSP_OK;
}

extern "C" int bsp_build_layout_indices(const void* layout, int layout_dtype, int64_t B, int64_t R,
                                        int64_t C, int64_t* lut_out, int64_t capacity_rows,
                                        void* workspace, size_t workspace_bytes, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (B < 0 || R < 0 || C < 0 || capacity_rows < 0 || !workspace) return BSP_ERR_INVALID_ARG;
    const int64_t numel = B * R * C;
    if (workspace_bytes < bsp_lut_workspace_bytes(numel)) return BSP_ERR_WORKSPACE;
    if (numel == 0 || capacity_rows == 0) return BSP_OK;
    if (!layout || !lut_out) return BSP_ERR_INVALID_ARG;
    const int64_t nch = scan_chunks(numel);
    bool ok = dispatch_layout_dtype(layout_dtype, [&](auto tag) {
        using T = decltype(tag);
        lut_apply_kernel<T><<<(unsigned)nch, kScanThreads, 0, stream>>>(
            (const T*)layout, numel, R, C, (const int64_t*)workspace, lut_out, capacity_rows);
    });
    if (!ok) return BSP_ERR_UNSUPPORTED;
    BSP_LAUNCH_CHECK();
    return BSP_OK;
}

extern "C" int bsp_layout_matmul(const void* lx, int lx_dtype, const void* ly, int ly_dtype,
                                 int64_t B, int64_t R, int64_t K, int64_t C, int mode,
                                 uint8_t* out, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (B < 0 || R < 0 || K < 0 || C < 0) return BSP_ERR_INVALID_ARG;
    if (mode != BSP_LAYOUT_EXACT && mode != BSP_LAYOUT_FAST && mode != BSP_LAYOUT_OUTER)
        return BSP_ERR_INVALID_ARG;
    const int64_t total = B * R * C;
    if (total == 0) return BSP_OK;
    if (!out || (K > 0 && (!lx || !ly))) return BSP_ERR_INVALID_ARG;
    const int threads = 256;
    const int64_t blocks = ceil_div(total, threads);
    const unsigned grid = (unsigned)(blocks > 148 * 64 ? 148 * 64 : blocks);
    if (lx_dtype < BSP_L_BOOL || lx_dtype > BSP_L_F64 || ly_dtype < BSP_L_BOOL ||
        ly_dtype > BSP_L_F64)
        return BSP_ERR_UNSUPPORTED;
    dispatch_layout_dtype(lx_dtype, [&](auto tx) {
        using TX = decltype(tx);
        dispatch_layout_dtype(ly_dtype, [&](auto ty) {
            using TY = decltype(ty);
            layout_matmul_kernel<TX, TY><<<grid, threads, 0, stream>>>(
                (const TX*)lx, (const TY*)ly, B, R, K, C, mode, out);
        });
    });
    BSP_LAUNCH_CHECK();
    return BSP_OK;
}

static inline unsigned plan_grid(int64_t n_out) {
    int64_t blocks = ceil_div(n_out, 8);  // 8 warps per CTA
    return (unsigned)(blocks > 148 * 32 ? 148 * 32 : (blocks < 1 ? 1 : blocks));
}

extern "C" int bsp_plan_count(const int64_t* lut_out, int64_t n_out, const int64_t* packed_a,
                              int64_t a_sb, int64_t a_sr, int64_t a_st, const int64_t* packed_b,
                              int64_t b_sb, int64_t b_st, int64_t b_sc, int64_t T,
                              int32_t* counts_out, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (n_out < 0 || T < 0) return BSP_ERR_INVALID_ARG;
    if (n_out == 0) return BSP_OK;
    if (!lut_out || !counts_out || (T > 0 && (!packed_a || !packed_b))) return BSP_ERR_INVALID_ARG;
    plan_walk_kernel<false><<<plan_grid(n_out), 256, 0, stream>>>(
        lut_out, n_out, packed_a, a_sb, a_sr, a_st, packed_b, b_sb, b_st, b_sc, T, counts_out,
        nullptr, nullptr);
    BSP_LAUNCH_CHECK();
    return BSP_OK;
}

extern "C" size_t bsp_plan_workspace_bytes(int64_t n_out) {
    if (n_out < 0) n_out = 0;
    return (size_t)(scan_chunks(n_out) + 1) * sizeof(int64_t);
}

extern "C" int bsp_plan_offsets(const int32_t* counts, int64_t n_out, int32_t* offsets_out,
                                int64_t* total_out, void* workspace, size_t workspace_bytes,
                                void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (n_out < 0 || !offsets_out || !workspace) return BSP_ERR_INVALID_ARG;
    if (workspace_bytes < bsp_plan_workspace_bytes(n_out)) return BSP_ERR_WORKSPACE;
    if (n_out == 0) {
        total_only_kernel<<<1, 1, 0, stream>>>(offsets_out, total_out);
        BSP_LAUNCH_CHECK();
        return BSP_OK;
    }
    if (!counts) return BSP_ERR_INVALID_ARG;
    int64_t* ws = (int64_t*)workspace;
    const int64_t nch = scan_chunks(n_out);
    count_reduce_kernel<<<(unsigned)nch, kScanThreads, 0, stream>>>(counts, n_out, ws);
    chunk_scan_kernel<<<1, kScanThreads, 0, stream>>>(ws, nch, total_out);
    count_apply_kernel<<<(unsigned)nch, kScanThreads, 0, stream>>>(counts, n_out, ws, nch, offsets_out);
    BSP_LAUNCH_CHECK();
    return BSP_OK;
}

extern "C" int bsp_plan_fill(const int64_t* lut_out, int64_t n_out, const int64_t* packed_a,
                             int64_t a_sb, int64_t a_sr, int64_t a_st, const int64_t* packed_b,
                             int64_t b_sb, int64_t b_st, int64_t b_sc, int64_t T,
                             const int32_t* offsets, int32_t* pairs_out, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (n_out < 0 || T < 0) return BSP_ERR_INVALID_ARG;
    if (n_out == 0 || T == 0) return BSP_OK;
    if (!lut_out || !offsets || !packed_a || !packed_b) return BSP_ERR_INVALID_ARG;
    plan_walk_kernel<true><<<plan_grid(n_out), 256, 0, stream>>>(
        lut_out, n_out, packed_a, a_sb, a_sr, a_st, packed_b, b_sb, b_st, b_sc, T, nullptr,
        offsets, pairs_out);
    BSP_LAUNCH_CHECK();
    return BSP_OK;
}

extern "C" int bsp_plan_schedule(const int32_t* offsets, int64_t n_out, int32_t block_cost,
                                 int32_t n_chunks, int32_t* chunk_begin_out, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (n_out < 0 || n_chunks < 1 || block_cost < 0 || !offsets || !chunk_begin_out)
        return BSP_ERR_INVALID_ARG;
    const int threads = 128;
    plan_schedule_kernel<<<(n_chunks + 1 + threads - 1) / threads, threads, 0, stream>>>(
        offsets, n_out, block_cost, n_chunks, chunk_begin_out);
    BSP_LAUNCH_CHECK();
    return BSP_OK;
}

extern "C" int bsp_transpose_blocks(const void* x, int64_t n_x, void* out, int64_t n_out,
                                    const int64_t* src_index, int bs, int elem_bytes,
                                    void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (n_x < 0 || n_out < 0 || bs < 16 || (bs & (bs - 1))) return BSP_ERR_INVALID_ARG;
    if (n_out == 0) return BSP_OK;
    if (!out || !src_index || (n_x > 0 && !x)) return BSP_ERR_INVALID_ARG;
    if (n_out > INT_MAX) return BSP_ERR_UNSUPPORTED;
    const int ts = bs < 32 ? bs : 32;
    dim3 grid((unsigned)n_out, (unsigned)((bs / ts) * (bs / ts)));
    switch (elem_bytes) {
        case 1: transpose_blocks_kernel<uint8_t><<<grid, 256, 0, stream>>>((const uint8_t*)x, n_x, (uint8_t*)out, src_index, bs); break;
        case 2: transpose_blocks_kernel<uint16_t><<<grid, 256, 0, stream>>>((const uint16_t*)x, n_x, (uint16_t*)out, src_index, bs); break;
        case 4: transpose_blocks_kernel<uint32_t><<<grid, 256, 0, stream>>>((const uint32_t*)x, n_x, (uint32_t*)out, src_index, bs); break;
        case 8: transpose_blocks_kernel<uint64_t><<<grid, 256, 0, stream>>>((const uint64_t*)x, n_x, (uint64_t*)out, src_index, bs); break;
        default: return BSP_ERR_UNSUPPORTED;
    }
    BSP_LAUNCH_CHECK();
    return BSP_OK;
}

// ---- reverse LUT without caller-provided scratch --------------------------------------
// The chunk sums of the scan live in a fixed array inside the library image instead of a
// caller-allocated workspace.  Every GPU that loads the library carries the array
// (16 KiB + 8 B) until the process exits.
static constexpr int64_t kStaticMaxNumel = (int64_t)1 << 22;  // 4 194 304 layout entries
static __device__ __align__(256) int64_t g_static_scan_scratch[kStaticMaxNumel / bsp::kScanChunk + 1];

// Device address of the array on the current device.  The symbol's name is only a host-side
// handle, so the address is looked up once per device (with that device current) and cached.
static int static_scan_scratch(int64_t** out) {
    static std::mutex mu;
    static int64_t* cached[64] = {nullptr};
    int dev = -1;
    BSP_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return BSP_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(mu);
    if (!cached[dev]) {
        void* p = nullptr;
        BSP_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scan_scratch));
        if (!p) return BSP_ERR_CUDA;
        cached[dev] = (int64_t*)p;
    }
    *out = cached[dev];
    return BSP_OK;
}

extern "C" int64_t bsp_static_scratch_max_numel(void) { return kStaticMaxNumel; }

extern "C" int bsp_build_packed_indices_static(const void* layout, int layout_dtype, int64_t numel,
                                               int64_t* packed_out, int64_t* total_out, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (numel < 0 || (numel > 0 && (!layout || !packed_out))) return BSP_ERR_INVALID_ARG;
    if (numel > kStaticMaxNumel) return BSP_ERR_TOO_LARGE;
    int64_t* ws = nullptr;
    int st = static_scan_scratch(&ws);
    if (st != BSP_OK) return st;
    // Nothing in the array has to start at zero: phase 1 writes chunk sums [0, nch), phase 2
    // rewrites them in place and writes entry nch, phase 3 only reads what those two wrote.
    const int64_t nch = scan_chunks(numel);
    bool ok = dispatch_layout_dtype(layout_dtype, [&](auto tag) {
        using T = decltype(tag);
        if (nch > 0)
            chunk_reduce_kernel<T, kViewI64><<<(unsigned)nch, kScanThreads, 0, stream>>>((const T*)layout, numel, ws);
        chunk_scan_kernel<<<1, kScanThreads, 0, stream>>>(ws, nch, total_out);
        if (nch > 0)
            packed_apply_kernel<T><<<(unsigned)nch, kScanThreads, 0, stream>>>((const T*)layout, numel, ws, packed_out);
    });
    if (!ok) return BSP_ERR_UNSUPPORTED;
    BSP_LAUNCH_CHECK();
    return BSP_OK;
}
