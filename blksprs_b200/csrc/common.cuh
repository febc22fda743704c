// Shared host/device helpers for the blksprs_b200 C-ABI library.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/blksprs_b200.h"

namespace bsp {

// Records the text of a failed CUDA call for bsp_last_cuda_error().
void set_cuda_error(cudaError_t err, const char* what);

#define BSP_CUDA_TRY(expr)                                  \
    do {                                                    \
        cudaError_t _e = (expr);                            \
        if (_e != cudaSuccess) {                            \
            ::bsp::set_cuda_error(_e, #expr);               \
            return BSP_ERR_CUDA;                            \
        }                                                   \
    } while (0)

#define BSP_LAUNCH_CHECK()                                  \
    do {                                                    \
        cudaError_t _e = cudaGetLastError();                \
        if (_e != cudaSuccess) {                            \
            ::bsp::set_cuda_error(_e, "kernel launch");     \
            return BSP_ERR_CUDA;                            \
        }                                                   \
    } while (0)

// ---- layout element access ------------------------------------------------
// Two views of a layout entry are needed to reproduce the reference bit for
// bit: `to(int64)` (C-style truncation, used by build_packed_indices) and
// `!= 0` (used by torch.nonzero / torch.any).
template <typename T>
struct LayoutElem {
    __device__ static inline int64_t as_i64(T v) { return (int64_t)v; }
    __device__ static inline bool nonzero(T v) { return v != (T)0; }
};
template <>
struct LayoutElem<__half> {
    __device__ static inline int64_t as_i64(__half v) { return (int64_t)__half2float(v); }
    __device__ static inline bool nonzero(__half v) { return __half2float(v) != 0.0f; }
};
template <>
struct LayoutElem<__nv_bfloat16> {
    __device__ static inline int64_t as_i64(__nv_bfloat16 v) { return (int64_t)__bfloat162float(v); }
    __device__ static inline bool nonzero(__nv_bfloat16 v) { return __bfloat162float(v) != 0.0f; }
};

// Calls f(T{}) with T the C type behind a BSP_L_* code; returns false for an
// unknown code.
template <typename F>
inline bool dispatch_layout_dtype(int code, F&& f) {
    switch (code) {
        case BSP_L_BOOL: f(uint8_t{}); return true;
        case BSP_L_I8: f(int8_t{}); return true;
        case BSP_L_I16: f(int16_t{}); return true;
        case BSP_L_I32: f(int32_t{}); return true;
        case BSP_L_I64: f(int64_t{}); return true;
        case BSP_L_F16: f(__half{}); return true;
        case BSP_L_BF16: f(__nv_bfloat16{}); return true;
        case BSP_L_F32: f(float{}); return true;
        case BSP_L_F64: f(double{}); return true;
        default: return false;
    }
}

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Implemented in matmul_mma.cu / matmul_umma.cu.
int launch_matmul_mma(const void* a, int64_t n_a, const void* b, int64_t n_b, void* out,
                      int64_t n_out, const int32_t* offsets, const int32_t* pairs, int bs,
                      int dtype, int op, int32_t* status_word, cudaStream_t stream);
bool umma_applicable(int dtype, int bs);

}  // namespace bsp
