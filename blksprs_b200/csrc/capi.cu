// C-ABI entry points that are not tied to one kernel file: version, status
// text, error text, and the matmul dispatcher.
#include <stdio.h>
#include <string.h>

#include "common.cuh"
#include <cstdint>

namespace bsp {

static thread_local char g_cuda_error[256] = "";

void set_cuda_error(cudaError_t err, const char* what) {
    snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s (%s)", what, cudaGetErrorName(err),
             cudaGetErrorString(err));
    cudaGetLastError();  // clear the sticky-free error so later launches report their own
}

}  // namespace bsp

using namespace bsp;

extern "C" int bsp_version(void) { return 100; }  // 0.1.0

extern "C" const char* bsp_status_string(int status) {
    switch (status) {
        case BSP_OK: return "ok";
        case BSP_ERR_INVALID_ARG: return "invalid argument";
        case BSP_ERR_UNSUPPORTED: return "unsupported dtype, block size or index range";
        case BSP_ERR_WORKSPACE: return "workspace too small";
        case BSP_ERR_CUDA: return "CUDA call failed";
        case BSP_ERR_DEVICE_RANGE: return "device: block index out of range";
        case BSP_ERR_DEVICE_TIMEOUT: return "device: bounded wait ran out";
        case BSP_ERR_TOO_LARGE: return "size exceeds the limit of the built-in scratch array";
        default: return "unknown status";
    }
}

extern "C" const char* bsp_last_cuda_error(void) { return g_cuda_error; }

extern "C" int bsp_matmul_mma(const void* a, int64_t n_a, const void* b, int64_t n_b, void* out,
                              int64_t n_out, const int32_t* offsets, const int32_t* pairs, int bs, int dtype,
                              int op, int32_t* status_word, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (n_a < 0 || n_b < 0 || n_out < 0) return BSP_ERR_INVALID_ARG;
    if (bs < 16 || (bs & (bs - 1))) return BSP_ERR_INVALID_ARG;
    if (op != BSP_OP_NN && op != BSP_OP_NT && op != BSP_OP_TN) return BSP_ERR_INVALID_ARG;
    if (dtype != BSP_F16 && dtype != BSP_BF16 && dtype != BSP_F32) return BSP_ERR_UNSUPPORTED;
    if (n_out == 0) return BSP_OK;  // an empty grid is legal (empty output layout)
    if (!out || !offsets) return BSP_ERR_INVALID_ARG;
    if ((n_a > 0 && !a) || (n_b > 0 && !b)) return BSP_ERR_INVALID_ARG;
    // the kernels move 16-byte vectors
    if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(out)) & 15)
        return BSP_ERR_INVALID_ARG;
    return launch_matmul_mma(a, n_a, b, n_b, out, n_out, offsets, pairs, bs, dtype, op, status_word, stream);
}
