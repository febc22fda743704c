"""ctypes binding of ``libblksprs_b200.so`` (the C ABI declared in ``include/blksprs_b200.h``).

The library is the only compute path of this package: there is no Python or
CPU fallback.  If it has not been built, every call raises ``RuntimeError``.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_int32, c_int64, c_size_t, c_void_p, c_char_p
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libblksprs_b200.so"

# status codes (include/blksprs_b200.h)
OK, ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_WORKSPACE, ERR_CUDA, ERR_DEVICE_RANGE, ERR_DEVICE_TIMEOUT, ERR_TOO_LARGE = range(8)
# matmul ops / kernel selectors / layout modes
OP_NN, OP_NT, OP_TN = 0, 1, 2
LAYOUT_EXACT, LAYOUT_FAST, LAYOUT_OUTER = 0, 1, 2

LAYOUT_DTYPE_CODES = {
    torch.bool: 0, torch.uint8: 0, torch.int8: 1, torch.int16: 2, torch.int32: 3, torch.int64: 4,
    torch.float16: 5, torch.bfloat16: 6, torch.float32: 7, torch.float64: 8,
}
DATA_DTYPE_CODES = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}

# name -> (restype, argtypes); must list every symbol the header declares
SIGNATURES = {
    "bsp_version": (c_int, []),
    "bsp_status_string": (c_char_p, [c_int]),
    "bsp_last_cuda_error": (c_char_p, []),
    "bsp_lut_workspace_bytes": (c_size_t, [c_int64]),
    "bsp_build_packed_indices": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "bsp_build_packed_indices_static": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p]),
    "bsp_static_scratch_max_numel": (c_int64, []),
    "bsp_count_nonzero": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_size_t, c_void_p]),
    "bsp_build_layout_indices": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_int64,
                                         c_void_p, c_size_t, c_void_p]),
    "bsp_layout_matmul": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int,
                                  c_void_p, c_void_p]),
    "bsp_plan_count": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_int64,
                               c_int64, c_int64, c_void_p, c_void_p]),
    "bsp_plan_workspace_bytes": (c_size_t, [c_int64]),
    "bsp_plan_offsets": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "bsp_plan_fill": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_int64,
                              c_int64, c_int64, c_void_p, c_void_p, c_void_p]),
    "bsp_plan_schedule": (c_int, [c_void_p, c_int64, c_int32, c_int32, c_void_p, c_void_p]),
    "bsp_matmul_mma": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p,
                               c_int, c_int, c_int, c_void_p, c_void_p]),
    "bsp_umma_max_width": (c_int, [c_int, c_int]),
    "bsp_umma_num_ctas": (c_int, [c_int, c_int, c_int]),
    "bsp_panel_count": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64,
                                c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "bsp_panel_fill": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64,
                               c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p]),
    "bsp_matmul_umma": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p,
                                c_void_p, c_int64,
                                c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_void_p, c_int, c_int, c_int,
                                c_int, c_void_p, c_void_p]),
    "bsp_matmul_umma_softmax": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, ctypes.c_float,
                                        c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32,
                                        c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "bsp_softmax_normalize": (c_int, [c_void_p, c_int, c_void_p, c_int64, c_void_p, c_int64, c_int, c_void_p, c_int,
                                      c_void_p]),
    "bsp_to_sparse": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "bsp_to_dense": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int64, c_int, c_int, ctypes.c_uint64,
                             c_void_p, c_void_p]),
    "bsp_softmax_fwd": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "bsp_softmax_fwd_scaled": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_int64, c_int64, c_int64, c_int, ctypes.c_float,
                                       c_void_p, c_int, c_void_p]),
    "bsp_softmax_bwd_scaled": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int64, c_void_p, c_int64, c_int64, c_int64, c_int,
                                       ctypes.c_float, c_void_p, c_int, c_void_p]),
    "bsp_softmax_bwd": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p,
                                c_void_p]),
    "bsp_bias_add": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_void_p, c_int64, c_int, c_void_p, c_void_p]),
    "bsp_bias_grad": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_int64, c_void_p]),
    "bsp_sum_chunks": (c_int, [c_void_p, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "bsp_selftest_wait_limit": (c_int, [ctypes.c_uint32, c_void_p, c_void_p]),
    "bsp_transpose_blocks": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int, c_int, c_void_p]),
}

_lib = None


def lib() -> ctypes.CDLL:
    """Returns the loaded library, loading it on first use."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"blksprs_b200: native library {LIB_PATH} is missing; there is no fallback path. "
                "Build it with `python -m blksprs_b200.build`.")
        handle = ctypes.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


class NativeError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, status: int, where: str):
        self.status = status
        text = lib().bsp_status_string(status).decode()
        detail = lib().bsp_last_cuda_error().decode() if status == ERR_CUDA else ""
        super().__init__(f"blksprs_b200: {where} failed: {text}" + (f" [{detail}]" if detail else ""))


def check(status: int, where: str) -> None:
    if status != OK:
        raise NativeError(status, where)


def ptr(t: torch.Tensor | None) -> int | None:
    """Device pointer of a tensor (``None`` -> NULL)."""
    if t is None:
        return None
    return t.data_ptr()


def aligned(tensor: torch.Tensor) -> torch.Tensor:
    """``tensor`` itself if its data start on a 16-byte boundary (the kernels move 16-byte vectors), else a
    copy that does: a contiguous view into the middle of a larger buffer may start anywhere."""
    return tensor if tensor.data_ptr() % 16 == 0 else tensor.clone(memory_format=torch.contiguous_format)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_handle(device: torch.device) -> int:
    """The ``cudaStream_t`` of the calling thread's current stream on ``device``."""
    if _raw_stream is not None and device.index is not None:
        return _raw_stream(device.index)
    return torch.cuda.current_stream(device).cuda_stream


class _NoGuard:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_GUARD = _NoGuard()


def device_guard(device: torch.device):
    """Context that makes ``device`` the current CUDA device; free when it already is."""
    if device.index is not None and torch.cuda.current_device() == device.index:
        return _NO_GUARD
    return torch.cuda.device(device)
