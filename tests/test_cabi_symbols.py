"""The C-ABI library loads without a GPU and exports every symbol include/blksprs_b200.h declares."""
import ctypes
import os
import re

import pytest

from blksprs_b200 import _cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "blksprs_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bsp_\w+)\s*\(", text)))


def test_header_declares_entry_points():
    names = declared_symbols()
    for must in ("bsp_build_packed_indices", "bsp_build_layout_indices", "bsp_layout_matmul", "bsp_plan_fill",
                 "bsp_matmul_mma", "bsp_matmul_umma", "bsp_panel_fill", "bsp_transpose_blocks"):
        assert must in names


def test_library_exports_every_declared_symbol():
    if not _cabi.LIB_PATH.exists():
        pytest.fail(f"{_cabi.LIB_PATH} not built (run `python -m blksprs_b200.build`)")
    handle = ctypes.CDLL(str(_cabi.LIB_PATH))
    for name in declared_symbols():
        assert hasattr(handle, name), name


def test_binding_table_matches_header():
    assert sorted(_cabi.SIGNATURES) == declared_symbols()


def test_no_compute_calls_needed_for_status_text():
    lib = _cabi.lib()
    assert lib.bsp_version() >= 100
    assert lib.bsp_status_string(0) == b"ok"
    assert b"wait" in lib.bsp_status_string(_cabi.ERR_DEVICE_TIMEOUT)
    assert lib.bsp_lut_workspace_bytes(0) == 8
    assert lib.bsp_lut_workspace_bytes(2049) == 24


def test_argument_errors_are_reported_without_a_device():
    lib = _cabi.lib()
    # invalid enum / sizes are rejected before any CUDA call
    assert lib.bsp_matmul_mma(None, -1, None, 0, None, 0, None, None, 64, 1, 0, None, None) == _cabi.ERR_INVALID_ARG
    assert lib.bsp_matmul_mma(None, 0, None, 0, None, 0, None, None, 48, 1, 0, None, None) == _cabi.ERR_INVALID_ARG
    assert lib.bsp_matmul_mma(None, 0, None, 0, None, 0, None, None, 64, 7, 0, None, None) == _cabi.ERR_UNSUPPORTED
    assert lib.bsp_matmul_mma(None, 0, None, 0, None, 0, None, None, 64, 1, 0, None, None) == _cabi.OK
    assert lib.bsp_matmul_umma(None, 1, None, 1, None, 0, None, None, None, 0, None, None, None, None, None, 0, None,
                               2, 32, 1, 0, None, None) == _cabi.ERR_UNSUPPORTED
    assert lib.bsp_bias_add(None, None, 0, 24, None, 0, 1, None, None) == _cabi.ERR_INVALID_ARG
    assert lib.bsp_bias_add(None, None, 0, 32, None, 0, 1, None, None) == _cabi.OK
    assert lib.bsp_bias_grad(None, None, -1, 32, 1, None, 0, None) == _cabi.ERR_INVALID_ARG
    assert lib.bsp_sum_chunks(None, 0, 0, 1, None, None) == _cabi.ERR_INVALID_ARG
    assert lib.bsp_sum_chunks(None, 2, 0, 1, None, None) == _cabi.OK
    assert lib.bsp_umma_max_width(2, 64) == 2 and lib.bsp_umma_max_width(1, 32) == 0 and lib.bsp_umma_max_width(9, 64) == 0
    assert lib.bsp_layout_matmul(None, 0, None, 0, 1, 1, 1, 1, 9, None, None) == _cabi.ERR_INVALID_ARG
