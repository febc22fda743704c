"""The allocation-free reverse-LUT entry point against the regular one, through the C ABI.

Some hosts of this library cannot allocate device memory at call time: they carve up all of HBM
once at start-up from their own arena, or cannot tolerate the device-wide synchronisation a
cudaMalloc brings.  For them ``bsp_build_packed_indices_static`` keeps the scan's scratch in a
fixed array inside the library.  The test (collected last, so a failure here cannot hide
another test) calls it twice in a row on different layouts — the array keeps the first call's
contents — and expects bit-identical results to ``bsp_build_packed_indices``, which takes a
caller-allocated workspace.  All buffers the test passes are the caller's (torch) allocations.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _regular(lib, cabi, layout):
    numel = layout.numel()
    ws_bytes = lib.bsp_lut_workspace_bytes(numel)
    ws = torch.empty(ws_bytes // 8, dtype=torch.int64, device=layout.device)
    packed = torch.empty(numel, dtype=torch.int64, device=layout.device)
    total = torch.empty(1, dtype=torch.int64, device=layout.device)
    cabi.check(lib.bsp_build_packed_indices(layout.data_ptr(), cabi.LAYOUT_DTYPE_CODES[layout.dtype], numel,
                                            packed.data_ptr(), total.data_ptr(), ws.data_ptr(), ws_bytes,
                                            cabi.stream_handle(layout.device)), "bsp_build_packed_indices")
    return packed, total


def _static(lib, cabi, layout):
    numel = layout.numel()
    packed = torch.full((numel,), -7, dtype=torch.int64, device=layout.device)
    total = torch.full((1,), -7, dtype=torch.int64, device=layout.device)
    cabi.check(lib.bsp_build_packed_indices_static(layout.data_ptr(), cabi.LAYOUT_DTYPE_CODES[layout.dtype], numel,
                                                   packed.data_ptr(), total.data_ptr(),
                                                   cabi.stream_handle(layout.device)),
               "bsp_build_packed_indices_static")
    return packed, total


def test_static_scratch_entry_point_matches_regular_one_twice_in_a_row():
    from blksprs_b200 import _cabi as cabi
    lib = cabi.lib()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    g = torch.Generator().manual_seed(123)
    # first a large layout (many scan chunks), then a smaller one of another dtype: the second call
    # finds the first call's chunk sums in the shared array and must not be affected by them
    first = (torch.rand((16, 128, 96), generator=g) < 0.3).to(dev)
    second = (torch.rand((3, 37, 41), generator=g) < 0.6).to(torch.float32).to(dev)
    for layout in (first, second):
        want_packed, want_total = _regular(lib, cabi, layout)
        got_packed, got_total = _static(lib, cabi, layout)
        torch.cuda.synchronize()
        assert torch.equal(got_packed, want_packed)
        assert torch.equal(got_total, want_total)
        assert int(got_total) == int((layout != 0).sum())


@pytest.mark.parametrize("numel", ["limit", 2048 * 37 + 1, 2048, 2049])
def test_static_scratch_entry_point_at_its_size_limit_and_at_partial_chunks(numel):
    """The largest accepted layout fills every slot of the fixed scratch array (one chunk sum per 2048
    entries plus the total); sizes one past a chunk boundary leave a partial last chunk."""
    from blksprs_b200 import _cabi as cabi
    lib = cabi.lib()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    if numel == "limit":
        numel = lib.bsp_static_scratch_max_numel()
    g = torch.Generator(device=dev).manual_seed(7)
    layout = torch.rand((numel,), generator=g, device=dev) < 0.4
    layout[-1] = True   # the last entry's rank depends on every chunk sum before it
    want_packed, want_total = _regular(lib, cabi, layout)
    got_packed, got_total = _static(lib, cabi, layout)
    torch.cuda.synchronize()
    assert torch.equal(got_packed, want_packed)
    assert torch.equal(got_total, want_total)
    assert int(got_packed[-1]) == int(got_total) - 1


def test_static_scratch_entry_point_rejects_oversized_layouts():
    from blksprs_b200 import _cabi as cabi
    lib = cabi.lib()
    limit = lib.bsp_static_scratch_max_numel()
    assert limit == 1 << 22
    dev = torch.device("cuda:0")
    dummy = torch.zeros(8, dtype=torch.bool, device=dev)
    out = torch.zeros(8, dtype=torch.int64, device=dev)
    status = lib.bsp_build_packed_indices_static(dummy.data_ptr(), 0, limit + 1, out.data_ptr(), None,
                                                 cabi.stream_handle(dev))
    assert status == cabi.ERR_TOO_LARGE
    assert b"scratch" in lib.bsp_status_string(status)
    # the limit itself and an empty layout are accepted argument-wise
    assert lib.bsp_build_packed_indices_static(None, 0, 0, None, None, cabi.stream_handle(dev)) == cabi.OK
