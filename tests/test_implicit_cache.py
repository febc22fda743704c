"""The library-owned layout caches behind calls that pass ``layout_cache=None`` (host logic, CPU tensors):
same reuse rule as a caller-owned cache (blksprs/utils/tools.py:60-156), least-recently-used eviction, never
for inference tensors, and a switch that restores the reference's rebuild-on-every-call behaviour."""
import torch

from blksprs_b200.utils import tools


def _layouts():
    return tuple(torch.ones((2, 3, 4), dtype=torch.bool) for _ in range(3))


def test_same_layout_objects_share_one_cache_until_one_is_mutated():
    tools.clear_implicit_layout_caches()
    lx, ly, lo = _layouts()
    first = tools.implicit_layout_cache("matmul", lx, ly, lo)
    assert first == {} and tools.implicit_layout_cache("matmul", lx, ly, lo) is first   # empty until the op fills it
    assert tools.implicit_layout_cache("transpose", lx) is not first            # keyed by operation too
    assert tools.implicit_layout_cache("matmul", lx, ly, lo.clone()) is not first  # and by object identity
    lo[0, 0, 0] = False   # in-place change: version bump
    assert tools.implicit_layout_cache("matmul", lx, ly, lo) is not first


def test_prepare_uses_it_only_without_a_caller_cache_and_applies_the_reuse_rule():
    tools.clear_implicit_layout_caches()
    lx, ly, lo = _layouts()
    cache = tools.prepare_layout_cache(None, "matmul", lx, ly, lo)
    cache["packed_indices_x"] = torch.zeros(3)
    tools.finalize_layout_cache(cache)
    again = tools.prepare_layout_cache(None, "matmul", lx, ly, lo)
    assert again is cache and "packed_indices_x" in again
    mine = {}
    assert tools.prepare_layout_cache(mine, "matmul", lx, ly, lo) is mine and "packed_indices_x" not in mine
    cache["packed_indices_x"].add_(1)   # a stored entry mutated behind the library's back: rebuilt from empty
    rebuilt = tools.prepare_layout_cache(None, "matmul", lx, ly, lo)
    assert rebuilt is cache and "packed_indices_x" not in rebuilt


def test_eviction_inference_tensors_and_switch():
    tools.clear_implicit_layout_caches()
    sets = [_layouts() for _ in range(tools.IMPLICIT_CACHE_ENTRIES + 1)]
    caches = [tools.implicit_layout_cache("matmul", *s) for s in sets]
    assert tools.implicit_layout_cache("matmul", *sets[-1]) is caches[-1]
    assert tools.implicit_layout_cache("matmul", *sets[0]) is not caches[0]      # the oldest entry was evicted
    with torch.inference_mode():
        inf = torch.ones((1, 2, 2), dtype=torch.bool)
    assert tools.implicit_layout_cache("softmax", inf) is None
    tools.set_implicit_layout_caches(False)
    try:
        assert tools.implicit_layout_cache("matmul", *sets[-1]) is None
        fresh = tools.prepare_layout_cache(None, "matmul", *sets[-1])   # a new dict with bookkeeping only
        assert fresh is not caches[-1] and all(k.startswith("_blksprs") for k in fresh)
    finally:
        tools.set_implicit_layout_caches(True)
