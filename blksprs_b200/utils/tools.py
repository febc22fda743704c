"""LUT construction, layout-cache bookkeeping and small tensor helpers.

The two look-up tables are built by the CUDA library (no torch ops):
``build_layout_indices`` (LUT, blksprs/utils/tools.py:33-35) and
``build_packed_indices`` (reverse LUT, blksprs/utils/tools.py:38-57); results
are bit-identical to the reference's ``torch.nonzero`` / ``cumsum`` forms.
The cache protocol follows blksprs/utils/tools.py:60-156.
"""
from __future__ import annotations

import functools
import threading
from collections import OrderedDict
from typing import Any

import torch
from torch import Tensor, Size

from .. import _cabi
from .validation import _known_layout_facts

INT32_INDEX_MAX = 2_147_483_647

LayoutCache = dict[str, Any]

_KEY, _REFS, _STATE = "_blksprs_cache_key", "_blksprs_cache_refs", "_blksprs_cache_state"
_BOOKKEEPING = frozenset((_KEY, _REFS, _STATE))


def plain_dispatch(fn):
    """Runs ``fn`` with the Python-level ``__torch_function__`` dispatch of tensor subclasses switched
    off.  Compressed tensors arrive as ``BlksprsTensor`` (a subclass that changes nothing but ``repr``);
    with the dispatch on, every ``size()``, ``data_ptr()`` or ``is_contiguous()`` an op asks of them
    costs a few microseconds of handler code, several times the op's own host work."""
    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        with torch._C.DisableTorchFunctionSubclass():
            return fn(*args, **kwargs)
    return wrapper


def as_base_tensor(value: Tensor) -> Tensor:
    """``value`` as an exact ``torch.Tensor`` (subclasses stripped, storage shared)."""
    return value if type(value) is Tensor else Tensor(value)


def _require_cuda_layout(sparsity_layout: Tensor) -> Tensor:
    if sparsity_layout.device.type != "cuda":
        raise RuntimeError("blksprs_b200 builds LUTs on the GPU only; layout is on " + str(sparsity_layout.device))
    if sparsity_layout.dtype not in _cabi.LAYOUT_DTYPE_CODES:
        raise ValueError(f"Unsupported sparsity layout dtype {sparsity_layout.dtype}")
    return sparsity_layout.contiguous()


def _layout_dims(sparsity_layout: Tensor) -> tuple[int, int, int]:
    """(B, R, C) with leading dimensions folded so that any rank >= 1 works."""
    if sparsity_layout.dim() == 3:
        return tuple(sparsity_layout.shape)  # type: ignore[return-value]
    if sparsity_layout.dim() == 0:
        return 1, 1, 1
    shape = list(sparsity_layout.shape)
    while len(shape) < 3:
        shape.insert(0, 1)
    return shape[0], shape[1], shape[2]


def count_active_blocks(sparsity_layout: Tensor) -> int:
    """Number of non-zero layout entries (one device->host read per layout object and state: the count is
    remembered with the other facts validation keeps about a layout)."""
    facts = _known_layout_facts(sparsity_layout)
    known = facts.get("n_nonzero")
    if known is not None:
        return known
    layout = _require_cuda_layout(sparsity_layout)
    numel = layout.numel()
    lib = _cabi.lib()
    with torch.cuda.device(layout.device):
        ws_bytes = lib.bsp_lut_workspace_bytes(numel)
        ws = torch.empty(ws_bytes // 8, dtype=torch.int64, device=layout.device)
        count = torch.empty(1, dtype=torch.int64, device=layout.device)
        _cabi.check(lib.bsp_count_nonzero(_cabi.ptr(layout), _cabi.LAYOUT_DTYPE_CODES[layout.dtype], numel,
                                          _cabi.ptr(count), _cabi.ptr(ws), ws_bytes,
                                          _cabi.stream_handle(layout.device)), "bsp_count_nonzero")
        facts["n_nonzero"] = int(count.item())
        return facts["n_nonzero"]


def build_layout_indices(sparsity_layout: Tensor, n_active: int | None = None) -> Tensor:
    """LUT: int64 ``(n, 3)`` rows ``(batch, row, col)`` of the active blocks, row-major order.

    Equals ``torch.nonzero(sparsity_layout).contiguous()`` for 3-D layouts.
    """
    layout = _require_cuda_layout(sparsity_layout)
    if layout.dim() != 3:
        raise ValueError("Sparsity layout must have exactly 3 dimensions")
    B, R, C = layout.shape
    numel = layout.numel()
    lib = _cabi.lib()
    code = _cabi.LAYOUT_DTYPE_CODES[layout.dtype]
    with torch.cuda.device(layout.device):
        stream = _cabi.stream_handle(layout.device)
        ws_bytes = lib.bsp_lut_workspace_bytes(numel)
        ws = torch.empty(ws_bytes // 8, dtype=torch.int64, device=layout.device)
        count = torch.empty(1, dtype=torch.int64, device=layout.device)
        _cabi.check(lib.bsp_count_nonzero(_cabi.ptr(layout), code, numel, _cabi.ptr(count), _cabi.ptr(ws),
                                          ws_bytes, stream), "bsp_count_nonzero")
        if n_active is None:
            # one count serves the read and the build; the figure is remembered with the layout's other facts
            facts = _known_layout_facts(sparsity_layout)
            n_active = facts.get("n_nonzero")
            if n_active is None:
                n_active = facts["n_nonzero"] = int(count.item())
        lut = torch.empty((n_active, 3), dtype=torch.int64, device=layout.device)
        _cabi.check(lib.bsp_build_layout_indices(_cabi.ptr(layout), code, B, R, C, _cabi.ptr(lut), n_active,
                                                 _cabi.ptr(ws), ws_bytes, stream), "bsp_build_layout_indices")
    return lut


def build_packed_indices(sparsity_layout: Tensor) -> Tensor:
    """Reverse LUT: flat int64 tensor, rank of each active block among the active ones, ``-1`` elsewhere."""
    layout = _require_cuda_layout(sparsity_layout)
    numel = layout.numel()
    lib = _cabi.lib()
    with torch.cuda.device(layout.device):
        ws_bytes = lib.bsp_lut_workspace_bytes(numel)
        ws = torch.empty(ws_bytes // 8, dtype=torch.int64, device=layout.device)
        packed = torch.empty(numel, dtype=torch.int64, device=layout.device)
        _cabi.check(lib.bsp_build_packed_indices(_cabi.ptr(layout), _cabi.LAYOUT_DTYPE_CODES[layout.dtype], numel,
                                                 _cabi.ptr(packed), None, _cabi.ptr(ws), ws_bytes,
                                                 _cabi.stream_handle(layout.device)), "bsp_build_packed_indices")
    return packed


# ---- layout cache ------------------------------------------------------------

def _tensor_identity(value: Tensor, inference_token: object):
    version = inference_token if torch.is_inference(value) else int(value._version)
    return ("tensor", id(value), version, tuple(value.shape), tuple(value.stride()), value.dtype, value.device,
            value.requires_grad)


def _snapshot(value: object):
    """State of a cached value; changes whenever the caller mutates or replaces it."""
    if isinstance(value, Tensor):
        # a fresh token per look makes inference tensors (no version counter) never match
        return _tensor_identity(value, object())
    if isinstance(value, dict):
        return tuple((k, _snapshot(v)) for k, v in sorted(value.items()) if k not in _BOOKKEEPING)
    if isinstance(value, (tuple, list, Size)):
        return tuple(_snapshot(v) for v in value)
    return value


def _cache_contents_state(layout_cache: LayoutCache) -> tuple:
    return tuple((k, _snapshot(v)) for k, v in sorted(layout_cache.items()) if k not in _BOOKKEEPING)


def _cache_key(operation: str, values, held: list | None = None):
    token = object()

    def key_of(value: object):
        if isinstance(value, Tensor):
            if held is not None:
                held.append(value)
            return _tensor_identity(value, token)
        if isinstance(value, (tuple, list, Size)):
            return tuple(key_of(v) for v in value)
        if isinstance(value, dict):
            return tuple(sorted((k, key_of(v)) for k, v in value.items()))
        return value

    return operation, tuple(key_of(v) for v in values)


def layout_cache_is_current(layout_cache: LayoutCache | None, operation: str, *values: object) -> bool:
    """True if ``layout_cache`` was built by ``operation`` for exactly these inputs and nothing stored in
    it was replaced or mutated since ``finalize_layout_cache`` (the reuse rule of ``prepare_layout_cache``)."""
    if not layout_cache:
        return False
    recorded = layout_cache.get(_STATE)
    return (recorded is not None and layout_cache.get(_KEY) == _cache_key(operation, values)
            and _cache_contents_state(layout_cache) == recorded)


# Calls that pass no ``layout_cache`` (the reference's default, under which it rebuilds all metadata on
# every call) get one from a small library-owned LRU keyed like a caller-owned cache: operation name plus
# identity / version / shape / stride / dtype / device / requires_grad of every layout.  An entry holds
# references to its layouts (so their ids cannot be recycled while it lives) and is subject to the same
# reuse rule as any cache: an in-place change of a layout bumps its version and misses.  Results are the
# same as without it; only the rebuild (LUT kernels, plan kernels and their device reads) is saved.
IMPLICIT_CACHE_ENTRIES = 4
_implicit_caches: "OrderedDict[tuple, LayoutCache]" = OrderedDict()
_implicit_lock = threading.Lock()
_implicit_enabled = True


def implicit_layout_cache(operation: str, *values: object) -> LayoutCache | None:
    """The library-owned cache for a call without ``layout_cache``; None when disabled or when a layout
    is an inference tensor (no version counter: never reusable)."""
    if not _implicit_enabled:
        return None
    for value in values:
        if isinstance(value, Tensor) and torch.is_inference(value):
            return None
    key = _cache_key(operation, values)
    with _implicit_lock:
        cache = _implicit_caches.get(key)
        if cache is None:
            cache = {}
            _implicit_caches[key] = cache
            while len(_implicit_caches) > IMPLICIT_CACHE_ENTRIES:
                _implicit_caches.popitem(last=False)
        else:
            _implicit_caches.move_to_end(key)
    return cache


def clear_implicit_layout_caches() -> None:
    """Drops the library-owned caches of calls made without ``layout_cache`` (and the layouts, LUTs and
    plans they hold)."""
    with _implicit_lock:
        _implicit_caches.clear()


def set_implicit_layout_caches(enabled: bool) -> None:
    """Switches the library-owned caches on or off (off: every call without ``layout_cache`` rebuilds its
    metadata, as the reference does)."""
    global _implicit_enabled
    _implicit_enabled = bool(enabled)
    if not enabled:
        clear_implicit_layout_caches()


def prepare_layout_cache(layout_cache: LayoutCache | None, operation: str, *values: object) -> LayoutCache:
    """Returns a cache dict for ``operation`` that is empty unless it was built for exactly these inputs.

    A cache is reused only if the operation name, the identity / version /
    shape / stride / dtype / device / requires_grad of every tensor argument
    and every scalar argument are unchanged, and nothing stored in the cache
    was replaced or mutated since ``finalize_layout_cache``.
    """
    if layout_cache is None:
        layout_cache = implicit_layout_cache(operation, *values)
    if layout_cache is None:
        layout_cache = {}
    held: list[Tensor] = []
    wanted = _cache_key(operation, values, held)
    recorded = layout_cache.get(_STATE)
    fresh = (layout_cache.get(_KEY) != wanted or recorded is None
             or _cache_contents_state(layout_cache) != recorded)
    if fresh:
        layout_cache.clear()
        layout_cache[_KEY] = wanted
        # holding the source tensors keeps their ids from being recycled
        layout_cache[_REFS] = tuple(held)
    return layout_cache


def finalize_layout_cache(layout_cache: LayoutCache) -> LayoutCache:
    """Records the cache contents so that later caller mutations invalidate them."""
    layout_cache[_STATE] = _cache_contents_state(layout_cache)
    return layout_cache


# ---- small helpers -----------------------------------------------------------

def stride(x: Tensor):
    """Strides a contiguous tensor of this shape has (1-D to 3-D)."""
    if x.dim() == 1:
        return 1
    if x.dim() == 2:
        return x.size(1), 1
    if x.dim() == 3:
        return x.size(1) * x.size(2), x.size(2), 1
    raise NotImplementedError(f"stride() not implemented for {x.dim()}-dimensional tensors")


def can_use_int32_indexing(*values: Tensor | int | None) -> bool:
    """True if every buffer (tensor numel or explicit count) fits signed int32 element indices."""
    for value in values:
        if value is None:
            continue
        count = value.numel() if isinstance(value, Tensor) else int(value)
        if count > INT32_INDEX_MAX:
            return False
    return True


def cast_for_autocast(*values: Tensor):
    """Casts fp16/bf16/fp32 CUDA tensors to the active autocast dtype; fp64 is left alone so validation rejects it."""
    if torch.is_autocast_enabled():
        target = torch.get_autocast_dtype("cuda")
        values = tuple(v.to(target) if v.is_cuda and v.dtype in (torch.float16, torch.bfloat16, torch.float32) else v
                       for v in values)
    return values[0] if len(values) == 1 else values


def do_shape_blocksparse(x: Tensor) -> tuple[Tensor, Size]:
    """Folds all leading dimensions into one batch dimension; returns the 3-D tensor and the original shape."""
    if x.dim() < 2:
        raise ValueError("Tensor must have at least 2 dimensions")
    if x.dim() == 3:
        return x.contiguous(), x.size()
    batch = 1
    for extent in x.shape[:-2]:
        batch *= extent
    return x.reshape(batch, x.size(-2), x.size(-1)).contiguous(), x.size()


def undo_shape_blocksparse(x: Tensor, shape: Size | tuple[int, ...]) -> Tensor:
    """Restores the leading dimensions folded by ``do_shape_blocksparse`` (trailing two taken from ``x``)."""
    if x.dim() != 3:
        raise ValueError("Tensor must have exactly 3 dimensions")
    if len(shape) < 2:
        raise ValueError("Original shape must have at least 2 dimensions")
    batch = 1
    for extent in shape[:-2]:
        batch *= extent
    if x.size(0) != batch:
        raise ValueError("Tensor batch dimension does not match original shape")
    if x.shape[:-2] == tuple(shape[:-2]):
        return x
    return x.reshape((*shape[:-2], *x.shape[-2:]))
