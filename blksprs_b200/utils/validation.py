"""Input validation of the matmul path, with the reference's exception types and messages.

Covers the validators ``bs.ops.matmul`` and the matmul layout helpers call
(blksprs/utils/validation.py:54-99, 179-205, 297-386) and the thread-local
switches ``disable/enable_validation`` and ``disable/enable_contiguous``
(blksprs/utils/validation.py:447-472).
"""
from __future__ import annotations

import threading

import torch
from torch import Tensor
from torch.utils.weak import WeakIdKeyDictionary

_state = threading.local()

_FLOAT_DTYPES = (torch.float16, torch.bfloat16, torch.float32)
_SUPPORTED_MOVE_DTYPES = (torch.bool, torch.uint8, torch.int8, torch.int16, torch.int32, torch.int64,
                          torch.float16, torch.bfloat16, torch.float32, torch.float64)


def validation_enabled() -> bool:
    return getattr(_state, "validation", True)


def contiguous_enabled() -> bool:
    return getattr(_state, "contiguous", True)


def disable_validation() -> None:
    """Turns input validation off for the calling thread."""
    _state.validation = False


def enable_validation() -> None:
    """Turns input validation on for the calling thread."""
    _state.validation = True


def disable_contiguous() -> None:
    """Stops ops from calling ``.contiguous()`` on their inputs (calling thread only)."""
    _state.contiguous = False


def enable_contiguous() -> None:
    """Lets ops call ``.contiguous()`` on their inputs (calling thread only)."""
    _state.contiguous = True


def ensure_contiguous(*tensors: Tensor):
    """Contiguous versions of ``tensors`` unless the thread-local switch is off."""
    if contiguous_enabled():
        tensors = tuple(t.contiguous() for t in tensors)
    return tensors[0] if len(tensors) == 1 else tensors


def validate_dimensions(*tensors: Tensor, dims: int = 3) -> None:
    if not validation_enabled():
        return
    if any(t.dim() != dims for t in tensors):
        raise ValueError(f"Tensor must have {dims} dimensions")


def validate_contiguous(*tensors: Tensor) -> None:
    if not validation_enabled():
        return
    if not all(t.is_contiguous() for t in tensors):
        raise ValueError("Tensor must be contiguous")


def validate_dtype_float(*tensors: Tensor) -> None:
    """All tensors fp16 / bf16 / fp32 and of one dtype."""
    if not validation_enabled():
        return
    for t in tensors:
        if t.dtype not in _FLOAT_DTYPES:
            raise ValueError("Tensor must have either float16, bfloat16, or float32 dtype")
        if t.dtype != tensors[0].dtype:
            raise ValueError("Tensors must have same dtype")


def validate_dtype_float_32(*tensors: Tensor) -> None:
    if not validation_enabled():
        return
    if any(t.dtype != torch.float32 for t in tensors):
        raise ValueError("Tensor must have float32 dtype")


def validate_dtype_supported(*tensors: Tensor) -> None:
    if not validation_enabled():
        return
    if any(t.dtype not in _SUPPORTED_MOVE_DTYPES for t in tensors):
        raise ValueError("Tensor dtype is not supported")


def validate_device(*tensors: Tensor) -> None:
    """All tensors on one CUDA device."""
    if not validation_enabled() or not tensors:
        return
    first = tensors[0].device
    if first.type != "cuda":
        raise ValueError("Tensors must be on GPU")
    if any(t.device != first for t in tensors[1:]):
        raise ValueError("Tensors must be on same device")


def validate_shape(tensor: Tensor, expected_shape, name: str = "Tensor") -> None:
    if not validation_enabled():
        return
    expected = tuple(torch.Size(expected_shape))
    if tuple(tensor.shape) != expected:
        raise ValueError(f"{name} shape {tuple(tensor.shape)} doesn't match expected {expected}")


# What the device reads below establish about a layout is remembered per layout object (weakly) together
# with the state it was established in: version counter, shape, strides, dtype, device.  A later check
# of the same, unchanged layout then needs no device read; an in-place change bumps the version and the
# facts are read again.  Inference tensors have no version counter and are never remembered.  (The
# reference reads on every call: blksprs/utils/validation.py:297-315, 358-366.)
_layout_facts = WeakIdKeyDictionary()


def _layout_state(layout: Tensor) -> tuple:
    return layout._version, layout.shape, layout.stride(), layout.dtype, layout.device


def _known_layout_facts(layout: Tensor) -> dict:
    """The facts on record for ``layout`` in its current state (a fresh record if there are none)."""
    if torch.is_inference(layout):
        return {}
    state = _layout_state(layout)
    entry = _layout_facts.get(layout)
    if entry is None or entry[0] != state:
        entry = (state, {})
        _layout_facts[layout] = entry
    return entry[1]


def validate_layout_values(sparsity_layout: Tensor) -> None:
    """Real dtype and only 0/1 entries (bool layouts need no device read)."""
    if sparsity_layout.is_complex():
        raise ValueError("Sparsity layout must not have a complex dtype")
    if sparsity_layout.dtype == torch.bool:
        return
    facts = _known_layout_facts(sparsity_layout)
    if facts.get("binary"):
        return
    if not bool(torch.all((sparsity_layout == 0) | (sparsity_layout == 1))):
        raise ValueError("Sparsity layout values must be either 0 or 1")
    facts["binary"] = True


def active_block_count(sparsity_layout: Tensor) -> int:
    """Number of non-zero layout entries: one device->host read per layout state."""
    facts = _known_layout_facts(sparsity_layout)
    n_active = facts.get("n_active")
    if n_active is None:
        n_active = int(torch.sum(sparsity_layout.reshape(-1).to(torch.int)))
        facts["n_active"] = n_active
    return n_active


def validate_sparsity(sparsity_block_size: int, *pairs: tuple[Tensor, Tensor], counts=None) -> None:
    """Checks compressed tensors against their layouts.

    ``counts`` may give the already known number of active blocks per layout
    (from a warm layout cache); otherwise the count is read from the device,
    once per layout state.
    """
    if not validation_enabled():
        return
    for i, (tensor, layout) in enumerate(pairs):
        validate_layout_values(layout)
        if tensor.device != layout.device:
            raise ValueError("Tensor and sparsity layout must be on same device")
        if not layout.is_contiguous():
            raise ValueError("Sparsity layout must be contiguous")
        if layout.dim() != 3:
            raise ValueError("Sparsity layout must have exactly 3 dimensions")
        if not (tensor.size(-1) == tensor.size(-2) == sparsity_block_size):
            raise ValueError("Blocks not conforming to sparsity block size")
        known = None if counts is None else counts[i]
        n_active = active_block_count(layout) if known is None else known
        if tensor.size(0) != n_active:
            raise ValueError("Mismatch between sparsity layout and blocks")


def validate_sparsity_dense(sparsity_block_size: int, *pairs: tuple[Tensor, Tensor]) -> None:
    """Checks dense tensors against their layouts (blksprs/utils/validation.py:318-339)."""
    if not validation_enabled():
        return
    for tensor, layout in pairs:
        validate_layout_values(layout)
        if tensor.device != layout.device:
            raise ValueError("Tensor and sparsity layout must be on same device")
        if not layout.is_contiguous():
            raise ValueError("Sparsity layout must be contiguous")
        if layout.dim() != 3:
            raise ValueError("Sparsity layout must have exactly 3 dimensions")
        if tensor.size(0) != layout.size(0):
            raise ValueError("Tensor batch dimension does not match sparsity layout")
        if tensor.size(-1) % sparsity_block_size or tensor.size(-2) % sparsity_block_size:
            raise ValueError("Tensor sizes must be divisible by sparsity block size")
        if (tensor.size(-1) // sparsity_block_size != layout.size(-1)
                or tensor.size(-2) // sparsity_block_size != layout.size(-2)):
            raise ValueError("Tensor not conforming to sparsity layout")


def validate_sparsity_layout(*sparsity_layouts: Tensor) -> None:
    if not validation_enabled():
        return
    for layout in sparsity_layouts:
        validate_layout_values(layout)
        if layout.dim() != 3:
            raise ValueError("Sparsity layout must have exactly 3 dimensions")
        if not layout.is_contiguous():
            raise ValueError("Sparsity layout must be contiguous")
        if layout.device.type != "cuda":
            raise ValueError("Sparsity layout must be on GPU")


def validate_sparsity_block_size(sparsity_block_size: int, *values) -> None:
    if not validation_enabled():
        return
    if isinstance(sparsity_block_size, bool) or not isinstance(sparsity_block_size, int):
        raise TypeError("Sparsity block size must be an integer")
    if sparsity_block_size < 16:
        raise ValueError("Sparsity block size must be at least 16")
    if sparsity_block_size & (sparsity_block_size - 1):
        raise ValueError("Sparsity block size must be a power of 2")
    for value in values:
        size = value if isinstance(value, (torch.Size, tuple, list)) else value.size()
        if size[-1] % sparsity_block_size or size[-2] % sparsity_block_size:
            raise ValueError("Tensor sizes must be divisible by sparsity block size")
