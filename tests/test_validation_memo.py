"""Validation reads a layout's facts (only 0/1 entries, number of active blocks) from the device once per
layout state and remembers them per layout object; the reference reads them on every call
(blksprs/utils/validation.py:297-315, 358-366).  Same exceptions and messages either way.  Runs on CPU
tensors: the bookkeeping does not depend on the device."""
import gc

import pytest
import torch

from blksprs_b200.utils import validation as v


@pytest.fixture
def reads(monkeypatch):
    """Counts the reductions validation performs on layouts."""
    counts = {"sum": 0, "all": 0}
    real_sum, real_all = torch.sum, torch.all

    def counting_sum(*a, **k):
        counts["sum"] += 1
        return real_sum(*a, **k)

    def counting_all(*a, **k):
        counts["all"] += 1
        return real_all(*a, **k)

    monkeypatch.setattr(torch, "sum", counting_sum)
    monkeypatch.setattr(torch, "all", counting_all)
    return counts


def test_unchanged_layout_is_read_once(reads):
    layout = torch.ones((2, 3, 3), dtype=torch.float32)
    x = torch.zeros((18, 16, 16))
    for _ in range(3):
        v.validate_sparsity(16, (x, layout))
    assert reads == {"sum": 1, "all": 1}
    # a second layout object with equal contents is a different layout
    v.validate_sparsity(16, (x, layout.clone()))
    assert reads == {"sum": 2, "all": 2}


def test_in_place_change_is_seen():
    layout = torch.ones((2, 3, 3), dtype=torch.float32)
    x = torch.zeros((18, 16, 16))
    v.validate_sparsity(16, (x, layout))
    layout[0, 0, 0] = 0
    with pytest.raises(ValueError, match="Mismatch between sparsity layout and blocks"):
        v.validate_sparsity(16, (x, layout))
    v.validate_sparsity(16, (x[:17], layout))
    layout[0, 0, 1] = 2
    with pytest.raises(ValueError, match="Sparsity layout values must be either 0 or 1"):
        v.validate_sparsity(16, (x[:17], layout))


def test_bool_layouts_skip_the_value_check(reads):
    layout = torch.ones((1, 2, 2), dtype=torch.bool)
    for _ in range(2):
        v.validate_sparsity(16, (torch.zeros((4, 16, 16)), layout))
    assert reads == {"sum": 1, "all": 0}


def test_inference_layouts_are_never_remembered(reads):
    with torch.inference_mode():
        layout = torch.ones((1, 2, 2))
    x = torch.zeros((4, 16, 16))
    before = len(v._layout_facts)
    for _ in range(2):
        v.validate_sparsity(16, (x, layout))
    assert reads == {"sum": 2, "all": 2} and len(v._layout_facts) == before


def test_records_go_with_their_layout():
    layout = torch.ones((1, 2, 2))
    v.validate_sparsity(16, (torch.zeros((4, 16, 16)), layout))
    gc.collect()
    n = len(v._layout_facts)
    del layout
    gc.collect()
    assert len(v._layout_facts) <= n - 1   # other tests' layouts may go at the same time


def test_switched_off_validation_reads_nothing(reads):
    layout = torch.ones((1, 2, 2))
    v.disable_validation()
    try:
        v.validate_sparsity(16, (torch.zeros((3, 16, 16)), layout))   # wrong count, unchecked
    finally:
        v.enable_validation()
    assert reads == {"sum": 0, "all": 0}
