"""Host-side bookkeeping of the slot cache (``vllm_integration/state_cache.py``):
slot ownership, page accounting, and which slot every move copies from and to.
The device copy is replaced by an eager one here; the kernels are covered by
``tests/test_gpu_state_cache.py``."""

from __future__ import annotations

import pytest
import torch

from oracle import gdn_oracle as orc
from carrykernel_b200.vllm_integration import quantized_packed_decode as qpd
from carrykernel_b200.vllm_integration import state_cache as sc
from carrykernel_b200.vllm_integration import state_pool


@pytest.fixture
def eager_copies(monkeypatch):
    log = []

    def copy_slots(src_pool, src_indices, dst_indices, dst_pool=None, resid_fmt=qpd.RESID_INT8):
        dst_pool = src_pool if dst_pool is None else dst_pool
        orc.pool_copy(src_pool, dst_pool, src_indices, dst_indices)
        log.append((int(src_indices[0]), int(dst_indices[0]), dst_pool is not src_pool))
    monkeypatch.setattr(state_pool, "copy_slots", copy_slots)
    return log


def _fill(cache, request, value):
    slot = cache.slot(request)
    for pool in cache.pools:
        for t in pool:
            t[slot] = value


def _holds(cache, request, value):
    slot = cache.slot(request)
    return all(bool((t[slot] == value).all()) for pool in cache.pools for t in pool)


def test_page_accounting_follows_state_bytes_per_slot():
    c = sc.SlotCache(3, 5, 32, 128, 128, "cpu", qpd.RESID_INT4, "v", spill_slots=3)
    # the reference's figure for int8 state + packed int4 residual with per-V scales
    # (vllm_integration/quantized_packed_decode.py:355-369): 16384 + 8192 + 2 * 512 bytes per head
    assert c.page_size_bytes() == 32 * (16384 + 8192 + 1024) == orc.state_bytes_per_slot(32, 128, 128, True, resid_fmt=orc.RESID_INT4)
    assert c.bytes_per_request() == 3 * c.page_size_bytes()
    assert c.pages_in_use() == 0 and c.free_slots() == 4
    c.allocate("a"); c.allocate("b")
    assert c.pages_in_use() == 2 * 3 and c.bytes_in_use() == 6 * c.page_size_bytes()
    assert c.capacity_bytes() == (5 + 3) * c.bytes_per_request()
    head = sc.SlotCache(1, 2, 32, 128, 128, "cpu", qpd.RESID_INT4, "head")
    assert head.page_size_bytes() == 32 * (16384 + 8192 + 512 + 4)
    held = sum(t.numel() * t.element_size() for t in head.pools[0]) // 2      # 2 slots allocated (one is padding)
    assert held == head.page_size_bytes()


def test_slots_are_unique_never_zero_and_reused():
    c = sc.SlotCache(1, 4, 2, 8, 8, "cpu")
    slots = [c.allocate(r) for r in "abc"]
    assert sorted(slots) == [1, 2, 3]
    with pytest.raises(sc.CacheFull):
        c.allocate("d")
    with pytest.raises(ValueError):
        c.allocate("a")
    c.free("b")
    assert c.allocate("d") == slots[1]
    idx = c.indices(["a", None, "d"], pad_to=5)
    assert idx.dtype == torch.int32 and idx.tolist() == [slots[0], 0, slots[1], 0, 0]
    with pytest.raises(KeyError):
        c.free("zzz")


def test_preempt_resume_fork_and_rollback_move_the_right_slots(eager_copies):
    c = sc.SlotCache(2, 4, 2, 8, 8, "cpu", qpd.RESID_INT8, "v", spill_slots=4)
    a, b = c.allocate("a"), c.allocate("b")
    _fill(c, "a", 11); _fill(c, "b", 22)
    c.preempt("a")
    assert not c.is_running("a") and c.free_slots() == 2
    c.allocate("intruder")                          # takes a's old slot
    assert c.slot("intruder") == a
    _fill(c, "intruder", 99)
    new_a = c.resume("a")
    assert new_a != a and _holds(c, "a", 11) and _holds(c, "b", 22) and _holds(c, "intruder", 99)
    # speculative tokens on b, rejected
    tok = c.checkpoint("b")
    _fill(c, "b", 33)
    c.rollback(tok)
    assert _holds(c, "b", 22)
    tok = c.checkpoint("b")
    _fill(c, "b", 44)
    c.release_checkpoint(tok)
    assert _holds(c, "b", 44)
    c.free("intruder")
    c.fork("a", "child")
    assert _holds(c, "child", 11) and c.slot("child") != c.slot("a")
    # every copy touched both layers; spill traffic went through the second pool
    assert len(eager_copies) % 2 == 0 and any(x[2] for x in eager_copies)
    assert c.pages_in_use() == 3 * 2                 # a, b, child; no spill slot left in use
    with pytest.raises(KeyError):
        c.rollback(tok)
    # freeing a request drops its checkpoints too
    tok = c.checkpoint("a")
    c.free("a")
    assert c.pages_in_use() == 2 * 2


def test_spill_pool_can_run_out(eager_copies):
    c = sc.SlotCache(1, 3, 2, 8, 8, "cpu", spill_slots=2)
    c.allocate("a"); c.allocate("b")
    c.preempt("a")
    with pytest.raises(sc.CacheFull):
        c.preempt("b")
    assert c.is_running("b")
