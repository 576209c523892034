"""Host logic of the offloaded-expert pipeline, run without a GPU: the record / group builder
and the slot pool's prefetch stack and slot-reuse ordering (a pool created without a context
records the copies it would issue)."""
import pytest
import torch

from mole_b200 import _lib
from mole_b200.core import UniMem, build_records


def make_pool(size, M=128, F=256):
    return UniMem(0, size, torch.bfloat16, [[F, M], [F], [F, M], [M]], dry=True)


def test_records_resident_only():
    recs, groups = build_records(s_experts=5, d_experts=0, ebatch_size=2, use_pool=False,
                                 view_pool_size=0, prefetched=0)
    assert [(r.base_in_all, r.batch_size, r.use_cpu_param) for r in recs] == \
        [(0, 2, False), (2, 2, False), (4, 1, False)]
    assert groups == [[0, 1, 2]]


def test_records_offloaded_wrap_into_groups():
    # 7 offloaded experts, batches of 2, 4 visible slots: the pool wraps after two records
    recs, groups = build_records(s_experts=1, d_experts=7, ebatch_size=2, use_pool=True,
                                 view_pool_size=4, prefetched=3)
    d = [r for r in recs if r.use_cpu_param]
    assert [(r.batch_base, r.base_in_all, r.batch_size, r.view_base, r.prefetched) for r in d] == \
        [(0, 1, 2, 0, 2), (2, 3, 2, 2, 1), (4, 5, 2, 0, 0), (6, 7, 1, 2, 0)]
    assert groups == [[0, 1, 2], [3, 4]]


def test_records_batch_limited_by_visible_pool():
    recs, groups = build_records(0, 5, ebatch_size=8, use_pool=True, view_pool_size=2, prefetched=0)
    assert [r.batch_size for r in recs] == [2, 2, 1]
    assert [r.view_base for r in recs] == [0, 0, 0]
    assert groups == [[0], [1], [2]]
    with pytest.raises(RuntimeError):
        build_records(0, 3, 4, True, 0, 0)


def test_prefetch_stack_and_view():
    p = make_pool(8)
    assert p.view_pool_size() == 8
    assert p.prefetch(moe_id=1, n=3) == 0
    assert p.view_pool_size() == 5
    assert p.prefetch(1, 2) == 3              # same layer on top of the stack: merged
    assert p.prefetch(2, 1) == 5
    assert p.view_pool_size() == 2
    assert p.abs_slot(0) == 6                 # the visible pool starts after the reservations
    assert p.fetch_top_prefetched_batch(1) == 0        # layer 1 is not on top
    assert p.fetch_top_prefetched_batch(2) == 1
    assert p.fetch_top_prefetched_batch(1) == 5
    assert p.view_pool_size() == 8 and p.abs_slot(0) == 0
    with pytest.raises(_lib.MoleError) as e:
        p.prefetch(3, 9)
    assert e.value.status == -5
    p.prefetch(3, 2)
    p.clear_virtual_mem()
    assert p.view_pool_size() == 8


def test_fetch_plan_skips_prefetched_and_orders_slot_reuse():
    p = make_pool(4)
    host = [None, None, None, None]           # never dereferenced by a pool without a context
    first = p.prefetch(0, 2)
    p.fetch(host, 0, 2, first, 0, absolute=True)       # prefetch copy into the reserved slots
    assert p.fetch_top_prefetched_batch(0) == 2
    t0 = p.fetch(host, 0, 2, 0, 2)            # both experts already there: nothing to copy
    t1 = p.fetch(host, 2, 2, 2, 0)
    p.mark_used(0, 2, torch.cuda.Stream() if torch.cuda.is_available() else _FakeStream())
    p.mark_used(2, 2, _FakeStream())
    t2 = p.fetch(host, 4, 2, 0, 0)            # reuses slots 0,1: must wait for their last user
    assert (t0, t1, t2) == (1, 2, 3)
    assert p.log() == [
        (0, 0, 0, 2),                          # copy 2 experts from expert 0 into slot 0
        (0, 2, 2, 2),                          # copy experts 2,3 into slots 2,3
        (1, 0, 2, 0), (1, 2, 2, 0),            # slots marked used
        (2, 0, 0, 0), (2, 1, 0, 0),            # the refill waits for slots 0 and 1
        (0, 4, 0, 2),
    ]
    with pytest.raises(_lib.MoleError):
        p.fetch(host, 0, 3, 2, 0)             # runs past the end of the pool


class _FakeStream:
    cuda_stream = 0
