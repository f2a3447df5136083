"""The cache manager's bookkeeping (no GPU): no page lost, held twice or freed twice."""
import random

import pytest

from openinfer_b200.cache import (RELEASED, CacheManager, DoubleFree, IdPool, KvNeed, OutOfPages, StateNeed)


def make(page=4, pages=10, slots=4, window=None, two_groups=False):
    cm = CacheManager(page_size=page)
    h = [cm.add_kv_layer(KvNeed(2, 16, None)), cm.add_kv_layer(KvNeed(2, 16, None))]
    if two_groups or window:
        h.append(cm.add_kv_layer(KvNeed(2, 16, window)))
    cm.add_state(StateNeed((3,)))
    cm.allocate(pages, slots)
    return cm, h


def test_pool_basics():
    p = IdPool(3)
    a = p.allocate(2)
    assert sorted(a) == [0, 1] and p.free_count == 1
    with pytest.raises(OutOfPages):
        p.allocate(2)
    assert p.free_count == 1  # nothing taken
    p.release([a[0]])
    with pytest.raises(DoubleFree):
        p.release([a[0]])
    with pytest.raises(DoubleFree):
        p.release([a[1], a[1]])
    p.check()
    assert p.allocate(1) == [a[0]]  # last freed, first reused


def test_layers_with_same_need_share_a_group():
    cm, h = make(two_groups=True, window=6)
    assert h[0].group == h[1].group == 0 and (h[0].layer, h[1].layer) == (0, 1)
    assert h[2].group == 1 and len(cm.groups) == 2 and cm.groups[0].layers == 2
    assert cm.bytes_per_page(0, 2) == 2 * 2 * 4 * 2 * 16 * 2


def test_exact_pages_at_every_boundary():
    cm, _ = make(page=4, pages=64)
    cm.open("r")
    total = 0
    for n in [1, 2, 1, 4, 3, 5, 1, 1, 1, 8, 2]:
        start = cm.reserve("r", n)
        assert start == total
        total += n
        assert len(cm.block_table("r", 0)) == -(-total // 4)  # exactly ceil(tokens / page)
        cm.commit("r")
        assert cm.num_tokens("r") == total
        cm.check()
    cm.close("r")
    assert cm.free_pages() == [64]
    cm.check()


def test_out_of_pages_changes_nothing_and_rollback():
    cm, _ = make(page=4, pages=3)
    cm.open("a")
    cm.reserve("a", 8)
    cm.commit("a")
    cm.open("b")
    with pytest.raises(OutOfPages):
        cm.reserve("b", 5)  # needs 2, 1 free
    assert cm.free_pages() == [1] and cm.block_table("b", 0) == []
    cm.reserve("b", 4)
    cm.rollback("b")
    assert cm.free_pages() == [1] and cm.num_tokens("b") == 0
    cm.check()
    with pytest.raises(RuntimeError):
        cm.commit("b")  # nothing reserved
    cm.close("a")
    cm.close("b")
    assert cm.free_pages() == [3]
    with pytest.raises(KeyError):
        cm.close("a")


def test_state_slots():
    cm, _ = make(slots=2)
    s0, s1 = cm.open("a"), cm.open("b")
    assert {s0, s1} == {0, 1}
    with pytest.raises(OutOfPages):
        cm.open("c")
    with pytest.raises(KeyError):
        cm.open("a")
    cm.close("a")
    assert cm.open("c") == s0
    cm.check()


def test_window_pages_go_back_when_passed():
    W, P = 6, 4
    cm, _ = make(page=P, pages=16, window=W)
    cm.open("r")
    total = 0
    for n in [3, 5, 1, 1, 7, 2, 1, 1, 1, 1, 9]:
        cm.reserve("r", n)
        total += n
        cm.commit("r")
        table = cm.block_table("r", 1)
        # a later query at position >= total sees keys > total - W: pages wholly below are released
        first_needed = max(0, total - W + 1) // P
        for i, p in enumerate(table):
            assert (p == RELEASED) == (i < first_needed), (total, i, table)
        assert all(p != RELEASED for p in cm.block_table("r", 0))  # the full-attention group keeps all
        cm.check()
    assert cm.groups[1].pool.used_count <= -(-W // P) + 1
    cm.close("r")
    assert cm.free_pages() == [16, 16]


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_invariants(seed):
    rng = random.Random(seed)
    cm, _ = make(page=4, pages=24, slots=5, window=rng.choice([None, 5, 9]))
    live, next_id = {}, 0
    for _ in range(400):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            cm.open(next_id)
            live[next_id] = 0
            next_id += 1
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 3, 7, 13])
            try:
                cm.reserve(rid, n)
            except OutOfPages:
                before = cm.free_pages()
                cm.check()
                assert cm.free_pages() == before
                continue
            if rng.random() < 0.15:
                cm.rollback(rid)
            else:
                cm.commit(rid)
                live[rid] += n
            assert cm.num_tokens(rid) == live[rid]
        elif live:
            rid = rng.choice(list(live))
            cm.close(rid)
            del live[rid]
        cm.check()
    for rid in list(live):
        cm.close(rid)
    cm.check()
    assert all(f == 24 for f in cm.free_pages()) and cm.slot_pool.free_count == 5
