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


def test_pool_hands_out_ascending_runs():
    """A fresh pool gives consecutive ids in ascending order, and ids that come back together come out ascending
    again (before older free ones): neighbouring table entries then name neighbouring pages."""
    p = IdPool(12)
    assert p.allocate(5) == [0, 1, 2, 3, 4]
    b = p.allocate(4)
    assert b == [5, 6, 7, 8]
    p.release([7, 5, 8, 6])
    assert p.allocate(3) == [5, 6, 7]
    p.release([2, 0, 1])
    assert p.allocate(5) == [0, 1, 2, 8, 9]
    p.check()


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


# ---------------------------------------------------------------------------
# prefix cache: registered full pages of prompt tokens, shared between requests
# ---------------------------------------------------------------------------
def _prefix_cm(pages=12, page=4, groups=2):
    from openinfer_b200.cache import CacheManager, KvNeed
    cm = CacheManager(page_size=page, prefix_cache=True)
    for g in range(groups):
        cm.add_kv_layer(KvNeed(2 + g, 8))
    cm.allocate(pages, 6)
    return cm


def _run(cm, rid, tokens, chunk=100):
    """begin + prefill in portions; returns the cached token count."""
    cached = cm.begin(rid, tokens)
    at = cached
    while at < len(tokens):
        n = min(chunk, len(tokens) - at)
        assert cm.reserve(rid, n) == at
        cm.commit(rid, tokens=tokens[at: at + n])
        at += n
    return cached


def test_prefix_cache_shares_full_prompt_pages_and_leaves_one_token():
    cm = _prefix_cm()
    a = list(range(100, 111))                 # 11 tokens: two full pages and 3
    assert _run(cm, "a", a, chunk=5) == 0
    cm.check()
    # the same prompt again: the two full pages are shared, the rest is computed
    assert _run(cm, "b", a) == 8
    assert cm.block_table("b", 0)[:2] == cm.block_table("a", 0)[:2] and cm.block_table("b", 1)[:2] == cm.block_table("a", 1)[:2]
    assert cm.block_table("b", 0)[2] != cm.block_table("a", 0)[2]
    cm.check()
    # a prompt of exactly two pages: only ONE page may be taken from the cache (a token must be left to compute)
    assert _run(cm, "c", a[:8]) == 4
    # a different second page: one page shared
    assert _run(cm, "d", a[:4] + [1, 2, 3, 4, 5]) == 4
    # a different first token: nothing shared, although later pages hold the same tokens
    assert _run(cm, "e", [7] + a[1:]) == 0
    cm.check()
    for r in "abcde":
        cm.close(r)
    cm.check()
    assert cm.min_free_pages() == 12 and cm.prefix_hits == 16
    # registered pages outlive their requests: a newcomer still finds them
    assert _run(cm, "f", a) == 8
    cm.close("f")
    cm.check()


def test_prefix_cache_evicts_idle_pages_when_room_is_needed_and_never_a_used_one():
    cm = _prefix_cm(pages=6, page=4, groups=1)
    a, b = list(range(10, 19)), list(range(50, 59))       # 9 tokens each: two full pages and 1 -> 3 pages
    _run(cm, "a", a)
    cm.close("a")                                          # two idle registered pages, one free again
    assert cm.min_free_pages() == 6 and len(cm._idle) == 2
    _run(cm, "b", b)                                       # takes 3 of the 4 truly free pages
    _run(cm, "a2", a)                                      # shares a's two pages, takes the last free one
    assert cm.prefix_hits == 8 and cm.min_free_pages() == 0
    with pytest.raises(Exception):                         # nothing free, nothing idle: a's pages are in use
        cm.begin("c", list(range(90, 99))) or cm.reserve("c", 9)
    cm.close("c")
    cm.close("a2")
    assert len(cm._idle) == 2 and cm.min_free_pages() == 3
    _run(cm, "d", list(range(70, 82)))                    # 12 tokens: 3 pages: must evict idle ones
    cm.check()
    assert len(cm._idle) <= 1
    # the leaf page of `a` went first: its root may still match
    cm.close("d"); cm.close("b")
    cm.check()
    assert cm.min_free_pages() == 6


def test_prefix_cache_tokens_unknown_to_the_host_end_registration_and_random_traffic_keeps_the_books():
    import random
    cm = _prefix_cm(pages=40, page=4, groups=2)
    cm.begin("x", [1, 2, 3, 4, 5, 6])
    cm.reserve("x", 6); cm.commit("x", tokens=[1, 2, 3, 4, 5, 6])      # one page registered
    cm.reserve("x", 1); cm.commit("x")                                 # a token still on the device: no more pages
    cm.reserve("x", 5); cm.commit("x", tokens=[9] * 5)
    assert len(cm.requests["x"].blocks) == 1
    cm.close("x")
    rng = random.Random(0)
    stems = [[rng.randrange(5) for _ in range(12)] for _ in range(3)]
    live = []
    for step in range(300):
        if live and (rng.random() < 0.4 or len(live) >= 5):
            cm.close(live.pop(rng.randrange(len(live))))
        else:
            rid = f"r{step}"
            prompt = stems[rng.randrange(3)][: rng.randrange(1, 13)] + [rng.randrange(5) for _ in range(rng.randrange(0, 6))]
            try:
                _run(cm, rid, prompt, chunk=rng.randrange(1, 7))
                live.append(rid)
            except Exception:
                if cm.has(rid):
                    cm.rollback(rid); cm.close(rid)
        cm.check()
    for rid in live:
        cm.close(rid)
    cm.check()
    assert cm.min_free_pages() == 40 and cm.prefix_hits > 0


def test_prefix_cache_is_not_used_with_windows_or_state():
    from openinfer_b200.cache import CacheManager, KvNeed, StateNeed
    cm = CacheManager(page_size=4, prefix_cache=True)
    cm.add_kv_layer(KvNeed(2, 8, window=6))
    cm.allocate(8, 2)
    assert not cm.prefix_usable() and cm.begin("a", list(range(20))) == 0
    cm2 = CacheManager(page_size=4, prefix_cache=True)
    cm2.add_kv_layer(KvNeed(2, 8))
    cm2.add_state(StateNeed((3,)))
    cm2.allocate(8, 2)
    assert not cm2.prefix_usable()
