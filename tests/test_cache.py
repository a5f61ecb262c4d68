"""The cache manager's bookkeeping (no GPU, no tensors): no page lost, held twice or
freed twice under random orders of requests; windows give pages back; slots."""

import random

import pytest

from pulsarlm_b200.cache.manager import CacheError, CacheManager
from pulsarlm_b200.cache.pages import PageError, PagePool
from pulsarlm_b200.parts.spec import KVCacheNeed, StateNeed


def manager(needs, page=4, pages=12, slots=4):
    import torch

    return CacheManager(needs, page, pages, slots, torch.float32, None, allocate=False)


def check_invariants(m: CacheManager):
    for g in m.groups:
        held = [p for r in m.open_requests() for p in m.held_pages(r, g.index)]
        assert len(held) == len(set(held)), "a page is held twice"
        assert len(held) == g.pool.used_count, "a page is lost or counted twice"
        assert all(g.pool.is_held(p) for p in held)
        assert g.pool.used_count + g.pool.free_count == g.pool.n_pages
    slots = [m.slot(r) for r in m.open_requests()]
    assert len(slots) == len(set(slots))


def test_pool_take_is_all_or_nothing_and_lifo():
    pool = PagePool(4)
    a = pool.take(3)
    assert a == [0, 1, 2] and pool.take(2) is None and pool.free_count == 1
    pool.give([1])
    assert pool.take(1) == [1]  # the page given back last is reused first
    with pytest.raises(PageError):
        pool.give([3])  # never taken
    pool.give([0])
    with pytest.raises(PageError):
        pool.give([0])  # freed twice
    assert pool.high_water == 3


def test_groups_by_need_and_layer_binding_order():
    full = KVCacheNeed(2, 8)
    win = KVCacheNeed(2, 8, window=6)
    m = manager([full, win, full, None, StateNeed((3,)), win])
    assert [g.layers for g in m.groups] == [[0, 2], [1, 5]]
    assert m.layer_group == {0: 0, 2: 0, 1: 1, 5: 1}
    assert list(m.state_layers) == [4]


def test_reserve_commit_close_and_tables():
    m = manager([KVCacheNeed(1, 4)], page=4, pages=5, slots=2)
    assert m.open("a") == 0 and m.open("b") == 1 and m.open("c") is None
    assert m.reserve("a", 9) and m.held_pages("a", 0) == [0, 1, 2]
    m.commit("a", 9)
    assert m.reserve("a", 12) and m.held_pages("a", 0) == [0, 1, 2]  # still fits page 2
    assert not m.reserve("b", 9)  # needs 3, only 2 free: nothing taken
    assert m.held_pages("b", 0) == [] and m.free_pages() == 2
    assert m.reserve("b", 8)
    table = m.table_rows(0, ["b", "a"])
    assert table.shape == (2, 8) and table[0, :2].tolist() == [3, 4] and table[1, :3].tolist() == [0, 1, 2]
    assert (table[0, 2:] == -1).all()
    m.close("a")
    assert m.open("c") == 0  # the slot is used again
    assert m.reserve("c", 4) and m.held_pages("c", 0) == [2]  # and the page freed last
    check_invariants(m)
    with pytest.raises(CacheError):
        m.commit("c", 9)  # no pages reserved for that length
    with pytest.raises(CacheError):
        m.open("c")


def test_window_gives_pages_back_as_it_passes():
    m = manager([KVCacheNeed(1, 4, window=6), KVCacheNeed(1, 4)], page=4, pages=8, slots=1)
    m.open("r")
    for new_len in range(1, 30):
        assert m.reserve("r", new_len)
        m.commit("r", new_len)
        # keys >= new_len - 6 + 1 stay readable; pages wholly before them are gone
        first_page = max(0, new_len - 6 + 1) // 4
        rows = m.table_rows(0, ["r"])[0]
        n_pages = -(-new_len // 4)
        assert (rows[:first_page] == -1).all() and (rows[first_page:n_pages] >= 0).all()
        assert len(m.held_pages("r", 0)) <= 3
        assert len(m.held_pages("r", 1)) == n_pages
        check_invariants(m)
    m.close("r")
    assert all(g.pool.used_count == 0 for g in m.groups)


def test_long_portion_in_a_windowed_group_holds_all_its_pages_for_the_step():
    m = manager([KVCacheNeed(1, 4, window=4)], page=4, pages=8, slots=1)
    m.open("r")
    assert m.reserve("r", 20) and len(m.held_pages("r", 0)) == 5
    m.commit("r", 20)
    assert len(m.held_pages("r", 0)) == 1


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_keep_the_invariants(seed):
    rng = random.Random(seed)
    m = manager([KVCacheNeed(2, 8), KVCacheNeed(2, 8, window=5), StateNeed((2,))], page=4, pages=10, slots=3)
    lengths = {}
    next_id = 0
    for _ in range(400):
        action = rng.random()
        live = list(lengths)
        if action < 0.25 or not live:
            rid = f"r{next_id}"
            next_id += 1
            if m.open(rid) is not None:
                lengths[rid] = 0
            else:
                assert len(live) == 3
        elif action < 0.85:
            rid = rng.choice(live)
            grow = rng.choice([1, 1, 1, 2, 5, 13])
            before = [g.pool.free_count for g in m.groups]
            if m.reserve(rid, lengths[rid] + grow):
                lengths[rid] += grow
                m.commit(rid, lengths[rid])
            else:
                assert before == [g.pool.free_count for g in m.groups], "a failed reserve took pages"
        else:
            rid = rng.choice(live)
            m.close(rid)
            del lengths[rid]
        check_invariants(m)
        for rid, n in lengths.items():
            assert m.length(rid) == n
    for rid in list(lengths):
        m.close(rid)
    assert all(g.pool.used_count == 0 for g in m.groups) and m.stats()["slots_used"] == 0


def test_a_windowed_group_gets_only_the_pages_its_requests_can_hold():
    import torch

    needs = [KVCacheNeed(2, 8), KVCacheNeed(2, 8, window=10), KVCacheNeed(2, 8, window=300)]
    m = CacheManager(needs, 4, 100, 3, torch.float32, None, allocate=False, step_tokens=6)
    # window 10, at most 6 tokens a step, pages of 4: ceil(17 / 4) + 1 = 6 pages a request
    assert [g.pool.n_pages for g in m.groups] == [100, 3 * 6, 100]
    # without a bound on a step's tokens every group is sized alike
    same = CacheManager(needs, 4, 100, 3, torch.float32, None, allocate=False)
    assert [g.pool.n_pages for g in same.groups] == [100, 100, 100]


@pytest.mark.parametrize("seed", range(6))
def test_the_smaller_pool_of_a_windowed_group_never_runs_out_first(seed):
    """Requests that bring at most `step_tokens` tokens a step: as long as the group that
    keeps every key has room, so has the windowed one (also when the step before is
    committed only after the next was reserved, as pipelined decode steps do)."""
    import torch

    rng = random.Random(seed)
    page, window, step_tokens, slots = rng.choice([2, 4, 8]), rng.randint(1, 40), rng.randint(1, 12), 3
    needs = [KVCacheNeed(1, 4), KVCacheNeed(1, 4, window=window)]
    m = CacheManager(needs, page, 4000, slots, torch.float32, None, allocate=False, step_tokens=step_tokens)
    assert m.groups[1].pool.n_pages < 4000
    lengths, late = {}, {}
    for step in range(600):
        live = list(lengths)
        if len(live) < slots and rng.random() < 0.3:
            name = f"r{step}"
            assert m.open(name) is not None
            lengths[name] = 0
        elif live and rng.random() < 0.05:
            name = rng.choice(live)
            m.close(name)
            del lengths[name]
            late.pop(name, None)
        for name in lengths:
            n = rng.randint(1, step_tokens) if lengths[name] == 0 or rng.random() < 0.3 else 1
            if name in late:
                # a single token reserved before the step before it is committed
                assert m.reserve(name, late[name] + 1)
                m.commit(name, late[name])
                m.commit(name, late[name] + 1)
                lengths[name] = late.pop(name) + 1
                continue
            new_len = lengths[name] + n
            assert m.reserve(name, new_len), (name, lengths[name], n, m.stats())
            if rng.random() < 0.3:
                late[name] = new_len
            else:
                m.commit(name, new_len)
            lengths[name] = new_len
        check_invariants(m)
        assert m.groups[1].pool.high_water <= m.groups[1].pool.n_pages


def test_a_byte_budget_is_split_among_groups_by_what_they_can_hold():
    import torch

    from pulsarlm_b200.cache.manager import cache_bytes
    from pulsarlm_b200.engine.engine import pages_for_bytes

    needs = [KVCacheNeed(2, 16), KVCacheNeed(2, 16, window=40), KVCacheNeed(2, 16), None, StateNeed((4,))]
    for budget in (1 << 16, 1 << 20, 3 << 20):
        n = pages_for_bytes(needs, 8, 4, torch.float32, 32, budget)
        assert cache_bytes(needs, n, 8, 32, 4, torch.float32) <= budget < cache_bytes(needs, n + 1, 8, 32, 4, torch.float32)
    # the windowed layer's pool stops growing at what four requests can hold: more of the budget goes to the others
    even = (1 << 20) // (3 * 2 * 2 * 8 * 16 * 4)
    assert pages_for_bytes(needs, 8, 4, torch.float32, 32, 1 << 20) > even
    # a model whose groups all have windows, or that keeps no keys at all, still gets an answer
    assert pages_for_bytes([KVCacheNeed(1, 8, window=16)], 8, 2, torch.float32, 8, 1 << 30) >= 1
    assert pages_for_bytes([None, StateNeed((2,))], 8, 2, torch.float32, 8, 1 << 30) >= 1
