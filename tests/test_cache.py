"""The cache manager's books (no GPU): no page lost, held twice or freed twice, under random
orders of requests; window groups give pages back as the window passes; slots are reused."""

from __future__ import annotations

import random

import pytest
import torch

from tokenomos_b200.cache.manager import CacheError, CacheManager, OutOfPages
from tokenomos_b200.parts.contract import PagedKV, SharedState, SlotState, WindowKV

SPECS = {
    (0, "conv"): SlotState((2, 8)),
    (1, "kv"): PagedKV(2, 16),
    (2, "kv"): WindowKV(2, 16, 10),
    (3, "kv"): PagedKV(2, 16),
    (4, "kv"): WindowKV(1, 8, 10),
    (5, "kv"): SharedState(1, "kv"),
}


def make(pages=20, page=4, slots=4, max_len=None):
    return CacheManager(SPECS, page, pages, slots, torch.float32, "meta", max_len)


def test_layout_of_what_the_specs_ask_for():
    c = make()
    assert set(c.groups) == {("full",), ("window", 10)}
    assert c.groups[("full",)].members == [(1, "kv"), (3, "kv")]
    assert tuple(c.states[(1, "kv")].shape) == (20, 2, 2, 4, 16)
    assert tuple(c.states[(4, "kv")].shape) == (20, 2, 1, 4, 8)
    assert tuple(c.states[(0, "conv")].shape) == (5, 2, 8)
    assert c.states[(5, "kv")] is c.states[(1, "kv")]
    assert c.state_groups[(5, "kv")] == ("full",)
    assert c.bytes_per_page() == 4 * (2 * 2 * 4 * 16 * 3 + 2 * 1 * 4 * 8)


def test_pages_follow_the_tokens_and_return():
    c = make()
    c.admit("a")
    c.extend("a", 9)
    assert c.block_table("a", ("full",)) == [1, 2, 3]
    c.commit("a", 9)
    c.check()
    assert c.free_pages(("full",)) == 19 - 3
    c.admit("b")
    c.extend("b", 1)
    assert c.block_table("b", ("full",)) == [4] and c.slot("b") == 2
    c.release("a")
    c.check()
    c.admit("c")
    c.extend("c", 5)
    assert c.block_table("c", ("full",)) == [1, 2] and c.slot("c") == 1   # lowest free first


def test_window_group_gives_back_what_it_has_passed():
    c = make(page=4)
    c.admit("a")
    total = 0
    for n in (3, 9, 1, 1, 14, 2):
        c.extend("a", n)
        c.commit("a", n)
        total += n
        c.check()
        table = c.block_table("a", ("window", 10))
        first_needed = max(0, total - 10 + 1) // 4
        assert all(p == 0 for p in table[:first_needed])
        assert all(p != 0 for p in table[first_needed:-(-total // 4)])
        assert all(p != 0 for p in c.block_table("a", ("full",))[:-(-total // 4)])
    assert c.free_pages(("window", 10)) > c.free_pages(("full",))


def test_out_of_pages_takes_nothing():
    c = make(pages=4, page=4)           # 3 usable pages = 12 tokens
    c.admit("a")
    c.extend("a", 8)
    c.commit("a", 8)
    c.admit("b")
    assert not c.can_extend("b", 8)
    with pytest.raises(OutOfPages):
        c.extend("b", 8)
    c.check()
    assert c.free_pages(("full",)) == 1
    assert c.can_extend("b", 4)


def test_wrong_use_is_refused():
    c = make()
    c.admit("a")
    with pytest.raises(CacheError, match="already live"):
        c.admit("a")
    c.release("a")
    with pytest.raises(CacheError, match="released twice"):
        c.release("a")
    with pytest.raises(CacheError, match="not live"):
        c.extend("a", 1)
    c.admit("b")
    with pytest.raises(CacheError, match="beyond what was extended"):
        c.commit("b", 3)
    for i in range(3):
        c.admit(i)
    with pytest.raises(OutOfPages, match="slot"):
        c.admit("one too many")


def test_max_len_bounds_the_block_table():
    c = make(pages=200, max_len=16)
    assert c.max_blocks == 4
    c.admit("a")
    c.extend("a", 16)
    c.commit("a", 16)
    assert not c.can_extend("a", 1)
    with pytest.raises(OutOfPages, match="longest sequence"):
        c.extend("a", 1)


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_keep_the_books(seed):
    rng = random.Random(seed)
    c = make(pages=rng.choice([12, 30, 60]), page=rng.choice([1, 4, 8]), slots=4, max_len=120)
    live: dict[int, int] = {}
    next_id = 0
    for _ in range(400):
        op = rng.random()
        if op < 0.25 and c.free_slots():
            c.admit(next_id)
            live[next_id] = 0
            next_id += 1
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 5, 17])
            can = c.can_extend(rid, n)
            if rng.random() < 0.5:           # the scheduler's one call for both
                free_before = c.free_pages()
                assert c.try_extend(rid, n) == can
                if not can:
                    assert c.free_pages() == free_before      # all or nothing
            elif can:
                c.extend(rid, n)
            if can:
                if rng.random() < 0.9:       # sometimes a step is planned and re-planned
                    c.commit(rid, n)
                    live[rid] += n
            else:
                with pytest.raises(OutOfPages):
                    c.extend(rid, n)
        elif live:
            rid = rng.choice(list(live))
            c.release(rid)
            del live[rid]
        c.check()
        for rid, n in live.items():
            assert c.length(rid) == n
    for rid in list(live):
        c.release(rid)
    c.check()
    assert c.free_pages(("full",)) == c.num_pages - 1 and c.free_slots() == 4


def _replay_books(cache, steps):
    """A replay trace at the level of the books: what ``trace_util.run_in_process`` asks of the
    cache manager, without a model."""
    for s in steps:
        for e in s["entries"]:
            if e["id"] not in cache.requests:
                cache.admit(e["id"])
            cache.extend(e["id"], len(e["tokens"]))
        for e in s["entries"]:
            cache.commit(e["id"], len(e["tokens"]))
        for rid in s["end"]:
            cache.release(rid)
        cache.check()


@pytest.mark.parametrize("page", [4, 8, 16])
def test_a_replay_pool_sized_by_its_own_pages_is_exactly_enough_and_shows_a_leak(page):
    """The replay tests size the pool as ``max_live_tokens(steps, page)`` in the configuration's
    own page size: the mixed trace then runs on exactly the pages its live requests need at the
    worst moment (one page fewer cannot hold it), and a manager that leaks a single page when a
    request ends cannot finish the trace. (Broken on purpose below: ``release`` keeps one page
    of the first request that ends.)"""
    import trace_util

    rng = random.Random(page)
    reqs = {f"r{i}": [0] * n for i, n in enumerate([5, 17, 33, 70, 96, 41])}
    steps = trace_util.mixed(reqs, live=4, seed=3)
    need = trace_util.max_live_tokens(steps, page)
    specs = {(0, "conv"): SlotState((2, 8)), (1, "kv"): PagedKV(2, 16)}
    pages = need // page + 1

    def manager(n):
        return CacheManager(specs, page, n, 8, torch.float32, "meta", max_len=max(need, page))

    _replay_books(manager(pages), steps)
    with pytest.raises(OutOfPages):
        _replay_books(manager(pages - 1), steps)

    leaky = manager(pages)
    real_release, leaked = leaky.release, []

    def release_but_keep_a_page(rid):
        st = leaky.requests[rid]
        if not leaked and st.tables[("full",)]:
            leaked.append(st.tables[("full",)].pop())        # this page never goes back
        real_release(rid)

    leaky.release = release_but_keep_a_page
    with pytest.raises((OutOfPages, CacheError)):
        _replay_books(leaky, steps)
    assert leaked


def test_poisoned_pool_keeps_free_pages_and_rows_as_nan():
    c = CacheManager(SPECS, 4, 8, 3, torch.float32, "cpu", poison=True)
    kv, conv = c.states[(1, "kv")], c.states[(0, "conv")]
    assert torch.isnan(kv[1:]).all() and not torch.isnan(kv[0]).any()
    assert torch.isnan(conv[1:]).all() and not torch.isnan(conv[0]).any()
    st = c.admit("a")
    c.extend("a", 6)
    pages = list(st.tables[("full",)])
    kv[pages] = 1.0
    conv[st.slot] = 2.0
    c.commit("a", 6)
    c.release("a")
    assert torch.isnan(kv[pages]).all() and torch.isnan(conv[st.slot]).all()
    # a window group's pages are poisoned as soon as the window has passed them
    st = c.admit("b")
    c.extend("b", 24)
    first = st.tables[("window", 10)][0]
    wkv = c.states[(2, "kv")]
    wkv[first] = 3.0
    c.commit("b", 24)
    assert st.tables[("window", 10)][0] == 0 and torch.isnan(wkv[first]).all()
