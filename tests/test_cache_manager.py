"""The cache manager on the CPU: no page lost, held twice or freed twice, under
random orders of requests; windows give pages back; state slots."""
import random

import pytest

from mini_llm_b200.cache.manager import RELEASED, CacheManager, PagedNeed, StateNeed
from mini_llm_b200.cache.pages import PageAllocator, PageError


def test_allocator_basics():
    a = PageAllocator(4)
    p = a.allocate(3)
    assert sorted(p) == [0, 1, 2] and a.num_free == 1 and not a.can_allocate(2)
    with pytest.raises(PageError):
        a.allocate(2)
    assert a.num_free == 1                      # all or nothing
    a.free([p[0]])
    with pytest.raises(PageError):
        a.free([p[0]])                          # freed twice
    with pytest.raises(PageError):
        a.free([17])                            # invalid id
    assert a.allocate(1) == [p[0]]              # last freed, first reused
    a.check()


def _manager(num_pages=8, page=4, seqs=3, window=None):
    needs = {0: PagedNeed(2, 16), 1: PagedNeed(2, 16), 2: PagedNeed(2, 16, window=window) if window else PagedNeed(2, 16)}
    return CacheManager(needs, page_size=page, num_pages=num_pages, max_num_seqs=seqs, allocate=False)


def test_groups_by_need():
    cm = _manager(window=6)
    assert len(cm.groups) == 2
    assert cm.groups[0].layers == [0, 1] and cm.groups[1].layers == [2]
    assert cm.group_of_layer == {0: 0, 1: 0, 2: 1}


def test_reserve_commit_release():
    cm = _manager()
    cm.admit("a")
    assert cm.reserve("a", 5) and cm.table("a", 0) == [0, 1]
    cm.commit("a", 5)
    assert cm.reserve("a", 3) and len(cm.table("a", 0)) == 2         # 8 tokens fit two pages
    cm.commit("a", 3)
    assert cm.reserve("a", 1) and len(cm.table("a", 0)) == 3
    assert cm.slots_for("a", 0, 7, 2) == [1 * 4 + 3, cm.table("a", 0)[2] * 4]
    cm.admit("b")
    assert not cm.reserve("b", 4 * 6)                                 # 6 pages wanted, 5 free
    assert cm.table("b", 0) == [] and cm.num_free_pages() == 5       # nothing taken
    cm.release("a")
    assert cm.num_free_pages() == 8
    with pytest.raises(PageError):
        cm.release("a")
    with pytest.raises(PageError):
        cm.commit("b", 9)                                              # committing what was never reserved
    cm.check()


def test_slots_are_limited_and_reused():
    cm = _manager(seqs=2)
    s0, s1 = cm.admit("a"), cm.admit("b")
    assert {s0, s1} == {0, 1} and not cm.can_admit()
    with pytest.raises(PageError):
        cm.admit("c")
    cm.release("a")
    assert cm.admit("c") == s0
    cm.check()


def test_window_pages_go_back_as_the_window_passes():
    cm = _manager(num_pages=6, page=4, window=6)
    cm.admit("a")
    for n in (3, 4, 2, 5, 1, 1, 1, 1):
        assert cm.reserve("a", n)
        cm.commit("a", n)
        c = cm.computed("a")
        tab = cm.table("a", 1)
        first_needed = max(0, c - 6 + 1) // 4
        assert all(p == RELEASED for p in tab[:first_needed]) and all(p != RELEASED for p in tab[first_needed:])
        assert all(p != RELEASED for p in cm.table("a", 0))          # the full-attention group keeps everything
        cm.check()
    assert cm.computed("a") == 18
    assert cm.groups[1].allocator.num_in_use == 2 and cm.groups[0].allocator.num_in_use == 5
    with pytest.raises(PageError):
        cm.slots_for("a", 1, 0, 1)
    cm.release("a")
    assert cm.num_free_pages(0) == 6 and cm.num_free_pages(1) == 6


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_nothing(seed):
    rng = random.Random(seed)
    cm = _manager(num_pages=20, page=4, seqs=5, window=9 if seed % 2 else None)
    live, n_done = {}, 0
    for it in range(600):
        r = rng.random()
        if r < 0.25 and cm.can_admit():
            rid = f"r{it}"
            cm.admit(rid)
            live[rid] = 0
        elif r < 0.85 and live:
            rid = rng.choice(sorted(live))
            n = rng.choice([1, 1, 1, 2, 3, 7, 13])
            before = [cm.num_free_pages(g.index) for g in cm.groups]
            if cm.reserve(rid, n):
                if rng.random() < 0.9:
                    cm.commit(rid, n)
                    live[rid] += n
                    assert cm.computed(rid) == live[rid]
            else:
                assert before == [cm.num_free_pages(g.index) for g in cm.groups]
        elif live:
            rid = rng.choice(sorted(live))
            cm.release(rid)
            del live[rid]
            n_done += 1
        cm.check()
    for rid in list(live):
        cm.release(rid)
    cm.check()
    assert all(g.allocator.num_free == 20 for g in cm.groups) and n_done > 10


def test_state_slots_are_zeroed_on_admit():
    import torch
    cm = CacheManager({0: StateNeed((3,), "float32"), 1: PagedNeed(1, 16)}, page_size=4, num_pages=2, max_num_seqs=2,
                      dtype=torch.float32, device="cpu")
    assert cm.states[0].shape == (2, 3) and cm.groups[0].pool.shape == (1, 2, 2, 1, 4, 16)
    s = cm.admit("a")
    cm.states[0][s] += 5
    cm.release("a")
    assert cm.admit("b") == s and torch.all(cm.states[0][s] == 0)
