"""The cache manager on the CPU: no page lost, held twice or freed twice, under random orders of
requests; windows give pages back; state slots; all-or-nothing reservations."""
import random

import pytest

from infinilm_b200.cache import CacheManager, CacheStateError, OutOfPages, PagePool, StateSlots
from infinilm_b200.parts.spec import CacheNeed

FULL = CacheNeed("paged_kv", n_kv_heads=2, head_dim=16)
WIN = CacheNeed("paged_kv", n_kv_heads=2, head_dim=16, window=20)
STATE = CacheNeed("state", shape=(4, 8))


def test_page_pool_fifo_and_double_free():
    p = PagePool(3)
    a, b, c = p.alloc(), p.alloc(), p.alloc()
    assert (a, b, c) == (0, 1, 2) and p.n_free == 0
    with pytest.raises(OutOfPages):
        p.alloc()
    p.free(b)
    with pytest.raises(CacheStateError):
        p.free(b)
    with pytest.raises(CacheStateError):
        p.free(7)
    p.free(a)
    assert p.alloc() == b and p.alloc() == a      # first freed, first reused


def test_state_slots_keep_zero_slot():
    s = StateSlots(4)
    got = [s.alloc(), s.alloc(), s.alloc()]
    assert got == [1, 2, 3]
    with pytest.raises(OutOfPages):
        s.alloc()
    with pytest.raises(CacheStateError):
        s.free(0)
    s.free(2)
    with pytest.raises(CacheStateError):
        s.free(2)
    assert s.alloc() == 2


def test_groups_by_need():
    m = CacheManager([FULL, WIN, FULL, None, STATE, WIN], page_size=16, num_pages=8, max_seqs=4)
    assert [g.entries for g in m.groups] == [[0, 2], [1, 5], [4]]
    assert m.group_of_entry == {0: 0, 2: 0, 1: 1, 5: 1, 4: 2}
    assert m.has_state


def test_reserve_commit_close():
    m = CacheManager([FULL], page_size=16, num_pages=6, max_seqs=4)
    a = m.open("a")
    assert a.state_slot == 1 and a.fresh_state
    m.reserve(a, 17)
    assert a.tables[0] == [0, 1]
    m.commit(a, 17)
    assert a.length == 17 and not a.fresh_state
    m.reserve(a, 32)                               # still two pages
    assert a.tables[0] == [0, 1]
    m.reserve(a, 33)
    assert a.tables[0] == [0, 1, 2]
    b = m.open("b")
    assert not m.can_reserve([(b, 16 * 4)])
    with pytest.raises(OutOfPages):
        m.reserve(b, 16 * 4)
    assert b.tables[0] == [] and m.free_pages() == {0: 3}    # nothing was taken
    assert m.can_reserve([(b, 48)]) and not m.can_reserve([(b, 48), (a, 49)])
    m.check_invariants()
    m.close(a)
    with pytest.raises(CacheStateError):
        m.close(a)
    with pytest.raises(CacheStateError):
        m.reserve(a, 40)
    m.reserve(b, 64)
    assert b.tables[0] == [3, 4, 5, 0]             # freed pages come back, in order
    m.close(b)
    m.check_invariants()
    assert m.free_pages() == {0: 6} and not m.live
    with pytest.raises(CacheStateError):
        m.open("c") and m.open("c")


def test_live_request_limit():
    m = CacheManager([FULL], page_size=16, num_pages=6, max_seqs=2)
    m.open(1), m.open(2)
    with pytest.raises(OutOfPages):
        m.open(3)


def test_window_gives_pages_back():
    m = CacheManager([FULL, WIN], page_size=16, num_pages=8, max_seqs=2)
    a = m.open("a")
    m.reserve(a, 50)
    assert a.tables[0] == [0, 1, 2, 3] and a.tables[1] == [0, 1, 2, 3]
    m.commit(a, 50)                                # next query at 50 reads from 31: page 0 is passed
    assert a.tables[0] == [0, 1, 2, 3] and a.tables[1] == [-1, 1, 2, 3]
    assert m.free_pages() == {0: 4, 1: 5}
    for n in range(51, 120):
        m.reserve(a, n)
        m.commit(a, n)
        m.check_invariants()
    live = [p for p in a.tables[1] if p >= 0]
    assert len(live) <= 3 and len(a.tables[1]) == 8 and len(a.tables[0]) == 8
    m.close(a)
    assert m.free_pages() == {0: 8, 1: 8}


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_nothing(seed):
    rng = random.Random(seed)
    needs = [FULL, WIN, FULL] if seed % 2 else [FULL]
    m = CacheManager(needs, page_size=16, num_pages=24, max_seqs=5)
    live = {}
    n_open = 0
    for it in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            n_open += 1
            live[n_open] = m.open(n_open)
        elif op < 0.85 and live:
            k = rng.choice(list(live))
            s = live[k]
            new_len = s.length + rng.choice([1, 1, 1, 2, 7, 16, 40])
            if m.can_reserve([(s, new_len)]):
                m.reserve(s, new_len)
                m.commit(s, new_len)
            else:
                before = {g: list(t) for g, t in s.tables.items()}
                with pytest.raises(OutOfPages):
                    m.reserve(s, new_len)
                assert before == s.tables
        elif live:
            k = rng.choice(list(live))
            m.close(live.pop(k))
        m.check_invariants()
    for s in list(live.values()):
        m.close(s)
    m.check_invariants()
    assert all(f == 24 for f in m.free_pages().values())
    assert m.slots.n_free == 5


@pytest.mark.parametrize("sub", [1, 2, 16])
def test_page_table_array_follows_the_list(sub):
    """The int32 array a step copies from stays in step with the list under every way the list can change: page p
    stands there as the `sub` kernel pages p*sub .. p*sub+sub-1, a page given back as -1s."""
    import random

    import numpy as np

    from infinilm_b200.cache.manager import PageTable
    rng = random.Random(5)
    t = PageTable(sub=sub)
    for step in range(400):
        op = rng.choice(["append"] * 6 + ["set", "set", "clear", "extend", "pop", "slice", "iadd"])
        if op == "append":
            t.append(rng.randrange(1000))
        elif op == "set" and len(t):
            t[rng.randrange(len(t))] = -1
        elif op == "clear" and rng.random() < 0.2:
            t.clear()
        elif op == "extend":
            t.extend([7, 8, 9])
        elif op == "pop" and len(t):
            t.pop()
        elif op == "slice" and len(t) > 2:
            t[0:2] = [-1, -1]
        elif op == "iadd":
            t += [4]
        a = t.array()
        want = [(-1 if p < 0 else p * sub + j) for p in t for j in range(sub)]
        assert a.dtype == np.int32 and a.tolist() == want


@pytest.mark.parametrize("page_size,kernel_page,sub", [(4, 4, 1), (16, 16, 1), (32, 16, 2), (256, 16, 16)])
def test_pages_larger_than_the_kernels_tile_are_runs_of_kernel_pages(page_size, kernel_page, sub):
    m = CacheManager([FULL, WIN], page_size=page_size, num_pages=6, max_seqs=2)
    assert (m.kernel_page, m.sub) == (kernel_page, sub)
    a = m.open("a")
    m.reserve(a, page_size + 1)                    # two pages of each group, whatever their size
    assert a.tables[0] == [0, 1] and m.free_pages() == {0: 4, 1: 4}
    assert a.tables[0].array().tolist() == list(range(2 * sub))
    m.commit(a, page_size + 1)
    b = m.open("b")
    m.reserve(b, 1)
    assert b.tables[0].array().tolist() == list(range(2 * sub, 3 * sub))
    m.close(a), m.close(b)
    m.check_invariants()
    assert m.free_pages() == {0: 6, 1: 6}
