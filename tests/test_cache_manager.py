"""The cache manager on the host: no page lost, held twice or freed twice, under random orders of
requests; windows give pages back; slots."""
import random

import pytest

from transformers_neuronx_b200.cache import (CacheManager, FixedStateNeed, OutOfPages, PagedKVNeed, PagePool,
                                             SlotTable, group_needs)


def manager(num_pages=16, page=16, slots=4, window=None, extra_group_window=None):
    needs = {0: PagedKVNeed(2, 16, window), 1: PagedKVNeed(2, 16, window)}
    if extra_group_window is not None:
        needs[2] = PagedKVNeed(2, 16, extra_group_window)
    needs[7] = FixedStateNeed((4,))
    return CacheManager(group_needs(needs), page, num_pages, slots)


def test_pool_basics():
    p = PagePool(3)
    a = p.alloc(2, "x")
    assert p.num_free == 1 and a == [0, 1]
    with pytest.raises(OutOfPages):
        p.alloc(2, "y")
    assert p.num_free == 1                      # nothing taken by the failed call
    with pytest.raises(ValueError, match="held by"):
        p.free([a[0]], "y")
    p.free(a, "x")
    with pytest.raises(ValueError, match="twice"):
        p.free([a[0]], "x")
    assert p.alloc(1, "z") == [1]               # last freed, first used again
    assert p.reuse_count == 1
    p.check()


def test_groups():
    g = group_needs({0: PagedKVNeed(2, 16), 1: PagedKVNeed(2, 16), 2: PagedKVNeed(2, 16, 32), 3: FixedStateNeed((8,)), 4: None})
    assert [(x.key, x.cache_ids) for x in g] == [(("paged", None), [0, 1]), (("paged", 32), [2]), (("state",), [3])]


def test_append_and_tables():
    m = manager(num_pages=4)
    m.add_request("a")
    assert m.append("a", 17) == 0 and m.block_table("a") == [0, 1]
    assert m.append("a", 15) == 17 and m.block_table("a") == [0, 1]
    assert m.append("a", 1) == 32 and len(m.block_table("a")) == 3
    assert m.slot_of_position("a", 33) == m.block_table("a")[2] * 16 + 1
    m.add_request("b")
    assert m.pages_needed("b", 17) == [2] and not m.can_append("b", 17)
    with pytest.raises(OutOfPages):
        m.append("b", 17)
    assert m.length("b") == 0 and m.free_pages() == [1]       # all or nothing
    m.free_request("a")
    assert m.free_pages() == [4]
    m.append("b", 64)
    m.check()
    with pytest.raises(ValueError):
        m.add_request("b")


def test_window_gives_pages_back():
    m = manager(num_pages=8, window=20)
    m.add_request("a")
    m.append("a", 16); assert m.release_behind_window("a") == 0
    m.append("a", 16); assert m.release_behind_window("a") == 0    # next query (32) reads 13..: page 0 still needed
    m.append("a", 4)                                               # length 36: next query reads 17.. -> page 0 gone
    assert m.release_behind_window("a") == 1 and m.block_table("a")[0] == -1
    with pytest.raises(ValueError, match="window"):
        m.slot_of_position("a", 3)
    used_before = m.pools[0].num_used
    for _ in range(20):
        m.append("a", 16); m.release_behind_window("a")
    assert m.pools[0].num_used <= used_before + 1                  # a window needs a bounded number of pages
    m.check()
    m.free_request("a")
    assert m.free_pages() == [8]


def test_two_groups_have_pools_of_their_own():
    m = manager(num_pages=8, window=None, extra_group_window=16)
    m.add_request("a")
    for _ in range(6):
        m.append("a", 16); m.release_behind_window("a")
    assert m.pools[0].num_used == 6 and m.pools[1].num_used <= 2
    m.check()


def test_slots():
    s = SlotTable(2)
    a, b = s.take("x"), s.take("y")
    assert {a, b} == {0, 1}
    with pytest.raises(OutOfPages):
        s.take("z")
    with pytest.raises(ValueError):
        s.give_back(a, "y")
    s.give_back(a, "x")
    assert s.take("z") == a
    s.check()


@pytest.mark.parametrize("seed", range(8))
def test_random_orders(seed):
    rng = random.Random(seed)
    m = manager(num_pages=12, slots=4, window=[None, 40][seed % 2], extra_group_window=[24, None][seed % 2])
    live, next_id = {}, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 4:
            rid = f"r{next_id}"; next_id += 1
            m.add_request(rid); live[rid] = 0
        elif op < 0.8 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 5, 16, 17, 40])
            if m.can_append(rid, n):
                assert m.append(rid, n) == live[rid]
                live[rid] += n
                m.release_behind_window(rid)
            else:
                before = m.free_pages()
                with pytest.raises(OutOfPages):
                    m.append(rid, n)
                assert m.free_pages() == before and m.length(rid) == live[rid]
        elif live:
            rid = rng.choice(list(live))
            m.free_request(rid); del live[rid]
            with pytest.raises(KeyError):
                m.free_request(rid)
        m.check()
        for rid, n in live.items():            # every position a later query may read has a page
            for gi, g in enumerate(m.paged_groups):
                first = 0 if g.window is None else max(0, n - g.window + 1)
                for pos in range(first, n):
                    assert m.block_table(rid, gi)[pos // 16] >= 0
    for rid in list(live):
        m.free_request(rid)
    assert all(f == 12 for f in m.free_pages()) and m.slots.num_free == 4
    assert any(p.reuse_count > 0 for p in m.pools)


@pytest.mark.parametrize("seed", range(6))
def test_reorder_moves_pages_and_names_the_copies(seed):
    """Beam search's reorder: request i goes on from what request sources[i] holds.  Pages change hands
    without a copy for the first request that names a source; the others get the pages of requests that
    nobody goes on from, with the copies to make.  No page is lost or held twice, sources and
    destinations of copies are disjoint, and after 'copying' every request's pages hold its source's data."""
    rng = random.Random(seed)
    cm = CacheManager(group_needs({0: PagedKVNeed(2, 16), 1: PagedKVNeed(2, 16, window=40)}), 16, 200, 8)
    n = rng.randint(2, 6)
    rids = [f"b{i}" for i in range(n)]
    length = rng.randint(1, 150)
    for r in rids:
        cm.add_request(r)
        cm.append(r, length)
        cm.release_behind_window(r)
    other = "bystander"
    cm.add_request(other); cm.append(other, 33)
    content = {}                      # (group, page) -> whose data it holds
    for i, r in enumerate(rids):
        for g in range(2):
            for p in cm.block_table(r, g):
                if p >= 0:
                    content[(g, p)] = i
    bystander_pages = [list(cm.block_table(other, g)) for g in range(2)]
    for _ in range(4):
        sources = [rng.randrange(n) for _ in range(n)]
        want = {i: None for i in range(n)}
        before = {i: content[(0, next(p for p in cm.block_table(rids[i], 0) if p >= 0))] for i in range(n)}
        copies, slot_copies = cm.reorder(rids, sources)
        cm.check()
        for g in range(2):
            srcs, dsts = {s for s, _ in copies[g]}, {d for _, d in copies[g]}
            assert not (srcs & dsts), "a page is both read and written"
            assert len(dsts) == len(copies[g]), "a page is written twice"
            for s, d in copies[g]:
                content[(g, d)] = content[(g, s)]
        for i, r in enumerate(rids):
            for g in range(2):
                held = [p for p in cm.block_table(r, g) if p >= 0]
                assert held, "the last block is always held"
                assert {content[(g, p)] for p in held} == {before[sources[i]]}, "the request holds its source's data"
        assert sorted(slot_copies) == sorted((cm.slot(rids[s]), cm.slot(rids[i])) for i, s in enumerate(sources) if s != i)
        assert [list(cm.block_table(other, g)) for g in range(2)] == bystander_pages
    free_before = cm.free_pages()
    with pytest.raises(ValueError, match="same number"):
        cm.append(rids[0], 1)
        cm.reorder(rids, list(range(n)))
    for r in rids + [other]:
        cm.free_request(r)
    cm.check()
    assert cm.free_pages() == [200, 200]
