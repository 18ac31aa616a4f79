"""The cache manager's bookkeeping, on the CPU (restates
crates/ai-engine-candle/src/paged/block_table.rs:61-117 and adds groups, windows,
slots and random orders of requests)."""
import numpy as np
import pytest

from ai_engine_b200.cache import PagedCache, host
from ai_engine_b200.parts import KVRequest, StateRequest


def manager(groups, max_seqs=4, max_pages=64):
    h = host()
    return h.CacheManager([h.GroupSpec(p, n, w) for p, n, w in groups], max_seqs, max_pages)


def test_pages_round_up_low_ids_first_and_are_used_again():
    c = manager([(16, 4, 0)])
    s = c.admit()
    assert c.ensure(s, 1) and c.pages(0, s) == [0]
    assert c.ensure(s, 16) and c.pages(0, s) == [0]
    assert c.ensure(s, 17) and c.pages(0, s) == [0, 1]
    assert c.free_pages(0) == 2
    c.finish(s)
    assert c.free_pages(0) == 4
    s2 = c.admit()
    assert c.ensure(s2, 40) and sorted(c.pages(0, s2)) == [0, 1, 2] and c.free_pages(0) == 1
    c.check_invariants()


def test_all_or_nothing_when_pages_run_out():
    c = manager([(16, 2, 0)])
    s = c.admit()
    assert not c.ensure(s, 48)
    assert c.pages(0, s) == [] and c.free_pages(0) == 2
    assert c.tokens_that_fit(s, 48) == 32
    c.check_invariants()


def test_all_or_nothing_across_groups():
    c = manager([(16, 8, 0), (8, 2, 0)])
    s = c.admit()
    assert not c.ensure(s, 24)          # group 1 would need 3 pages of 2
    assert c.pages(0, s) == [] and c.pages(1, s) == []
    assert c.ensure(s, 16) and len(c.pages(0, s)) == 1 and len(c.pages(1, s)) == 2
    c.check_invariants()


def test_window_gives_pages_back_and_they_are_used_again():
    c = manager([(8, 6, 20)])
    s = c.admit()
    assert c.ensure(s, 40)              # 5 pages during a 40-token portion
    assert c.advance(s, 40) == 2        # first key still read: 40 - 20 + 1 = 21 -> pages 0, 1 go
    assert c.pages(0, s)[:2] == [-1, -1] and c.first_live(0, s) == 2 and c.free_pages(0) == 3
    for n in range(41, 200):
        assert c.ensure(s, n), n        # never more than ceil(20/8) + 2 pages held
        c.advance(s, n)
        assert c.pages_in_use(0) <= 4
        c.check_invariants()
    assert c.total_allocations(0) > 6
    c.finish(s)
    assert c.free_pages(0) == 6


def test_double_free_and_dead_slot_are_errors():
    h = host()
    p = h.PagePool(3)
    a = p.alloc(2)
    p.release(a[0])
    with pytest.raises(Exception, match="freed twice"):
        p.release(a[0])
    with pytest.raises(Exception, match="outside the pool"):
        p.release(9)
    assert p.alloc(5) is None and p.free_count == 2
    c = manager([(16, 4, 0)])
    s = c.admit()
    c.finish(s)
    with pytest.raises(Exception, match="not live"):
        c.ensure(s, 1)
    with pytest.raises(Exception, match="not live"):
        c.finish(s)


def test_slots_run_out_and_come_back():
    c = manager([(16, 64, 0)], max_seqs=3)
    slots = [c.admit() for _ in range(3)]
    assert sorted(slots) == [0, 1, 2] and c.admit() == -1
    c.finish(slots[1])
    assert c.admit() == slots[1]


def test_block_table_rows_for_a_batch():
    c = manager([(4, 16, 0)])
    a, b = c.admit(), c.admit()
    c.ensure(a, 9)
    c.ensure(b, 3)
    out = np.zeros((2, 4), dtype=np.int32)
    c.fill_block_table(0, [b, a], 4, out)
    assert out.tolist() == [[c.pages(0, b)[0], -1, -1, -1], c.pages(0, a) + [-1]]


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_nothing(seed):
    """Requests grow, finish and are replaced in random order, in two groups (all keys
    and a window); after every operation no page is lost, held twice or freed twice."""
    rng = np.random.RandomState(seed)
    c = manager([(8, 24, 0), (4, 30, 10)], max_seqs=5, max_pages=40)
    live = {}
    for _ in range(600):
        op = rng.rand()
        if op < 0.25 and c.free_slots:
            live[c.admit()] = 0
        elif op < 0.85 and live:
            s = list(live)[rng.randint(len(live))]
            grow = int(rng.choice([1, 1, 1, 2, 5, 17]))
            if c.ensure(s, live[s] + grow):
                live[s] += grow
                c.advance(s, live[s])
            else:
                before = (c.free_pages(0), c.free_pages(1))
                assert before == (c.free_pages(0), c.free_pages(1))   # nothing was taken
        elif live:
            s = list(live)[rng.randint(len(live))]
            c.finish(s)
            del live[s]
        c.check_invariants()
        for s, n in live.items():
            assert len(c.pages(0, s)) == (n + 7) // 8
            assert sum(p >= 0 for p in c.pages(1, s)) <= (10 + 4 - 1) // 4 + 1 + (17 + 3) // 4
    for s in list(live):
        c.finish(s)
    assert c.free_pages(0) == 24 and c.free_pages(1) == 30 and c.free_slots == 5


def test_groups_by_what_parts_ask_for():
    """Parts with the same need share a group; a window or another head size makes a group of its
    own; an entry that reads another's cache gets that one's place; two parts of one entry (two
    roles) have a cache each."""
    from ai_engine_b200.parts import CacheNeed

    full, win = KVRequest(2, 16, 0), KVRequest(2, 16, 32)
    reqs = [CacheNeed(0, "mixer", full), CacheNeed(1, "mixer", win), CacheNeed(2, "mixer", full),
            CacheNeed(2, "side", win, StateRequest((3,))), CacheNeed(3, "mixer", None, StateRequest((4,))),
            CacheNeed(4, "mixer", None, None, 1)]
    c = PagedCache(reqs, page_size=8, num_pages=10, max_seqs=2, max_seq_len=64, dtype=None, allocate=False)
    assert len(c.groups) == 2
    assert c.groups[0].entries == [(0, "mixer"), (2, "mixer")] and c.groups[1].entries == [(1, "mixer"), (2, "side")]
    assert c.where[4, "mixer"] == c.where[1, "mixer"] and (3, "mixer") not in c.where
    assert c.writes[1, "mixer"] and not c.writes[4, "mixer"]
    assert c.roles[2] == ["mixer", "side"]
    assert c.book.group(1).window == 32
    with pytest.raises(ValueError):
        PagedCache([CacheNeed(1, "mixer", None, None, 0)], 8, 10, 2, 64, None, allocate=False)
