"""The cache manager: no page lost, held twice or freed twice, under random orders of requests."""
import random

import pytest

from leone_b200.cache.pages import CacheError, CacheManager, GroupSpec, OutOfPages, PagePool, StateSlots


def _manager(pages=16, page_tokens=4, slots=4, window=None):
    groups = [GroupSpec("full", 2, 16)]
    if window:
        groups.append(GroupSpec("window", 1, 8, window))
    return CacheManager(groups, page_tokens, pages, slots)


def test_pool_take_and_give_back():
    pool = PagePool(4)
    pages = pool.take(3)
    assert len(set(pages)) == 3 and pool.num_free == 1
    with pytest.raises(OutOfPages):
        pool.take(2)
    assert pool.num_free == 1                     # a refused take takes nothing
    pool.give_back(pages[:1])
    with pytest.raises(CacheError):
        pool.give_back(pages[:1])                 # freed twice
    with pytest.raises(CacheError):
        pool.give_back([99])
    assert pool.take(1) == pages[:1]              # the page just freed is used again first


def test_slots():
    slots = StateSlots(2)
    a, b = slots.take(), slots.take()
    assert {a, b} == {0, 1}
    with pytest.raises(OutOfPages):
        slots.take()
    slots.give_back(a)
    with pytest.raises(CacheError):
        slots.give_back(a)
    assert slots.take() == a


def test_reserve_commit_rollback_close():
    m = _manager()
    m.open("a")
    m.reserve({"a": 9})                           # 3 pages of 4 tokens
    assert m.free_pages() == [13] and m.length("a") == 0
    m.commit("a", 9)
    m.reserve({"a": 13})
    m.rollback("a")                               # the failed step's page goes back
    assert m.free_pages() == [13] and m.length("a") == 9
    with pytest.raises(CacheError):
        m.commit("a", 20)                         # more than was reserved
    table = m.block_table(0, ["a"])
    assert table.shape == (1, 3) and (table >= 0).all()
    m.close("a")
    assert m.free_pages() == [16]
    with pytest.raises(CacheError):
        m.close("a")
    m.check_invariants()


def test_reserve_is_all_or_nothing_across_requests():
    m = _manager(pages=5)
    m.open("a"), m.open("b")
    with pytest.raises(OutOfPages):
        m.reserve({"a": 12, "b": 12})             # 3 + 3 pages > 5
    assert m.free_pages() == [5]
    assert m.can_reserve({"a": 12, "b": 8})
    m.reserve({"a": 12, "b": 8})
    assert m.free_pages() == [0]
    m.check_invariants()


def test_truncate():
    m = _manager()
    m.open("a")
    m.reserve({"a": 14}), m.commit("a", 14)
    m.truncate("a", 5)
    assert m.length("a") == 5 and m.free_pages() == [14]
    with pytest.raises(CacheError):
        m.truncate("a", 6)


def test_a_rewind_into_what_a_window_has_released_is_refused():
    """Pages that a window has passed are gone; a query at a shorter length would read them."""
    m = _manager(pages=16, page_tokens=4, window=6)
    m.open("a")
    m.reserve({"a": 30}), m.commit("a", 30)                 # blocks before position 24 are released
    free = m.free_pages()
    table = list(m.groups[0].tables["a"])
    with pytest.raises(CacheError, match="released"):
        m.truncate("a", 20)                                 # needs keys from position 15: block 3 is gone
    assert m.length("a") == 30 and m.free_pages() == free and m.groups[0].tables["a"] == table
    m.truncate("a", 29)                                     # needs keys from 24: still there
    assert m.length("a") == 29
    m.rollback("a")                                         # a rollback never goes below the committed length
    m.check_invariants()


def test_table_version_changes_only_when_a_table_does_not_just_grow():
    m = _manager(pages=16, page_tokens=4)
    m.open("a")
    v0 = m.table_version("a")
    m.reserve({"a": 9})
    m.commit("a", 9)
    m.reserve({"a": 17})
    m.commit("a", 17)
    assert m.table_version("a") == v0                      # growing at the end
    m.reserve({"a": 30})
    m.rollback("a")                                         # pages past the committed length go back
    v1 = m.table_version("a")
    assert v1 != v0
    m.truncate("a", 17)                                     # nothing dropped
    assert m.table_version("a") == v1
    m.truncate("a", 3)
    assert m.table_version("a") != v1
    m.close("a")
    m.open("a")
    assert m.table_version("a") not in (v0, v1)             # a new life of the same name
    w = _manager(pages=16, page_tokens=4, window=6)
    w.open("b")
    vb = w.table_version("b")
    w.reserve({"b": 20})
    w.commit("b", 20)                                       # the window has passed whole pages
    assert w.table_version("b") != vb


def test_window_group_gives_pages_back_as_the_window_passes():
    m = _manager(pages=8, page_tokens=4, window=6)
    m.open("a")
    m.reserve({"a": 20}), m.commit("a", 20)
    full, win = m.groups
    assert full.pool.num_held == 5
    # the next query is at position 20 and reads keys 15..20: blocks 0..2 (keys 0..11) are passed
    assert win.tables["a"][:3] == [-1, -1, -1] and win.pool.num_held == 2
    row = m.block_table(1, ["a"])[0]
    assert list(row[:3]) == [-1, -1, -1] and (row[3:5] >= 0).all()
    m.reserve({"a": 24}), m.commit("a", 24)
    assert win.pool.num_held == 2                 # one taken, one passed
    m.close("a")
    assert m.free_pages() == [8, 8]
    m.check_invariants()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_never_lose_or_share_a_page(seed):
    rng = random.Random(seed)
    m = _manager(pages=24, page_tokens=4, slots=5, window=7 if seed % 2 else None)
    live, counter = {}, 0
    for _ in range(400):
        action = rng.random()
        if action < 0.25 and len(live) < 5:
            rid = f"r{counter}"
            counter += 1
            m.open(rid)
            live[rid] = 0
        elif action < 0.75 and live:
            picked = rng.sample(sorted(live), rng.randint(1, len(live)))
            wants = {r: live[r] + rng.randint(1, 9) for r in picked}
            try:
                m.reserve(wants)
            except OutOfPages:
                before = m.free_pages()
                assert before == m.free_pages()
            else:
                if rng.random() < 0.15:            # the step failed
                    for r in picked:
                        m.rollback(r)
                else:
                    for r, n in wants.items():
                        m.commit(r, n)
                        live[r] = n
        elif live:
            rid = rng.choice(sorted(live))
            m.close(rid)
            del live[rid]
        m.check_invariants()
        for rid, n in live.items():
            assert m.length(rid) == n
            for g in m.groups:
                table = g.tables[rid]
                for b in range(g.first_live_block(n), g.blocks_for(n)):
                    assert table[b] >= 0          # every block a query can still read has a page
    for rid in list(live):
        m.close(rid)
    assert all(f == 24 for f in m.free_pages())
    m.check_invariants()


def _same_error(native_call, plain_call):
    """Both raise the same kind of error, or neither raises."""
    from tests.plain import cache_model as plain
    kinds = []
    for call, errors in ((native_call, (OutOfPages, CacheError)), (plain_call, (plain.OutOfPages, plain.CacheError))):
        try:
            call()
            kinds.append(None)
        except errors as exc:
            kinds.append(type(exc).__name__)
    assert kinds[0] == kinds[1], kinds
    return kinds[0]


@pytest.mark.parametrize("seed", range(8))
def test_the_native_manager_and_the_plain_model_agree_call_by_call(seed):
    """The same random calls, rule-breaking ones among them, go to the C++ manager and to the
    Python model under tests/plain: same errors, same tables, lengths, slots, versions, counts."""
    from tests.plain import cache_model as plain
    rng = random.Random(1000 + seed)
    window = [None, 7, 5, 12][seed % 4]
    page_tokens = [4, 3, 8, 5][seed % 4]
    pages, slots = 20 + seed, 4

    def specs(mod):
        out = [mod.GroupSpec("full", 2, 16, None, [0])]
        if window:
            out.append(mod.GroupSpec("window", 2, 16, window, [1]))
        return out

    a = CacheManager(specs(__import__("leone_b200.cache.pages", fromlist=["x"])), page_tokens, pages, slots)
    b = plain.CacheManager(specs(plain), page_tokens, pages, slots)
    live, counter = {}, 0
    for _ in range(500):
        action = rng.random()
        if action < 0.2:
            rid = f"r{counter}" if rng.random() < 0.9 or not live else rng.choice(sorted(live))
            counter += 1
            if _same_error(lambda: a.open(rid), lambda: b.open(rid)) is None:
                live[rid] = 0
                assert a.slot(rid) == b.slot(rid)
        elif action < 0.7 and live:
            picked = rng.sample(sorted(live), rng.randint(1, len(live)))
            wants = {r: live[r] + rng.randint(-1 if rng.random() < 0.05 else 1, 11) for r in picked}
            assert a.can_reserve(wants) == b.can_reserve(wants)
            if _same_error(lambda: a.reserve(wants), lambda: b.reserve(wants)) is None:
                if rng.random() < 0.15:
                    for r in picked:
                        a.rollback(r)
                        b.rollback(r)
                else:
                    for r, n in wants.items():
                        n = n - (1 if rng.random() < 0.1 and n > live[r] + 1 else 0)    # fewer than reserved
                        if _same_error(lambda: a.commit(r, n), lambda: b.commit(r, n)) is None:
                            live[r] = n
        elif action < 0.75 and live:
            # the decode loop's calls: several requests, the same number of steps, one call each way
            picked = rng.sample(sorted(live), rng.randint(1, len(live)))
            steps = rng.randint(1, 6)
            got = []
            kind = _same_error(lambda: got.append(a.reserve_steps(picked, steps)),
                               lambda: b.reserve({r: live[r] + steps for r in picked}))
            if kind is None:
                lengths, versions, slots, table_lens = got[0]
                assert lengths.tolist() == [live[r] for r in picked]
                assert versions.tolist() == [b.table_version(r) for r in picked]
                assert slots.tolist() == [b.slot(r) for r in picked]
                for gi, gb in enumerate(b.groups):
                    assert table_lens[gi].tolist() == [len(gb.tables[r]) for r in picked]
                a.commit_many(picked, [live[r] + steps for r in picked])
                for r in picked:
                    b.commit(r, live[r] + steps)
                    live[r] += steps
        elif action < 0.8 and live:
            rid = rng.choice(sorted(live))
            to = rng.randint(0, live[rid] + 2)
            if _same_error(lambda: a.truncate(rid, to), lambda: b.truncate(rid, to)) is None:
                live[rid] = min(live[rid], to)
        elif action < 0.95 and live:
            rid = rng.choice(sorted(live))
            a.close(rid)
            b.close(rid)
            del live[rid]
        else:
            _same_error(lambda: a.close("nobody"), lambda: b.close("nobody"))
        a.check_invariants()
        b.check_invariants()
        assert a.free_pages() == b.free_pages()
        assert a.slots.num_free == b.slots.num_free
        for rid, n in live.items():
            assert a.length(rid) == b.length(rid) == n
            assert a.table_version(rid) == b.table_version(rid)
            for ga, gb in zip(a.groups, b.groups):
                assert ga.tables[rid] == gb.tables[rid]
                assert ga.first_live_block(n) == gb.first_live_block(n)
        if live:
            rids = sorted(live)
            for ga in a.groups:
                assert (a.block_table(ga.gid, rids) == b.block_table(ga.gid, rids)).all()
    assert [g.pool.high_water for g in a.groups] == [g.pool.high_water for g in b.groups]
