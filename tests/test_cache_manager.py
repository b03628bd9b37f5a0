"""The cache manager on the host: no page lost, held twice or freed twice; groups; windows; slots."""
import random

import pytest

from boring_llm_b200.cache import CacheError, CacheManager, PagedKVSpec, StateSpec

FULL = PagedKVSpec(2, 16, 0)
WIN = PagedKVSpec(2, 16, 20)


def mgr(specs=(FULL, FULL), tokens=128, reqs=4, page=16):
    return CacheManager(list(specs), page, tokens, reqs)


def test_groups_are_formed_by_equal_needs():
    m = mgr([FULL, WIN, FULL, StateSpec((4,)), WIN, None, StateSpec((4,)), StateSpec((2, 3))])
    assert [g.cache_layers for g in m.paged_groups] == [[0, 2], [1, 4]]
    assert [g.cache_layers for g in m.state_groups] == [[3, 6], [7]]
    assert m.layer_location[4] == ("paged", 1, 1) and m.layer_location[7] == ("state", 1, 0)
    assert 5 not in m.layer_location
    assert m.num_pages == 8


def test_reserve_commit_free_and_reuse():
    m = mgr()
    m.add_request("a")
    assert m.reserve("a", 17)                       # two pages
    assert m.get("a").tables == [[0, 1]]
    m.commit("a", 17)
    assert m.reserve("a", 15) and m.get("a").tables == [[0, 1]]      # still inside page 1
    m.commit("a", 15)
    assert m.reserve("a", 1) and m.get("a").tables == [[0, 1, 2]]
    m.commit("a", 1)
    m.add_request("b")
    assert m.reserve("b", 16) and m.get("b").tables == [[3]]
    m.free("a")
    m.check()
    m.add_request("c")
    assert m.reserve("c", 48)
    assert sorted(m.get("c").tables[0]) == [0, 1, 2]                 # a's pages are used again at once
    m.check()


def test_reserve_is_all_or_nothing_and_idempotent_before_commit():
    m = mgr(tokens=64)
    m.add_request("a"); m.add_request("b")
    assert m.reserve("a", 40)                        # 3 of 4 pages
    assert m.reserve("a", 40)                        # asking again takes nothing more
    assert m.free_pages() == [1]
    assert not m.reserve("b", 17)                    # needs 2, 1 free: nothing is taken
    assert m.free_pages() == [1] and m.get("b").tables == [[]]
    assert m.pages_short("b", 17) == 1 and m.can_reserve("b", 16)
    m.check()


def test_two_groups_move_together():
    m = mgr([FULL, WIN], tokens=64)
    m.add_request("a")
    assert m.reserve("a", 33)
    assert [len(t) for t in m.get("a").tables] == [3, 3]
    m.commit("a", 33)
    # window 20: the next query stands at 33 and sees keys 14..33, so page 0 (keys 0..15) is still needed
    assert m.get("a").tables[1] == [m.get("a").tables[1][0], m.get("a").tables[1][1], m.get("a").tables[1][2]]
    assert m.reserve("a", 3); m.commit("a", 3)       # next query at 36 sees 17..36: page 0 is dead
    assert m.get("a").tables[1][0] == -1 and m.get("a").tables[0][0] >= 0
    assert m.free_pages() == [1, 2]
    m.check()
    m.free("a")
    assert m.free_pages() == [4, 4]
    m.check()


def test_window_pages_come_back_and_long_requests_fit_small_pools():
    m = mgr([WIN], tokens=64)                        # 4 pages, window 20
    m.add_request("a")
    for _ in range(40):                              # 400 tokens through a pool of 64
        assert m.reserve("a", 10)
        m.commit("a", 10)
        m.check()
    live = [p for p in m.get("a").tables[0] if p >= 0]
    assert len(live) <= 3
    m.free("a"); m.check()
    assert m.free_pages() == [4]


def test_slots_and_state():
    zeroed = []
    m = CacheManager([StateSpec((3,)), FULL], 16, 64, 2, on_slot_assigned=zeroed.append)
    a = m.add_request("a"); b = m.add_request("b")
    assert {a.slot, b.slot} == {0, 1} and zeroed == [a.slot, b.slot]
    assert not m.has_free_slot()
    with pytest.raises(CacheError, match="slot"):
        m.add_request("c")
    m.free("a")
    c = m.add_request("c")
    assert c.slot == a.slot and zeroed[-1] == a.slot
    m.check()


def test_misuse_is_reported():
    m = mgr()
    with pytest.raises(CacheError, match="not live"):
        m.reserve("nobody", 1)
    m.add_request("a")
    with pytest.raises(CacheError, match="already live"):
        m.add_request("a")
    with pytest.raises(CacheError, match="past its reserved"):
        m.commit("a", 5)
    m.reserve("a", 5); m.commit("a", 5)
    m.free("a")
    with pytest.raises(CacheError, match="not live"):
        m.free("a")
    p = m.paged_groups[0].pool
    page = p.take("x")
    p.give_back(page, "x")
    with pytest.raises(CacheError, match="freed twice"):
        p.give_back(page, "x")
    page = p.take("x")
    with pytest.raises(CacheError, match="owned by"):
        p.give_back(page, "y")


def test_truncate_keeps_a_prefix():
    m = mgr()
    m.add_request("a")
    m.reserve("a", 50); m.commit("a", 50)
    m.truncate("a", 17)
    assert len(m.get("a").tables[0]) == 2 and m.get("a").num_tokens == 17
    m.check()
    w = mgr([WIN])
    w.add_request("a")
    w.reserve("a", 60); w.commit("a", 60)
    with pytest.raises(CacheError, match="window"):
        w.truncate("a", 30)


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_never_lose_or_double_a_page(seed):
    rng = random.Random(seed)
    specs = [FULL, WIN, FULL, StateSpec((2,))] if seed % 2 else [FULL]
    m = CacheManager(specs, 16, 256, 5)
    live, counter = {}, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and m.has_free_slot():
            rid = f"r{counter}"; counter += 1
            m.add_request(rid); live[rid] = 0
        elif op < 0.8 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 7, 16, 33])
            before = m.free_pages()
            if m.reserve(rid, n):
                m.commit(rid, n); live[rid] += n
                assert m.get(rid).num_tokens == live[rid]
            else:
                assert m.free_pages() == before
        elif live:
            rid = rng.choice(list(live))
            m.free(rid); del live[rid]
        m.check()
        for gi, g in enumerate(m.paged_groups):
            held = sum(1 for rid in live for p in m.get(rid).tables[gi] if p >= 0)
            assert held + g.pool.num_free == m.num_pages
    for rid in list(live):
        m.free(rid)
    m.check()
    assert m.free_pages() == [m.num_pages] * len(m.paged_groups)


def test_table_version_names_one_state_of_the_block_tables():
    """(uid, version) changes exactly when a block table does; a request id used again gets a new uid."""
    m = CacheManager([PagedKVSpec(1, 16, 0), PagedKVSpec(1, 16, 8)], page_size=4, capacity_tokens=64, max_requests=2)
    a = m.add_request("a")
    seen = {}

    def check():
        key = (a.uid, a.version)
        state = tuple(tuple(t) for t in a.tables)
        assert seen.setdefault(key, state) == state, "one name, two states"
        return key

    k0 = check()
    assert m.reserve("a", 3)
    k1 = check()
    assert k1 != k0
    m.commit("a", 3)
    assert check() == k1                          # no page came or went
    for _ in range(20):                           # token by token: new pages, and pages the window has passed
        before = tuple(tuple(t) for t in a.tables)
        kb = check()
        assert m.reserve("a", 1)
        m.commit("a", 1)
        after = tuple(tuple(t) for t in a.tables)
        assert (check() == kb) == (after == before)
    m.free("a")
    b = m.add_request("a")
    assert b.uid != a.uid
    assert m.find("a") is b and m.find("zz") is None
    full = CacheManager([PagedKVSpec(1, 16, 0)], page_size=4, capacity_tokens=64, max_requests=1)
    c = full.add_request("c")
    assert full.reserve("c", 10)
    full.commit("c", 10)
    v = c.version
    full.truncate("c", 9)                         # still three pages
    assert c.version == v
    full.truncate("c", 3)                         # two pages go back
    assert c.version != v and len(c.tables[0]) == 1
