"""The cache manager (no GPU): no page lost, held twice or freed twice under
random orders of requests; windows give pages back; pages are used again;
refusals change nothing. After the reference's random-operation model test
(crates/core/engine/src/blocks/tests.rs:329-892)."""
import random

import pytest

from metallix_b200.csrc import build


@pytest.fixture(scope="module")
def host():
    return build.host()


def make(host, pages=16, page_tokens=4, window=0, requests=4, groups=None):
    groups = groups or [host.GroupConfig(page_tokens, window, pages)]
    return host.CacheManager(groups, requests)


def test_reserve_commit_release(host):
    m = make(host)
    assert m.admit(7) in range(4)
    assert m.cost(7, 9) == [3] and m.cost(99, 4) == [1]
    m.reserve(7, 9)
    assert m.reserved(7) == 9 and m.computed(7) == 0 and len(m.table(7, 0)) == 3
    m.commit(7, 9)
    assert m.cost(7, 3) == [0] and m.cost(7, 4) == [1]
    m.reserve(7, 4)
    m.commit(7, 4)
    assert m.free_pages(0) == 12
    m.check_invariants()
    m.release(7)
    assert m.free_pages(0) == 16 and m.free_slots() == 4 and not m.has(7)
    m.check_invariants()


def test_out_of_pages_changes_nothing(host):
    m = make(host, pages=4)
    m.admit(1)
    m.reserve(1, 12)
    before = (m.table(1, 0), m.free_pages(0), m.reserved(1))
    with pytest.raises(RuntimeError, match="out of cache pages"):
        m.reserve(1, 9)
    assert (m.table(1, 0), m.free_pages(0), m.reserved(1)) == before
    assert not m.fits([(1, 9)]) and m.fits([(1, 4)]) and not m.fits([(1, 4), (55, 1)])
    m.check_invariants()


def test_pages_are_used_again_last_first(host):
    m = make(host, pages=4)
    m.admit(1)
    m.reserve(1, 16)
    first = m.table(1, 0)
    m.commit(1, 16)
    m.release(1)
    m.admit(2)
    m.reserve(2, 8)
    assert set(m.table(2, 0)) <= set(first) and m.pages_reused() == 2
    m.check_invariants()


def test_errors(host):
    m = make(host, requests=1)
    m.admit(1)
    with pytest.raises(ValueError):
        m.admit(1)
    with pytest.raises(RuntimeError):
        m.admit(2)
    with pytest.raises(ValueError):
        m.reserve(3, 1)
    with pytest.raises(ValueError):
        m.commit(1, 1)      # nothing reserved
    with pytest.raises(ValueError):
        m.reserve(1, 0)
    m.release(1)
    with pytest.raises(ValueError):
        m.release(1)        # freed twice


def test_rollback_drops_uncommitted(host):
    m = make(host)
    m.admit(1)
    m.reserve(1, 6)
    m.commit(1, 6)
    m.reserve(1, 9)
    assert m.free_pages(0) == 12
    epoch = m.epoch(1)
    m.rollback(1)
    assert m.reserved(1) == 6 and m.free_pages(0) == 14 and len(m.table(1, 0)) == 2
    assert m.epoch(1) != epoch          # whoever mirrors the longer table must fetch it again
    m.check_invariants()
    m.reserve(1, 1)                     # within the pages it holds: the table does not change
    epoch = m.epoch(1)
    m.rollback(1)
    assert m.epoch(1) == epoch


def test_window_gives_pages_back(host):
    m = make(host, pages=8, page_tokens=4, window=6)
    m.admit(1)
    held = []
    for step in range(40):
        m.reserve(1, 1)
        m.commit(1, 1)
        table = m.table(1, 0)
        computed = m.computed(1)
        # the next query (position computed) sees keys > computed - 6
        first_needed = max(0, computed - 6 + 1)
        for page, physical in enumerate(table):
            if (page + 1) * 4 <= first_needed:
                assert physical == -1, (step, page)
            else:
                assert physical >= 0, (step, page)
        held.append(sum(p >= 0 for p in table))
        m.check_invariants()
    assert max(held) <= 3 and m.pages_reused() > 0   # 40 positions through 8 pages
    assert m.first_live_page(1, 0) == (40 - 6 + 1) // 4


def test_window_release_waits_for_commit(host):
    m = make(host, pages=8, page_tokens=4, window=4)
    m.admit(1)
    m.reserve(1, 20)  # a prompt portion: every query of the portion needs its own window
    assert all(p >= 0 for p in m.table(1, 0))
    m.commit(1, 20)
    assert [p >= 0 for p in m.table(1, 0)] == [False, False, False, False, True]
    m.check_invariants()


def test_groups_have_pages_of_their_own(host):
    m = make(host, groups=[host.GroupConfig(4, 0, 6), host.GroupConfig(4, 5, 3)])
    m.admit(1)
    assert m.cost(1, 10) == [3, 3]
    m.reserve(1, 10)
    m.commit(1, 10)
    assert m.free_pages(0) == 3 and m.free_pages(1) == 1  # keys 6..9 stay visible: pages 1 and 2
    with pytest.raises(RuntimeError, match="group 0"):
        m.reserve(1, 16)
    m.check_invariants()
    m.release(1)
    assert (m.free_pages(0), m.free_pages(1)) == (6, 3)


@pytest.mark.parametrize("seed", range(8))
def test_random_orders(host, seed):
    rng = random.Random(seed)
    windows = [0, rng.choice([0, 3, 7, 16])]
    groups = [host.GroupConfig(rng.choice([1, 2, 4, 8]), w, rng.randint(6, 24)) for w in windows]
    page_tokens = [g.page_tokens for g in groups]
    m = host.CacheManager(groups, 5)
    shadow = {}  # id -> [reserved, computed]
    next_id = 0
    for _ in range(600):
        action = rng.random()
        if action < 0.2 and m.free_slots() > 0:
            m.admit(next_id)
            shadow[next_id] = [0, 0]
            next_id += 1
        elif action < 0.6 and shadow:
            rid = rng.choice(list(shadow))
            count = rng.randint(1, 20)
            if shadow[rid][0] != shadow[rid][1]:
                continue
            if m.fits([(rid, count)]):
                m.reserve(rid, count)
                shadow[rid][0] += count
            else:
                free = [m.free_pages(g) for g in range(2)]
                with pytest.raises(RuntimeError):
                    m.reserve(rid, count)
                assert free == [m.free_pages(g) for g in range(2)]
        elif action < 0.85 and shadow:
            rid = rng.choice(list(shadow))
            pending = shadow[rid][0] - shadow[rid][1]
            if pending:
                if rng.random() < 0.2:
                    m.rollback(rid)
                    shadow[rid][0] = shadow[rid][1]
                else:
                    m.commit(rid, pending)
                    shadow[rid][1] += pending
        elif shadow:
            rid = rng.choice(list(shadow))
            m.release(rid)
            del shadow[rid]
        m.check_invariants()
        held = [0, 0]
        for rid, (reserved, computed) in shadow.items():
            assert (m.reserved(rid), m.computed(rid)) == (reserved, computed)
            for g in range(2):
                table = m.table(rid, g)
                assert len(table) == -(-reserved // page_tokens[g])
                live = [p for p in table if p >= 0]
                held[g] += len(live)
                if windows[g] == 0:
                    assert len(live) == len(table)
                else:  # every position a later query can see is still held
                    first_needed = max(0, computed - windows[g] + 1)
                    for page in range(first_needed // page_tokens[g], len(table)):
                        assert table[page] >= 0
        for g in range(2):
            assert held[g] + m.free_pages(g) == groups[g].num_pages
    for rid in list(shadow):
        m.release(rid)
    m.check_invariants()
    assert [m.free_pages(g) for g in range(2)] == [g.num_pages for g in groups]
