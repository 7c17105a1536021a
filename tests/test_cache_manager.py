"""The cache manager (no GPU): no page lost, held twice or freed twice under
random orders of requests; windows give pages back; pages are used again;
refusals change nothing; forked requests share pages and never see each
other's writes. After the reference's random-operation model test
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


def test_fork_shares_full_pages_and_copies_the_partial_one(host):
    m = make(host, pages=8, page_tokens=4)
    m.admit(1)
    m.reserve(1, 10)
    with pytest.raises(ValueError, match="uncommitted"):
        m.fork(1, 2)
    m.commit(1, 10)
    parent = m.table(1, 0)
    source_slot, target_slot, copies = m.fork(1, 2)
    child = m.table(2, 0)
    assert (source_slot, target_slot) == (m.slot(1), m.slot(2)) and source_slot != target_slot
    assert child[:2] == parent[:2] and child[2] != parent[2] and copies == [(0, parent[2], child[2])]
    assert [m.references(0, p) for p in parent] == [2, 2, 1] and m.references(0, child[2]) == 1
    assert m.computed(2) == m.reserved(2) == 10 and m.free_pages(0) == 4
    m.check_invariants()
    with pytest.raises(ValueError, match="already live"):
        m.fork(1, 2)
    m.release(1)                       # the shared pages stay with the child
    assert m.free_pages(0) == 5 and [m.references(0, p) for p in child] == [1, 1, 1]
    m.check_invariants()
    m.reserve(2, 7)
    m.commit(2, 7)
    m.release(2)
    assert m.free_pages(0) == 8
    m.check_invariants()


def test_fork_at_a_page_edge_copies_nothing_and_a_refused_fork_changes_nothing(host):
    m = make(host, pages=3, page_tokens=4, requests=3)
    m.admit(1)
    m.reserve(1, 8)
    m.commit(1, 8)
    assert m.fork(1, 2)[2] == [] and m.table(2, 0) == m.table(1, 0) and m.free_pages(0) == 1
    m.reserve(1, 2)
    m.commit(1, 2)                      # the parent takes the last page: a partial one
    with pytest.raises(RuntimeError, match="out of cache pages"):
        m.fork(1, 3)
    assert not m.has(3) and m.free_slots() == 1 and m.free_pages(0) == 0
    m.check_invariants()
    m.release(2)
    assert m.free_pages(0) == 0         # both pages are still the parent's
    m.release(1)
    assert m.free_pages(0) == 3
    m.check_invariants()


def test_fork_under_a_window_shares_only_live_pages(host):
    m = make(host, pages=8, page_tokens=4, window=6)
    m.admit(1)
    for _ in range(5):
        m.reserve(1, 3)
        m.commit(1, 3)                  # 15 positions: pages 0 and 1 are behind the window
    parent = m.table(1, 0)
    assert parent[:2] == [-1, -1]
    _, _, copies = m.fork(1, 2)
    child = m.table(2, 0)
    assert child[:3] == parent[:3] and copies == [(0, parent[3], child[3])]
    m.reserve(2, 8)
    m.commit(2, 8)                      # the child's window passes the shared page
    assert m.table(2, 0)[2] == -1 and m.references(0, parent[2]) == 1
    m.check_invariants()
    m.release(1)
    m.release(2)
    assert m.free_pages(0) == 8


@pytest.mark.parametrize("seed", range(12))
def test_random_orders(host, seed):
    """Random admissions, reservations, commits, rollbacks, forks and releases
    against a shadow: what each request wrote at each position (a number of its
    own) must still be what its table leads to, whoever else shares the page."""
    rng = random.Random(seed)
    windows = [0, rng.choice([0, 3, 7, 16])]
    groups = [host.GroupConfig(rng.choice([1, 2, 4, 8]), w, rng.randint(6, 24)) for w in windows]
    page_tokens = [g.page_tokens for g in groups]
    m = host.CacheManager(groups, 5)
    shadow = {}   # id -> [reserved, computed]
    wrote = {}    # id -> the value at each position of the request
    pages = [dict(), dict()]   # group -> (page, offset) -> value: the device memory
    next_id, stamp = 0, 0
    for _ in range(700):
        action = rng.random()
        if action < 0.15 and m.free_slots() > 0:
            m.admit(next_id)
            shadow[next_id], wrote[next_id] = [0, 0], []
            next_id += 1
        elif action < 0.25 and shadow and m.free_slots() > 0:
            parent = rng.choice(list(shadow))
            if shadow[parent][0] != shadow[parent][1]:
                continue
            free = [m.free_pages(g) for g in range(2)]
            try:
                _, _, copies = m.fork(parent, next_id)
            except RuntimeError:
                assert free == [m.free_pages(g) for g in range(2)] and not m.has(next_id)
                continue
            for g, source, target in copies:
                for offset in range(page_tokens[g]):
                    if (source, offset) in pages[g]:
                        pages[g][(target, offset)] = pages[g][(source, offset)]
            shadow[next_id], wrote[next_id] = list(shadow[parent]), list(wrote[parent])
            next_id += 1
        elif action < 0.6 and shadow:
            rid = rng.choice(list(shadow))
            count = rng.randint(1, 20)
            if shadow[rid][0] != shadow[rid][1]:
                continue
            if m.fits([(rid, count)]):
                m.reserve(rid, count)
                for position in range(shadow[rid][0], shadow[rid][0] + count):   # the step writes
                    stamp += 1
                    del wrote[rid][position:]
                    wrote[rid].append(stamp)
                    for g in range(2):
                        page = m.table(rid, g)[position // page_tokens[g]]
                        assert page >= 0 and m.references(g, page) == 1   # never into a shared page
                        pages[g][(page, position % page_tokens[g])] = stamp
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
            del shadow[rid], wrote[rid]
        m.check_invariants()
        held = [set(), set()]
        for rid, (reserved, computed) in shadow.items():
            assert (m.reserved(rid), m.computed(rid)) == (reserved, computed)
            for g in range(2):
                table = m.table(rid, g)
                assert len(table) == -(-reserved // page_tokens[g])
                live = [p for p in table if p >= 0]
                held[g].update(live)
                first_needed = 0 if windows[g] == 0 else max(0, computed - windows[g] + 1)
                if windows[g] == 0:
                    assert len(live) == len(table)
                else:  # every position a later query can see is still held
                    for page in range(first_needed // page_tokens[g], len(table)):
                        assert table[page] >= 0
                for position in range(first_needed, computed):
                    where = (table[position // page_tokens[g]], position % page_tokens[g])
                    assert pages[g][where] == wrote[rid][position], (rid, g, position)
        for g in range(2):
            assert len(held[g]) + m.free_pages(g) == groups[g].num_pages
    for rid in list(shadow):
        m.release(rid)
    m.check_invariants()
    assert [m.free_pages(g) for g in range(2)] == [g.num_pages for g in groups]
