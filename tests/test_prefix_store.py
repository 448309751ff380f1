"""The prefix KV store's host side (ling_b200_prefix_*, ling_b200_arena_*): the reference's PrefixKvTree in paged mode and
its ArenaAlloc (src/core/prefix_kv.hpp) restated.  Checked against traces recorded from the reference's own code
(tests/golden/prefix_kv.json), live against that code where it is built, and on the known answers of the reference's own
paged-mode tests (tests/prefix_kv_tests.cpp:144-300), restated here."""
import ctypes as C
import json
import os

import pytest

import prefix_trace as pt
from golden.make_golden_prefix import STATE, arena_trace
from oracle import lo

GOLDEN = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "prefix_kv.json")))


def host(lb, states=2, pages=400):
    return pt.Host(lb.lib(), False, pages, states * STATE, STATE)


@pytest.mark.parametrize("case", GOLDEN["tree"], ids=lambda c: "seed%d" % c["seed"])
def test_tree_replays_the_reference_traces(lb, case):
    h = host(lb, case["states"])
    log = pt.random_sessions(h, case["seed"], case["steps"], STATE)
    h.close()
    for i, (got, want) in enumerate(zip(log, case["log"])):
        assert got == want, "step %d" % i
    assert len(log) == len(case["log"])
    assert sum(r["n"] for r in log[:-2]) > 5000  # the trace restores from the store for real


@pytest.mark.parametrize("case", GOLDEN["arena"], ids=lambda c: "seed%d" % c["seed"])
def test_arena_replays_the_reference_traces(lb, case):
    assert arena_trace(lb.lib(), "ling_b200_arena_", case) == case["log"]


@pytest.mark.skipif(lo.ref() is None, reason="the reference's host code is not built here")
@pytest.mark.parametrize("seed,states", [(101, 64), (202, 3), (303, 1)])
def test_tree_equals_the_reference_live(lb, seed, states):
    a, b = host(lb, states), pt.Host(lo.ref(), True, 400, states * STATE, STATE)
    assert pt.random_sessions(a, seed, 300, STATE) == pt.random_sessions(b, seed, 300, STATE)
    a.close(), b.close()
    case = {"seed": seed, "size": 1 << 18, "align": 128, "steps": 300}
    assert arena_trace(lb.lib(), "ling_b200_arena_", case) == arena_trace(lo.ref(), "ref_arena_", case)


def test_insert_split_and_evict_count_page_references(lb):
    h = host(lb)
    a = pt.family_prompt([], 1, 150)
    h.run(a, [], 0)
    ta = list(h.table)
    h.insert(a, 150, [], 1)
    assert h.counters()[:4] == [1, 0, 3, 0]
    m = h.match(a)
    assert m[0] == 150 and h.pages(m, 150) == ta and h.pages(m, 64) == ta[:1]
    assert [h.refs(p) for p in ta] == [2, 2, 2]
    h.insert(a, 150, [90], 2)  # a split inside page 1: both halves hold it
    assert h.counters()[0] == 2 and [h.refs(p) for p in ta] == [2, 3, 2]
    assert h.pages(h.match(a), 150) == ta
    h.insert(a, 150, [128], 3)  # a split on a page boundary shares nothing
    assert h.counters()[0] == 3 and [h.refs(p) for p in ta] == [2, 3, 2] and h.counters()[2] == 4
    assert h.evict_lru_leaf() == 1  # [128, 150)
    assert h.counters()[0] == 2 and h.refs(ta[2]) == 1
    assert h.evict_lru_leaf() == 1 and h.evict_lru_leaf() == 1 and h.evict_lru_leaf() == 0
    assert [h.refs(p) for p in ta] == [1, 1, 1] and h.counters()[:3] == [0, 0, 0]
    h.end_session()
    assert h.live_pages() == 0
    h.close()


def test_prompts_diverging_inside_a_page_get_their_own_copy(lb):
    h = host(lb, 0)
    a, b = pt.family_prompt(range(100), 1, 60), pt.family_prompt(range(100), 2, 60)
    h.run(a, [], 0)
    h.insert(a, 160, [], 1)
    mb = h.match(b)
    assert mb[0] == 100
    h.run(b, h.pages(mb, 100), 100)  # shares page 0, copies page 1 before writing it
    h.insert(b, 160, [], 2)
    assert h.counters()[0] == 3
    for p in (a, b):
        m = h.match(p)
        assert m[0] == 160
        pg = h.pages(m, 160)
        assert all(h.mem[pg[pos // pt.PT]][pos % pt.PT] == pt.kv_at(p, pos) for pos in range(160))
    pa, pb = h.pages(h.match(a), 160), h.pages(h.match(b), 160)
    assert pa[0] == pb[0] and pa[1] != pb[1]
    h.end_session()
    h.clear()
    assert h.live_pages() == 0 and h.counters()[2] == 0
    h.close()


def test_the_budget_holds_states_only(lb):
    h = host(lb, 2)
    a = pt.family_prompt([], 3, 300)
    h.run(a, [], 0)
    want = h.insert(a, 300, [100, 200, 300], 1)
    assert h.counters()[0] == 3 and h.counters()[3] == 0 and [w[1] for w in want] == [100, 200, 300]
    assert h.add_state(want[0][0], 1) and h.add_state(want[1][0], 1) and not h.add_state(want[2][0], 1)
    assert h.counters()[3] == 2 * STATE and h.counters()[1] == 2
    assert not h.add_state(want[0][0], 1)  # it has one
    m = h.match(a)
    assert h.best_state(m, 300)[0] == 200 and h.best_state(m, 199)[0] == 100 and h.best_state(m, 99)[0] == 0
    assert h.best_state((150, m[1]), 300)[0] == 100  # a state past the matched length does not count
    # a later prefill's state makes room by evicting the least recently used leaf stamped before it
    b = pt.family_prompt([], 4, 80)
    h.run(b, [], 0)
    wb = h.insert(b, 80, [80], 2)
    # ([200, 300) has no state and goes first without freeing a byte, then [100, 200) with its state)
    assert h.add_state(wb[0][0], 2) and h.counters()[0] == 2 and h.match(a)[0] == 100 and h.counters()[1] == 2
    h.fail_state_alloc = True  # storage that cannot be had: no state, nothing charged
    c = pt.family_prompt([], 5, 70)
    h.run(c, [], 0)
    wc = h.insert(c, 70, [70], 3)
    before = h.counters()[3]
    assert not h.add_state(wc[0][0], 3) and h.counters()[3] <= before
    h.end_session()
    h.close()


def test_scopes_never_match_across(lb):
    h = host(lb, 0)
    a = pt.family_prompt([], 4, 100)
    h.run(a, [], 0)
    h.insert(a, 100, [], 1, 1)
    assert h.match(a, 1)[0] == 100 and h.match(a, 2)[0] == 0 and h.match(a)[0] == 0
    h.insert(a, 100, [50], 2, 2)
    assert h.counters()[0] == 3 and h.match(a, 2)[0] == 100 and len(h.match(a, 1)[1]) == 1 and len(h.match(a, 2)[1]) == 2
    h.end_session()
    h.clear()
    assert h.live_pages() == 0
    h.close()


def test_a_failed_hold_stores_nothing_past_it_and_leaks_nothing(lb):
    h = host(lb, 0)
    a = pt.family_prompt([], 5, 200)
    h.run(a, [], 0)
    h.P("release")(h.pool, h.table[2])
    h.table[2] = 0
    h.insert(a, 200, [64], 1)
    assert h.counters()[0] == 1 and h.match(a)[0] == 64 and h.refs(h.table[1]) == 1
    h.end_session()
    h.clear()
    assert h.live_pages() == 0
    h.close()


def test_eviction_takes_the_oldest_leaf_and_spares_the_kept_path(lb):
    h = host(lb, 0)
    a, b = pt.family_prompt([], 6, 70), pt.family_prompt([], 7, 70)
    h.run(a, [], 0)
    h.insert(a, 70, [], 5)
    h.run(b, [], 0)
    h.insert(b, 70, [], 9)
    assert h.evict_lru_leaf(keep=h.match(a)[1]) == 1 and h.match(a)[0] == 70 and h.match(b)[0] == 0
    assert h.evict_lru_leaf(keep=h.match(a)[1]) == 0
    assert h.evict_lru_leaf() == 1 and h.match(a)[0] == 0
    h.end_session()
    h.close()


def test_page_lists_and_small_buffers(lb):
    L = lb.lib()
    h = host(lb, 0)
    a = pt.family_prompt([], 8, 130)
    h.run(a, [], 0)
    h.insert(a, 130, [64], 1)
    assert h.page_lists() == sorted([h.table[:1], h.table[1:3]])
    first = h.match(a)[1][0]
    assert h.page_lists(skip=[first]) == [h.table[1:3]]
    pages, lens = (C.c_int * 2)(), (C.c_int * 8)()
    assert L.ling_b200_prefix_page_lists(h.tree, None, 0, pages, 2, lens, 8) == -1  # three pages do not fit in two
    out = (C.c_int * 1)()
    m = h.match(a)
    assert L.ling_b200_prefix_pages(h.tree, pt.arr(m[1]), len(m[1]), 130, out, 1) == -1
    npth = C.c_int(0)
    assert L.ling_b200_prefix_match(h.tree, pt.arr(a), len(a), C.c_uint64(0), None, 0, C.byref(npth)) == 130 and npth.value == 2
    assert L.ling_b200_prefix_insert(h.tree, pt.arr(a), len(a), 0, None, 0, C.c_uint64(2), C.c_uint64(0), None, None, 0) == 0
    h.end_session()
    h.close()
    L.ling_b200_prefix_create.restype = C.c_void_p
    assert L.ling_b200_prefix_create(C.c_size_t(0), C.c_size_t(0), 64, None) is None
