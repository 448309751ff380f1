"""Host logic (no GPU): the oracle and the product's C-ABI host functions against the golden vectors recorded from the
reference's own host code (tests/golden/host_logic.json, made by tests/golden/make_golden.py), and against that code
itself where oracle/_ref was built.  Everything here is integer work: the bar is bit-exact."""
import ctypes as C
import hashlib
import json
import os

import numpy as np
import pytest

import helpers

GOLDEN = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "host_logic.json")))
L = C.c_long


def arr(x, t=C.c_int):
    return (t * max(len(x), 1))(*x)


def compact(t, n):
    return {"depth": list(t.depth)[:n], "var": list(t.var)[:n], "nvar": t.nvar, "paths": [list(t.path[v]) for v in range(t.nvar)],
            "ngdn": t.ngdn, "gdn": [list(t.gdn_step[p])[:t.gdn_len[p]] for p in range(t.ngdn)]}


def test_golden_holds_the_two_branch_tree_of_the_toy_configuration():
    # 16-row chain + 4-row lookup branch off the anchor: two variants, two DeltaNet paths; the chain's last row is
    # emitted as a leaf and once more as a non-writing step; the branch path restarts at the anchor without the write flag.
    c = GOLDEN["trees"][0]
    assert c["parent"] == helpers.chain_plus_branch(16, 4) and c["nvar"] == 2 and c["ngdn"] == 2
    assert c["gdn"][0][-2:] == [15 | 0x100 | 0x200, 15] and c["gdn"][1] == [0, 16 | 0x200, 17 | 0x200, 18 | 0x200, 19 | 0x300]


@pytest.mark.parametrize("side", ["oracle", "product"])
def test_describe_tree_and_greedy_accept_match_golden(side, lb, lo):
    for c in GOLDEN["trees"]:
        n = len(c["parent"])
        t = lb.TreeDesc()
        if side == "oracle":
            rc = lo.lo().lo_describe_tree(arr(c["parent"]), n, c["chain"], C.byref(t))
        else:
            rc = lb.lib().ling_b200_describe_tree(arr(c["parent"]), n, c["chain"], C.byref(t))
        assert (rc != 0) == (c["rc"] != 0)
        if c["rc"] == 0:
            assert hashlib.sha256(bytes(t)).hexdigest() == c["sha256"], c["parent"]
            assert compact(t, n) == {k: c[k] for k in ("depth", "var", "nvar", "paths", "ngdn", "gdn")}
        path, nxt = (C.c_int * 32)(), C.c_int()
        fn = lo.lo().lo_accept_tree_greedy if side == "oracle" else lb.lib().ling_b200_accept_tree_greedy
        ln = fn(arr(c["parent"]), arr(c["token"]), n, arr(c["argmax"]), path, C.byref(nxt))
        assert list(path)[:ln] == c["accept_path"] and nxt.value == c["accept_next"]


def test_tree_description_invariants(lb):
    # the properties the reference's own tree tests assert (tests/spec_tests.cpp:283-335): the chain is rows 0..E, every
    # parent precedes its child, path[var[r]][depth[r]] == r, every row is written exactly once, a leaf step follows its
    # parent's step
    rng = np.random.default_rng(5)
    for _ in range(500):
        n = int(rng.integers(1, 33))
        chain = int(rng.integers(0, n))
        parent = helpers.random_tree(rng, n, chain)
        rc, t = lb.describe_tree(parent, chain)
        leaves = sum(1 for r in range(n) if r not in parent[1:])
        if rc != 0:
            assert leaves > 32
            continue
        assert t.nvar == leaves
        writes = []
        for r in range(n):
            assert t.path[t.var[r]][t.depth[r]] == r
        for p in range(t.ngdn):
            steps = list(t.gdn_step[p])[:t.gdn_len[p]]
            last_adv = None
            for s in steps:
                row, leaf, wr = s & 0xff, bool(s & lb.TREE_LEAF), bool(s & lb.TREE_WRITE)
                if wr:
                    writes.append(row)
                if leaf:
                    assert parent[row] == last_adv
                else:
                    assert last_adv is None and row == 0 or parent[row] == last_adv
                    last_adv = row
        assert sorted(writes) == list(range(n))
        assert [s & 0xff for s in list(t.gdn_step[0])[:t.gdn_len[0]] if not s & lb.TREE_LEAF][:chain + 1] == list(range(chain + 1))


@pytest.mark.parametrize("side", ["oracle", "product"])
def test_lookup_matches_golden(side, lb, lo):
    fn = lo.lo().lo_lookup_propose if side == "oracle" else lb.lib().ling_b200_lookup_propose
    for c in GOLDEN["lookup"]:
        out, m = (C.c_int * 64)(), C.c_int()
        n = fn(arr(c["seq"]), len(c["seq"]), c["max"], c["ngram"], out, C.byref(m))
        assert list(out)[:n] == c["tokens"] and m.value == c["match"]


def test_lookup_known_answers(lb):
    # a verbatim copy in progress: the continuation of the most recent earlier occurrence, and how far back it agrees
    def run(seq, mx, ng=3):
        out, m = (C.c_int * 64)(), C.c_int()
        n = lb.lib().ling_b200_lookup_propose(arr(seq), len(seq), mx, ng, out, C.byref(m))
        return list(out)[:n], m.value
    assert run([1, 2, 3, 4, 5, 9, 1, 2, 3], 2) == ([4, 5], 3)
    assert run([7, 1, 2, 3, 4, 8, 7, 1, 2, 3], 4) == ([4, 8, 7, 1], 4)
    assert run([1, 2, 3], 4) == ([], 0)
    assert run([1, 2, 3, 1, 2, 3, 1, 2, 3], 5) == ([1, 2, 3], 6)


def test_build_tree_matches_golden(lb):
    fn = lb.lib().ling_b200_build_tree
    fn.argtypes = [C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_float), C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int),
                   C.c_int, C.c_double, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int),
                   C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_double)]
    for c in GOLDEN["build_tree"]:
        par, dep, tok, pk, mass = (C.c_int * 64)(), (C.c_int * 64)(), (C.c_int * 64)(), (C.c_int * 64)(), C.c_double()
        r = fn(7, arr(c["cand"]), arr(c["scores"], C.c_float), c["E"], 16, arr(c["tokens"]), arr(c["picks"]), c["nodes"], c["temp"],
               c["width"], c["max_depth"], c["chain"], 32, par, dep, tok, pk, C.byref(mass))
        rows = r & 0xffff
        assert rows == c["rows"] and (r >> 16) == c["E_out"]
        assert list(par)[:rows] == c["parent"] and list(dep)[:rows] == c["depth"]
        assert list(tok)[:rows] == c["token"] and list(pk)[:rows] == c["pick"]
        assert mass.value == pytest.approx(c["extra_mass"], rel=1e-12, abs=1e-300)


def test_kvpool_replays_the_reference_traces(lb):
    Lb = lb.lib()
    for tr in GOLDEN["kvpool"]:
        pool = C.c_void_p(Lb.ling_b200_kvpool_create(tr["pages"], 64))
        holders = [[], [], []]
        for rec in tr["ops"]:
            h, kind = rec["holder"], rec["op"]
            t = holders[h]
            cap = 64
            buf, ln = (C.c_int * cap)(*t), C.c_int(len(t))
            if kind == "ensure":
                copies, nc = (C.c_int * 64)(), C.c_int()
                ret = Lb.ling_b200_kvpool_ensure(pool, buf, C.byref(ln), cap, rec["from"], rec["to"], copies, 32, C.byref(nc))
                assert ret == rec["ret"] and list(copies)[:2 * nc.value] == rec["copies"]
                holders[h] = list(buf)[:ln.value]
            elif kind == "share":
                if rec["ret"] != -9:
                    s = holders[rec["src"]]
                    assert Lb.ling_b200_kvpool_share(pool, buf, C.byref(ln), cap, arr(s), len(s), rec["n"]) == rec["ret"]
                    holders[h] = list(buf)[:ln.value]
            elif kind in ("truncate", "unshare"):
                getattr(Lb, "ling_b200_kvpool_" + kind)(pool, buf, len(t), rec["n"])
                holders[h] = list(buf)[:len(t)]
            elif kind == "retire":
                Lb.ling_b200_kvpool_retire(pool)
            elif kind == "needed":
                assert Lb.ling_b200_kvpool_needed(pool, arr(t), len(t), rec["from"], rec["to"]) == rec["ret"]
            elif kind == "resume_need":
                d = holders[rec["donor"]] if rec["donor"] >= 0 else None
                got = Lb.ling_b200_kvpool_resume_need(pool, arr(t), len(t), rec["reuse"], rec["pages"],
                                                      arr(d) if d is not None else None, len(d) if d is not None else 0)
                assert got == rec["ret"]
            elif kind == "net_need":
                assert Lb.ling_b200_kvpool_net_need(pool, arr(t), len(t), rec["pages"]) == rec["ret"]
            elif kind == "reclaimable":
                keep = [arr(holders[i]) for i in rec["which"]]
                tabs = (C.POINTER(C.c_int) * max(len(keep), 1))(*[C.cast(k, C.POINTER(C.c_int)) for k in keep])
                lens = arr([len(holders[i]) for i in rec["which"]])
                assert Lb.ling_b200_kvpool_reclaimable(pool, tabs, lens, len(keep)) == rec["ret"]
            elif kind == "release_all":
                for p in t:
                    if p:
                        assert Lb.ling_b200_kvpool_release(pool, p) == 0
                holders[h] = []
            assert [list(x) for x in holders] == rec["tables"], kind
            assert Lb.ling_b200_kvpool_free_pages(pool) == rec["free"]
            assert Lb.ling_b200_kvpool_pending_pages(pool) == rec["pending"]
            assert [Lb.ling_b200_kvpool_refs(pool, p) for p in range(tr["pages"])] == rec["refs"]
        Lb.ling_b200_kvpool_destroy(pool)


def test_kvpool_literal_page_counts(lb):
    # 16-token pages (the toy configuration): a holder writing [0, 40) maps 3 pages, lowest ids first; a second holder
    # sharing [0, 20) and then writing position 18 gets a private copy of page index 1 only
    Lb = lb.lib()
    pool = C.c_void_p(Lb.ling_b200_kvpool_create(8, 16))
    a, la = (C.c_int * 8)(), C.c_int(0)
    copies, nc = (C.c_int * 16)(), C.c_int()
    assert Lb.ling_b200_kvpool_ensure(pool, a, C.byref(la), 8, 0, 40, copies, 8, C.byref(nc)) == 1
    assert list(a)[:la.value] == [1, 2, 3] and nc.value == 0 and Lb.ling_b200_kvpool_free_pages(pool) == 4
    b, lb_ = (C.c_int * 8)(), C.c_int(0)
    assert Lb.ling_b200_kvpool_share(pool, b, C.byref(lb_), 8, a, la.value, 20) == 0
    assert list(b)[:lb_.value] == [1, 2] and Lb.ling_b200_kvpool_refs(pool, 2) == 2
    assert Lb.ling_b200_kvpool_needed(pool, b, lb_.value, 18, 19) == 1
    assert Lb.ling_b200_kvpool_ensure(pool, b, C.byref(lb_), 8, 18, 19, copies, 8, C.byref(nc)) == 1
    assert list(b)[:lb_.value] == [1, 4] and list(copies)[:2] == [2, 4] and Lb.ling_b200_kvpool_refs(pool, 2) == 1
    # all or nothing: a write that needs more pages than are free changes nothing
    assert Lb.ling_b200_kvpool_ensure(pool, b, C.byref(lb_), 8, 32, 128, copies, 8, C.byref(nc)) == 0
    assert list(b)[:lb_.value] == [1, 4] and Lb.ling_b200_kvpool_free_pages(pool) == 3
    # a released page is handed out again only after retire()
    Lb.ling_b200_kvpool_truncate(pool, a, la.value, 16)
    assert list(a)[:3] == [1, 0, 0] and Lb.ling_b200_kvpool_pending_pages(pool) == 2 and Lb.ling_b200_kvpool_free_pages(pool) == 3
    Lb.ling_b200_kvpool_retire(pool)
    assert Lb.ling_b200_kvpool_free_pages(pool) == 5 and Lb.ling_b200_kvpool_pending_pages(pool) == 0
    Lb.ling_b200_kvpool_destroy(pool)


def test_pairing_and_policy_match_golden(lb):
    Lb = lb.lib()
    for c in GOLDEN["policy"]["pair"]:
        n = len(c["batchable"])
        order, batch = (C.c_int * 16)(), (C.c_int * 16)()
        no = Lb.ling_b200_pair_order(arr(c["batchable"]), arr(c["recent"]), arr(c["last"], L), n, c["fair"], order)
        nb = Lb.ling_b200_select_batch(arr(c["batchable"]), arr(c["recent"]), arr(c["last"], L), n, c["self"], c["fit"], c["fair"], batch)
        assert list(order)[:no] == c["order"] and list(batch)[:nb] == c["batch"]
    for c in GOLDEN["policy"]["verdict"]:
        assert Lb.ling_b200_kv_verdict(c["need"], c["free"], c["pending"], c["idle"]) == c["ret"]
    for c in GOLDEN["policy"]["last_resort"]:
        n = len(c["admitted"])
        assert Lb.ling_b200_kv_last_resort(arr(c["admitted"], L), arr(c["waiting"]), arr(c["need"]), n, c["free"], c["pending"],
                                           c["idle"]) == c["ret"]


def test_fair_pairing_evens_out_the_passes(lb):
    # Four decoding requests, room for two per batched pass.  In running order the first request is in every pass; with
    # fair pairing the passes even out (the behaviour src/serve/pairing.hpp:1-9 in the reference describes).
    Lb = lb.lib()

    def simulate(fair, turns=400):
        marks = [[] for _ in range(4)]
        passes, now = [0] * 4, 0
        for turn in range(turns):
            recent = [sum(1 for m in w if m > now - 16) for w in marks]
            last = [w[-1] if w and w[-1] > now - 16 else 0 for w in marks]
            batch = (C.c_int * 8)()
            nb = Lb.ling_b200_select_batch(arr([1] * 4), arr(recent), arr(last, L), 4, turn % 4, 2, fair, batch)
            now += 1
            for i in list(batch)[:nb]:
                marks[i] = [m for m in marks[i] if m > now - 16] + [now]
                if turn >= 100:
                    passes[i] += 1
        return passes
    legacy, fair = simulate(0), simulate(1)
    assert legacy[0] == max(legacy) and legacy[0] >= 2 * min(legacy)
    assert max(fair) - min(fair) <= 2


def test_admission_matches_golden(lb):
    Lb = lb.lib()
    Lb.ling_b200_start_plan.argtypes = [C.POINTER(lb.ModelConfig), C.c_size_t, C.c_size_t, C.c_int, C.c_int, C.c_int, C.c_long,
                                        C.c_long, C.c_int, C.c_size_t, C.c_long, C.c_int, C.c_int, C.POINTER(lb.MemoryPlan)]
    Lb.ling_b200_choose_size.argtypes = [C.POINTER(lb.ModelConfig), C.c_size_t, C.c_size_t, C.c_int, C.c_long, C.c_long, C.c_int,
                                         C.c_int, C.c_int, C.c_int, C.c_int, C.c_size_t, C.c_long, C.c_int, C.c_int] + \
        [C.POINTER(C.c_int)] * 5
    cfg = lb.config_27b()
    scratch = 4 << 30
    for c in GOLDEN["admission"]["plan"]:
        p = lb.MemoryPlan()
        # the reference's constants: 64-position pages, BF16 KV (2 bytes an element)
        assert Lb.ling_b200_start_plan(C.byref(cfg), c["weights"], scratch, c["drafter"], c["sessions"], c["ctx"], c["avail"],
                                       c["reserve"], c["kv_on"], c["store"], c["pool_mb"], 64, 2, C.byref(p)) == 0
        assert {f[0]: int(getattr(p, f[0])) for f in lb.MemoryPlan._fields_} == c["plan"], c
    for c in GOLDEN["admission"]["choose"]:
        o = [C.c_int() for _ in range(5)]
        Lb.ling_b200_choose_size(C.byref(cfg), c["weights"], scratch, c["drafter"], c["avail"], c["reserve"], c["full_ctx"],
                                 c["sessions_in"], c["ctx_in"], c["auto"], c["kv_on"], c["store"], c["pool_mb"], 64, 2,
                                 *[C.byref(x) for x in o])
        assert [x.value for x in o] == c["out"], c


def test_step_trace_line_matches_golden(lb):
    fn = lb.lib().ling_b200_format_step
    fn.argtypes = [C.c_double, C.c_long, C.c_char_p, C.c_size_t, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int),
                   C.POINTER(C.c_int), C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_long), C.POINTER(C.c_long), C.c_int, C.c_double,
                   C.c_int, C.c_char_p, C.c_int]
    for r in GOLDEN["trace"]:
        buf = C.create_string_buffer(2048)
        n = fn(r["t"], r["pass"], r["kind"].encode(), r["turn"], arr(r["sessions"]), arr(r["rows"]), arr(r["tokens"]),
               arr(r["left"]), len(r["sessions"]), arr(r["cand"]), arr(r["cand_request"], L), arr(r["cand_last"], L),
               len(r["cand_request"]), r["ms"], r["side"], buf, 2048)
        assert n == len(r["line"]) and buf.value.decode() == r["line"]


def test_against_the_reference_host_code_itself(lb, lo):
    ref = lo.ref()
    if ref is None:
        pytest.skip("oracle/_ref was not built (the reference project is not mounted here)")
    rng = np.random.default_rng(77)
    for _ in range(1500):
        n = int(rng.integers(1, 33))
        chain = int(rng.integers(0, n))
        parent = helpers.random_tree(rng, n, chain)
        a, b, c = lb.TreeDesc(), lb.TreeDesc(), lb.TreeDesc()
        ra = ref.ref_describe_tree(arr(parent), n, chain, C.byref(a))
        rb = lo.lo().lo_describe_tree(arr(parent), n, chain, C.byref(b))
        rc = lb.lib().ling_b200_describe_tree(arr(parent), n, chain, C.byref(c))
        assert (ra != 0) == (rb != 0) == (rc != 0)
        if ra == 0:
            assert bytes(a) == bytes(b) == bytes(c)


def run_reclaim(lib, c):
    """kv_reclaim through the C ABI on a scripted scenario: the callbacks keep the counters the reference's closures keep."""
    state = {"need": c["need0"], "have": c["have0"], "evicted": [0] * len(c["sizes"])}
    first = np.concatenate([[0], np.cumsum(c["sizes"])]).astype(int)
    COUNT, EVICT = C.CFUNCTYPE(C.c_int, C.c_void_p), C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int)

    def evict(_, g):
        if state["evicted"][g] >= c["sizes"][g]:
            return 0
        e = int(first[g]) + state["evicted"][g]
        state["evicted"][g] += 1
        state["need"] += c["dneed"][e]
        state["have"] += c["dhave"][e]
        return 1

    ret = lib.ling_b200_kv_reclaim(COUNT(lambda _: state["need"]), COUNT(lambda _: state["have"]), EVICT(evict), None, c["n_kept"],
                                   c["need_kept"], c["reach_kept"], c["n_source"], c["need_all"], c["reach_all"], c["must"])
    return ret, state["evicted"]


def test_reclaim_and_refusal_match_golden(lb, lo):
    lib = lb.lib()
    for c in GOLDEN["reclaim"]["reclaim"]:
        assert run_reclaim(lib, c) == (c["ret"], c["evicted"]), c
    lib.ling_b200_refuse_request.argtypes = [C.c_long, C.c_long, C.c_char_p, C.c_int]
    for c in GOLDEN["reclaim"]["refuse"]:
        buf = C.create_string_buffer(512)
        assert lib.ling_b200_refuse_request(c["avail"], c["reserve"], buf, 512) == c["len"] and buf.value.decode() == c["text"]
    assert lib.ling_b200_refuse_request(5, 16384, C.create_string_buffer(8), 8) == -1       # a buffer too small is reported
    ref = lo.ref()
    if ref is not None:   # and against the reference's own code, live
        rng = np.random.default_rng(77)
        for _ in range(200):
            n_kept, n_source = int(rng.integers(0, 4)), int(rng.integers(0, 3))
            sizes = [int(x) for x in rng.integers(0, 4, n_kept + n_source)]
            c = {"need0": int(rng.integers(0, 14)), "have0": int(rng.integers(0, 8)), "sizes": sizes,
                 "dneed": [int(x) for x in rng.integers(-2, 2, sum(sizes))], "dhave": [int(x) for x in rng.integers(0, 5, sum(sizes))],
                 "n_kept": n_kept, "n_source": n_source, "must": int(rng.integers(0, 2))}
            c["need_kept"], c["reach_kept"], c["need_all"], c["reach_all"] = (int(x) for x in rng.integers(0, 14, 4))
            ev = (C.c_int * 8)()
            ret = ref.ref_kv_reclaim(c["need0"], c["have0"], arr(sizes), arr(c["dneed"]), arr(c["dhave"]), n_kept, c["need_kept"],
                                     c["reach_kept"], n_source, c["need_all"], c["reach_all"], c["must"], ev)
            assert run_reclaim(lib, c) == (ret, list(ev)[:len(sizes)])


def test_row_classes_and_token_tiles(lb):
    """Steps run in capacity classes and the GEMMs in token tiles of 32, 64, 96 or 128 rows: up to 128 rows the smallest tile that
    holds them (the class is that tile); beyond, classes of 32 rows and the tile with the least padded rows weighted by the tile's
    measured cost per row (96: 1, 64: 1.05, 128: 1.08), never more padded rows than 128-row tiles would have."""
    L = lb.lib()
    assert [L.ling_b200_token_tile(m) for m in (1, 32, 33, 64, 65, 96, 97, 128)] == [32, 32, 64, 64, 96, 96, 128, 128]
    assert [L.ling_b200_row_class(m) for m in (1, 24, 33, 74, 100, 128, 129, 142, 260, 1135, 2048)] == \
        [32, 32, 64, 96, 128, 128, 160, 160, 288, 1152, 2048]
    assert L.ling_b200_token_tile(0) == 0 and L.ling_b200_row_class(-3) == 0
    for m in range(129, 2049):
        cls = L.ling_b200_row_class(m)
        nt = L.ling_b200_token_tile(cls)
        assert cls % 32 == 0 and m <= cls < m + 32 and nt in (64, 96, 128)
        pad = lambda t: -(-cls // t) * t
        cost = lambda t: pad(t) * {64: 1.05, 96: 1.0, 128: 1.08}[t]
        fits = [t for t in (64, 96, 128) if pad(t) <= pad(128)]     # the activation buffers hold whole 128-row tiles
        assert nt in fits and cost(nt) == min(cost(t) for t in fits)
    assert [L.ling_b200_token_tile(c) for c in (160, 192, 256, 288, 320, 1152, 2048)] == [96, 96, 64, 96, 64, 96, 64]
