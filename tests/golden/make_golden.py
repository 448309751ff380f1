"""Generates tests/golden/host_logic.json by running the REFERENCE's own host code (oracle/_ref/libling_ref.so, built by
`make -C oracle ref` from the reference project's sources) on seeded inputs.

    python tests/golden/make_golden.py

The fixture travels with the repository; the reference project does not, so the tests on a machine without it check the
oracle and the product against these recorded outputs.  Every input is produced by numpy's PCG64 from the seeds below.
"""
import ctypes as C
import hashlib
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
from oracle import lo as lom  # noqa: E402
import helpers  # noqa: E402


class TreeDesc(C.Structure):
    _fields_ = [("n", C.c_int), ("depth", C.c_int * 32), ("var", C.c_int * 32), ("nvar", C.c_int), ("path", (C.c_int * 32) * 32),
                ("ngdn", C.c_int), ("gdn_len", C.c_int * 32), ("gdn_step", (C.c_int * 64) * 32)]


def arr(x, t=C.c_int):
    return (t * max(len(x), 1))(*x)


def tree_cases(ref, rng):
    out = []
    shapes = [(helpers.chain_plus_branch(16, 4), 15), (helpers.chain_plus_branch(16, 8), 15), ([-1], 0),
              (helpers.chain_plus_branch(12, 0), 11), (helpers.chain_plus_branch(1, 5), 0)]
    for _ in range(300):
        n = int(rng.integers(1, 33))
        chain = int(rng.integers(0, n))
        shapes.append((helpers.random_tree(rng, n, chain), chain))
    for parent, chain in shapes:
        n = len(parent)
        t = TreeDesc()
        rc = ref.ref_describe_tree(arr(parent), n, chain, C.byref(t))
        case = {"parent": [int(p) for p in parent], "chain": chain, "rc": rc}
        if rc == 0:
            case.update({
                "sha256": hashlib.sha256(bytes(t)).hexdigest(), "depth": list(t.depth)[:n], "var": list(t.var)[:n],
                "nvar": t.nvar, "paths": [list(t.path[v]) for v in range(t.nvar)], "ngdn": t.ngdn,
                "gdn": [list(t.gdn_step[p])[:t.gdn_len[p]] for p in range(t.ngdn)]})
        tok = [int(x) for x in rng.integers(0, 4, n)]
        am = [int(x) for x in rng.integers(0, 4, n)]
        path = (C.c_int * 32)()
        nxt = C.c_int()
        ln = ref.ref_accept_tree_greedy(arr(parent), arr(tok), n, arr(am), path, C.byref(nxt))
        case.update({"token": tok, "argmax": am, "accept_path": list(path)[:ln], "accept_next": nxt.value})
        out.append(case)
    return out


def lookup_cases(ref, rng):
    out = []
    for _ in range(300):
        L = int(rng.integers(0, 120))
        vocab = int(rng.choice([2, 3, 5, 50]))
        seq = [int(x) for x in rng.integers(0, vocab, L)]
        if L > 30 and rng.random() < 0.5:  # a verbatim copy in progress
            k = int(rng.integers(5, 25))
            seq[-k:] = seq[3:3 + k]
        mx, ng = int(rng.integers(0, 17)), int(rng.integers(1, 5))
        o = (C.c_int * 64)()
        m = C.c_int()
        n = ref.ref_lookup_propose(arr(seq), L, mx, ng, o, C.byref(m))
        out.append({"seq": seq, "max": mx, "ngram": ng, "tokens": list(o)[:n], "match": m.value})
    return out


def build_cases(ref, rng):
    out = []
    ref.ref_build_tree.argtypes = [C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_float), C.c_int, C.c_int, C.POINTER(C.c_int),
                                   C.POINTER(C.c_int), C.c_int, C.c_double, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int),
                                   C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_double)]
    for _ in range(60):
        E, K16 = int(rng.integers(1, 16)), 16
        cand = rng.integers(0, 1000, (E, K16)).astype(np.int32)
        # scores on a coarse grid so that equal priorities (the tie rules) occur
        scores = (rng.integers(-8, 9, (E, K16, K16)) * 0.25).astype(np.float32)
        picks = rng.integers(0, K16, E).astype(np.int32)
        toks = np.array([cand[e, picks[e]] for e in range(E)], np.int32)
        nodes, temp = int(rng.integers(0, 20)), float(rng.choice([0.5, 1.0, 1.5]))
        width, max_depth, chain = int(rng.choice([1, 2, 16])), int(rng.choice([2, 5, 1000])), int(rng.choice([1, 4, 8, 1000]))
        par, dep, tok, pk = (C.c_int * 64)(), (C.c_int * 64)(), (C.c_int * 64)(), (C.c_int * 64)()
        mass = C.c_double()
        r = ref.ref_build_tree(7, cand.ctypes.data_as(C.POINTER(C.c_int)), scores.ctypes.data_as(C.POINTER(C.c_float)), E, K16,
                               toks.ctypes.data_as(C.POINTER(C.c_int)), picks.ctypes.data_as(C.POINTER(C.c_int)), nodes, temp,
                               width, max_depth, chain, par, dep, tok, pk, C.byref(mass))
        rows, Eout = r & 0xffff, r >> 16
        out.append({"E": E, "cand": cand.ravel().tolist(), "scores": scores.ravel().tolist(), "picks": picks.tolist(),
                    "tokens": toks.tolist(), "nodes": nodes, "temp": temp, "width": width, "max_depth": max_depth,
                    "chain": chain, "rows": rows, "E_out": Eout, "parent": list(par)[:rows], "depth": list(dep)[:rows],
                    "token": list(tok)[:rows], "pick": list(pk)[:rows], "extra_mass": mass.value})
    return out


def kvpool_traces(ref, rng):
    """Random walks over the pool's operations; every call and what it returned."""
    traces = []
    for _ in range(12):
        pages = int(rng.integers(4, 40))
        pool = C.c_void_p(ref.ref_kvpool_create(pages))
        holders = [[0] * 0 for _ in range(3)]
        ops = []
        for _ in range(80):
            h = int(rng.integers(0, 3))
            t = holders[h]
            kind = rng.choice(["ensure", "ensure", "share", "truncate", "unshare", "retire", "needed", "resume_need",
                               "net_need", "reclaimable", "release_all"])
            rec = {"op": str(kind), "holder": h}
            cap = 64
            buf = (C.c_int * cap)(*t)
            ln = C.c_int(len(t))
            if kind == "ensure":
                a = int(rng.integers(0, 64 * 8))
                b = a + int(rng.integers(0, 64 * 4))
                copies = (C.c_int * 64)()
                nc = C.c_int()
                rec.update({"from": a, "to": b})
                rec["ret"] = ref.ref_kvpool_ensure(pool, buf, C.byref(ln), cap, a, b, copies, 32, C.byref(nc))
                rec["copies"] = list(copies)[:2 * nc.value]
                holders[h] = list(buf)[:ln.value]
            elif kind == "share":
                src = int(rng.integers(0, 3))
                n = int(rng.integers(0, 64 * 6))
                rec.update({"src": src, "n": n})
                s = holders[src]
                np_ = (n + 63) // 64
                valid = src != h and np_ <= len(s) and all(s[i] != 0 for i in range(np_))  # share() is not atomic on bad input
                rec["ret"] = ref.ref_kvpool_share(pool, buf, C.byref(ln), cap, arr(s), len(s), n) if valid else -9
                if valid and rec["ret"] == 0:
                    holders[h] = list(buf)[:ln.value]
            elif kind in ("truncate", "unshare"):
                n = int(rng.integers(0, 64 * 6))
                rec["n"] = n
                getattr(ref, "ref_kvpool_" + kind)(pool, buf, len(t), n)
                holders[h] = list(buf)[:len(t)]
            elif kind == "retire":
                ref.ref_kvpool_retire(pool)
            elif kind == "needed":
                a = int(rng.integers(0, 64 * 8))
                b = a + int(rng.integers(0, 64 * 4))
                rec.update({"from": a, "to": b, "ret": ref.ref_kvpool_needed(pool, arr(t), len(t), a, b)})
            elif kind == "resume_need":
                reuse, pg = int(rng.integers(0, 64 * 4)), int(rng.integers(0, 10))
                d = int(rng.integers(-1, 3))
                donor = holders[d] if d >= 0 and d != h else None
                rec.update({"reuse": reuse, "pages": pg, "donor": d if donor is not None else -1})
                rec["ret"] = ref.ref_kvpool_resume_need(pool, arr(t), len(t), reuse, pg, arr(donor) if donor is not None else None,
                                                        len(donor) if donor is not None else 0)
            elif kind == "net_need":
                pg = int(rng.integers(0, 10))
                rec.update({"pages": pg, "ret": ref.ref_kvpool_net_need(arr(t), len(t), pg)})
            elif kind == "reclaimable":
                which = [i for i in range(3) if rng.random() < 0.6]
                keep = [arr(holders[i]) for i in which]  # keeps the arrays alive for the call
                tabs = (C.POINTER(C.c_int) * max(len(which), 1))(*[C.cast(k, C.POINTER(C.c_int)) for k in keep])
                lens = arr([len(holders[i]) for i in which])
                rec.update({"which": which, "ret": ref.ref_kvpool_reclaimable(pool, tabs, lens, len(which))})
            elif kind == "release_all":
                for p in t:
                    if p:
                        ref.ref_kvpool_release(pool, p)
                holders[h] = []
            rec["tables"] = [list(x) for x in holders]
            rec["free"] = ref.ref_kvpool_free_pages(pool)
            rec["pending"] = ref.ref_kvpool_pending_pages(pool)
            rec["refs"] = [ref.ref_kvpool_refs(pool, p) for p in range(pages)]
            ops.append(rec)
        ref.ref_kvpool_destroy(pool)
        traces.append({"pages": pages, "ops": ops})
    return traces


def policy_cases(ref, rng):
    out = {"pair": [], "verdict": [], "last_resort": []}
    L = C.c_long
    for _ in range(200):
        n = int(rng.integers(1, 9))
        b = [int(x) for x in rng.integers(0, 2, n)]
        r = [int(x) for x in rng.integers(0, 5, n)]
        last = [int(x) for x in rng.integers(0, 6, n)]
        fair, self_, fit = int(rng.integers(0, 2)), int(rng.integers(0, n)), int(rng.integers(1, 5))
        order, batch = (C.c_int * 16)(), (C.c_int * 16)()
        no = ref.ref_pair_order(arr(b), arr(r), arr(last, L), n, fair, order)
        nb = ref.ref_select_batch(arr(b), arr(r), arr(last, L), n, self_, fit, fair, batch)
        out["pair"].append({"batchable": b, "recent": r, "last": last, "fair": fair, "self": self_, "fit": fit,
                            "order": list(order)[:no], "batch": list(batch)[:nb]})
    for _ in range(200):
        need, fr, pe, idle = (int(x) for x in rng.integers(0, 12, 4))
        out["verdict"].append({"need": need, "free": fr, "pending": pe, "idle": idle, "ret": ref.ref_kv_verdict(need, fr, pe, idle)})
        n = int(rng.integers(0, 5))
        adm = [int(x) for x in rng.integers(0, 50, n)]
        wait = [int(x) for x in (rng.random(n) < 0.8)]
        nd = [int(x) for x in rng.integers(0, 12, n)]
        out["last_resort"].append({"admitted": adm, "waiting": wait, "need": nd, "free": fr, "pending": pe, "idle": idle,
                                   "ret": ref.ref_kv_last_resort(arr(adm, L), arr(wait), arr(nd), n, fr, pe, idle)})
    return out


CFG_27B = [5120, 17408, 64, 248320, 24, 4, 256, 64, 16, 48, 128, 128, 4]


def admission_cases(ref, rng):
    class Plan(C.Structure):
        _fields_ = [("weights", C.c_size_t), ("per_session", C.c_size_t), ("sessions", C.c_size_t), ("scratch", C.c_size_t),
                    ("kv_pool", C.c_size_t), ("session_count", C.c_int), ("kv_pool_pages", C.c_long), ("total", C.c_size_t),
                    ("refused", C.c_int)]
    ref.ref_start_plan.argtypes = [C.POINTER(C.c_int), C.POINTER(C.c_ubyte), C.c_size_t, C.c_size_t, C.c_int, C.c_int, C.c_int,
                                   C.c_long, C.c_long, C.c_int, C.c_size_t, C.c_long, C.POINTER(Plan)]
    ref.ref_choose_size.argtypes = [C.POINTER(C.c_int), C.POINTER(C.c_ubyte), C.c_size_t, C.c_size_t, C.c_int, C.c_long, C.c_long,
                                    C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_size_t, C.c_long, C.POINTER(C.c_int)]
    cfg = arr(CFG_27B)
    full = (C.c_ubyte * 64)(*[(l % 4) == 3 for l in range(64)])
    out = {"plan": [], "choose": []}
    scratch = 4 << 30
    for _ in range(150):
        weights = int(rng.integers(10, 40)) * (1 << 30) + int(rng.integers(0, 1 << 30))
        sessions, ctx = int(rng.integers(1, 9)), int(rng.choice([4096, 32768, 65536, 131072, 262144]))
        avail = int(rng.choice([-1, 30000, 60000, 90000, 117000, 200000]))
        reserve = int(rng.choice([0, 8192, 16384]))
        kv_on, drafter = int(rng.integers(0, 2)), int(rng.integers(0, 2))
        store = int(rng.choice([0, 4 << 30]))
        pool_mb = int(rng.choice([-1, -1, 2048, 20000]))
        p = Plan()
        ref.ref_start_plan(cfg, full, weights, scratch, drafter, sessions, ctx, avail, reserve, kv_on, store, pool_mb, C.byref(p))
        out["plan"].append({"weights": weights, "sessions": sessions, "ctx": ctx, "avail": avail, "reserve": reserve, "kv_on": kv_on,
                            "drafter": drafter, "store": store, "pool_mb": pool_mb,
                            "plan": {f[0]: int(getattr(p, f[0])) for f in Plan._fields_}})
        res = (C.c_int * 5)()
        s_in, c_in = int(rng.choice([-1, -1, 1, 2, 4])), int(rng.choice([-1, -1, 65536]))
        full_ctx, auto = int(rng.choice([0, 262144, 40000])), int(rng.random() < 0.85)
        ref.ref_choose_size(cfg, full, weights, scratch, drafter, avail, reserve, full_ctx, s_in, c_in, auto, kv_on, store, pool_mb, res)
        out["choose"].append({"weights": weights, "avail": avail, "reserve": reserve, "kv_on": kv_on, "drafter": drafter,
                              "store": store, "pool_mb": pool_mb, "sessions_in": s_in, "ctx_in": c_in, "full_ctx": full_ctx,
                              "auto": auto, "out": list(res)})
    return out


def trace_cases(ref, rng):
    ref.ref_format_step.argtypes = [C.c_double, C.c_long, C.c_char_p, C.c_size_t, C.POINTER(C.c_int), C.POINTER(C.c_int),
                                    C.POINTER(C.c_int), C.POINTER(C.c_int), C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_long),
                                    C.POINTER(C.c_long), C.c_int, C.c_double, C.c_int, C.c_char_p, C.c_int]
    out = []
    for _ in range(30):
        n, nc = int(rng.integers(1, 5)), int(rng.integers(0, 5))
        rec = {"t": float(np.round(rng.random() * 100, 6)), "pass": int(rng.integers(0, 1000)),
               "kind": str(rng.choice(["decode", "chunk", "hold"])), "turn": int(rng.integers(0, 4)),
               "sessions": [int(x) for x in rng.integers(0, 8, n)], "rows": [int(x) for x in rng.integers(0, 33, n)],
               "tokens": [int(x) for x in rng.integers(0, 9, n)], "left": [int(x) for x in rng.integers(0, 5000, n)],
               "cand": [int(x) for x in rng.integers(0, 9, 3 * nc)], "cand_request": [int(x) for x in rng.integers(0, 99, nc)],
               "cand_last": [int(x) for x in rng.integers(0, 99, nc)], "ms": float(np.round(rng.random() * 200, 3)),
               "side": int(rng.integers(0, 2))}
        buf = C.create_string_buffer(2048)
        ref.ref_format_step(rec["t"], rec["pass"], rec["kind"].encode(), rec["turn"], arr(rec["sessions"]), arr(rec["rows"]),
                            arr(rec["tokens"]), arr(rec["left"]), n, arr(rec["cand"]), arr(rec["cand_request"], C.c_long),
                            arr(rec["cand_last"], C.c_long), nc, rec["ms"], rec["side"], buf, 2048)
        rec["line"] = buf.value.decode()
        out.append(rec)
    return out


def reclaim_cases(ref, rng):
    """kv_reclaim on scripted scenarios and refuse_request's text."""
    out = {"reclaim": [], "refuse": []}
    for _ in range(300):
        n_kept, n_source = int(rng.integers(0, 4)), int(rng.integers(0, 3))
        sizes = [int(x) for x in rng.integers(0, 4, n_kept + n_source)]
        total = sum(sizes)
        dneed = [int(x) for x in rng.integers(-2, 2, total)]
        dhave = [int(x) for x in rng.integers(0, 5, total)]
        need0, have0 = int(rng.integers(0, 14)), int(rng.integers(0, 8))
        need_kept, reach_kept, need_all, reach_all = (int(x) for x in rng.integers(0, 14, 4))
        must = int(rng.integers(0, 2))
        ev = (C.c_int * 8)()
        ret = ref.ref_kv_reclaim(need0, have0, arr(sizes), arr(dneed), arr(dhave), n_kept, need_kept, reach_kept, n_source, need_all,
                                 reach_all, must, ev)
        out["reclaim"].append({"need0": need0, "have0": have0, "sizes": sizes, "dneed": dneed, "dhave": dhave, "n_kept": n_kept,
                               "need_kept": need_kept, "reach_kept": reach_kept, "n_source": n_source, "need_all": need_all,
                               "reach_all": reach_all, "must": must, "ret": ret, "evicted": list(ev)[:n_kept + n_source]})
    for avail, reserve in ((-1, 8192), (0, 8192), (8191, 8192), (8192, 8192), (9000, 8192), (12, 0), (117000, 16384), (5, 16384)):
        buf = C.create_string_buffer(512)
        n = ref.ref_refuse_request_text(C.c_long(avail), C.c_long(reserve), buf, 512)
        out["refuse"].append({"avail": avail, "reserve": reserve, "len": n, "text": buf.value.decode()})
    return out


def main():
    ref = lom.ref()
    if ref is None:
        raise SystemExit("oracle/_ref/libling_ref.so is missing: run `make -C oracle ref` where the reference project is mounted")
    assert ref.ref_tree_desc_bytes() == C.sizeof(TreeDesc)
    rng = np.random.default_rng(20261125)
    golden = {"trees": tree_cases(ref, rng), "lookup": lookup_cases(ref, rng), "build_tree": build_cases(ref, rng),
              "kvpool": kvpool_traces(ref, rng), "policy": policy_cases(ref, rng), "admission": admission_cases(ref, rng),
              "trace": trace_cases(ref, rng)}
    golden["reclaim"] = reclaim_cases(ref, rng)   # appended last: the sections above keep their random streams
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "host_logic.json")
    with open(path, "w") as f:
        json.dump(golden, f, separators=(",", ":"))
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
