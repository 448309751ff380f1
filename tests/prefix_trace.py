"""A host model of sessions using the prefix KV store, driven the same way against the product's tree
(ling_b200_prefix_* over ling_b200_kvpool_*) and against the reference's own PrefixKvTree and KvPool behind C wrappers
(ref_prefix_* over ref_kvpool_*), so that their observable behaviour can be compared step by step.

The KV "contents" of a position are a hash of the whole prompt up to it (as in the reference's tests/prefix_kv_tests.cpp:
the KV depends on every earlier token), kept per page on the host, so that a restore that maps a page another prompt wrote
is caught by the model itself, whichever implementation runs.
"""
import ctypes as C
import random

PT = 64  # the reference's page size is a constant; the product's is a parameter and the comparison uses 64

HOLD = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_int), C.c_int)
PAGE = C.CFUNCTYPE(None, C.c_void_p, C.c_int)
ALLOC = C.CFUNCTYPE(C.c_void_p, C.c_void_p, C.c_size_t)
FREE = C.CFUNCTYPE(None, C.c_void_p, C.c_void_p)


class Ops(C.Structure):
    _fields_ = [("user", C.c_void_p), ("hold", HOLD), ("retain", PAGE), ("drop", PAGE), ("state_alloc", ALLOC),
                ("state_release", FREE)]


def arr(v):
    return (C.c_int * max(len(v), 1))(*v)


def kv_at(prompt, pos):
    h = 1469598103934665603
    for i in range(pos + 1):
        h = ((h ^ (prompt[i] + 7)) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h


class Host:
    """One pool, one active session (table + per-page memory), one tree, on either implementation."""

    def __init__(self, L, is_ref, pool_pages, budget, state_bytes):
        self.L, self.is_ref = L, is_ref
        self.pp = "ref_kvpool_" if is_ref else "ling_b200_kvpool_"
        self.tp = "ref_prefix_" if is_ref else "ling_b200_prefix_"
        for n in ("create", "add_state"):
            getattr(L, self.tp + n).restype = C.c_void_p
        getattr(L, self.tp + "bytes").restype = C.c_size_t
        getattr(L, self.pp + "create").restype = C.c_void_p
        self.pool = C.c_void_p(self.P("create")(pool_pages) if is_ref else self.P("create")(pool_pages, PT))
        self.pool_pages = pool_pages
        self.table, self.mem = [], {}
        self.states, self.next_state = set(), 1
        self.fail_state_alloc = False
        self.ops = Ops(None, HOLD(self._hold), PAGE(self._retain), PAGE(self._drop), ALLOC(self._alloc), FREE(self._free))
        if is_ref:
            self.tree = C.c_void_p(self.T("create")(C.c_size_t(budget), C.c_size_t(state_bytes), C.byref(self.ops)))
        else:
            self.tree = C.c_void_p(self.T("create")(C.c_size_t(budget), C.c_size_t(state_bytes), PT, C.byref(self.ops)))

    def P(self, name):
        return getattr(self.L, self.pp + name)

    def T(self, name):
        return getattr(self.L, self.tp + name)

    def close(self):
        self.T("destroy")(self.tree)
        self.P("destroy")(self.pool)

    # ---- callbacks
    def _hold(self, _user, lo, hi, out, cap):
        n = 0
        for i in range(lo // PT, (hi - 1) // PT + 1):
            pg = self.table[i] if i < len(self.table) else 0
            if pg:
                self.P("retain")(self.pool, pg)
            if n < cap:
                out[n] = pg
            n += 1
        return n

    def _retain(self, _user, pg):
        self.P("retain")(self.pool, pg)

    def _drop(self, _user, pg):
        self.P("release")(self.pool, pg)

    def _alloc(self, _user, _bytes):
        if self.fail_state_alloc:
            return None
        s = self.next_state
        self.next_state += 1
        self.states.add(s)
        return s

    def _free(self, _user, p):
        self.states.discard(p)

    # ---- the pool
    def refs(self, pg):
        return self.P("refs")(self.pool, pg)

    def free_pages(self):
        return self.P("free_pages")(self.pool)

    def pending_pages(self):
        return self.P("pending_pages")(self.pool)

    def live_pages(self):
        return sum(1 for pg in range(1, self.pool_pages) if self.refs(pg) > 0)

    def end_session(self):
        for pg in self.table:
            if pg:
                self.P("release")(self.pool, pg)
        self.table = []

    def run(self, prompt, from_store, n):
        """A session that runs `prompt`: maps the store's pages for [0, n), copies the page n falls in when it is shared,
        writes [n, L) into private pages only."""
        self.end_session()
        for pg in from_store:
            self.P("retain")(self.pool, pg)
            self.table.append(pg)
        L = len(prompt)
        cap = max(len(self.table), (L + PT - 1) // PT) + 1
        buf = (C.c_int * cap)(*self.table)
        ln, nc = C.c_int(len(self.table)), C.c_int(0)
        copies = (C.c_int * (2 * cap))()
        ok = self.P("ensure")(self.pool, buf, C.byref(ln), cap, n, L, copies, cap, C.byref(nc))
        assert ok == 1, "the pool ran out"
        self.table = list(buf)[:ln.value]
        for i in range(nc.value):
            self.mem[copies[2 * i + 1]] = list(self.mem[copies[2 * i]])
        for pos in range(n, L):
            pg = self.table[pos // PT]
            assert self.refs(pg) == 1, "a shared page would be written"
            self.mem.setdefault(pg, [0] * PT)
            if len(self.mem[pg]) < PT:
                self.mem[pg] = [0] * PT
            self.mem[pg][pos % PT] = kv_at(prompt, pos)

    # ---- the tree
    def match(self, prompt, scope=0):
        path, npth = (C.c_int * 256)(), C.c_int(0)
        ln = self.T("match")(self.tree, arr(prompt), len(prompt), C.c_uint64(scope), path, 256, C.byref(npth))
        return ln, list(path)[:npth.value]

    def best_state(self, m, limit):
        st = C.c_void_p()
        pos = self.T("best_state")(self.tree, arr(m[1]), len(m[1]), m[0], limit, C.byref(st))
        return pos, st.value

    def pages(self, m, n):
        out = (C.c_int * 256)()
        if self.is_ref:
            c = self.T("pages")(self.tree, arr(m[1]), len(m[1]), m[0], n, out, 256)
        else:
            c = self.T("pages")(self.tree, arr(m[1]), len(m[1]), n, out, 256)
        assert c >= 0
        return list(out)[:c]

    def touch(self, m, epoch):
        self.T("touch")(self.tree, arr(m[1]), len(m[1]), C.c_uint64(epoch))

    def insert(self, prompt, q, cuts, epoch, scope=0):
        wn, wp = (C.c_int * 64)(), (C.c_int * 64)()
        c = self.T("insert")(self.tree, arr(prompt), len(prompt), q, arr(cuts), len(cuts), C.c_uint64(epoch), C.c_uint64(scope),
                             wn, wp, 64)
        return [(wn[i], wp[i]) for i in range(c)]

    def add_state(self, node, epoch):
        return self.T("add_state")(self.tree, node, C.c_uint64(epoch))

    def evict_lru_leaf(self, keep=()):
        return self.T("evict_lru_leaf")(self.tree, arr(list(keep)), len(keep))

    def clear(self):
        self.T("clear")(self.tree)

    def counters(self):
        return [self.T("nodes")(self.tree), self.T("states")(self.tree), self.T("pages_held")(self.tree), int(self.T("bytes")(self.tree)),
                self.free_pages(), self.pending_pages(), len(self.states)]

    def page_lists(self, skip=()):
        pages, lens = (C.c_int * 4096)(), (C.c_int * 1024)()
        n = self.T("page_lists")(self.tree, arr(list(skip)), len(skip), pages, 4096, lens, 1024)
        assert n >= 0
        out, at = [], 0
        for i in range(n):
            out.append(list(pages[at:at + lens[i]]))
            at += lens[i]
        return sorted(out)


def family_prompt(shared, salt, n):
    rng = random.Random(salt)
    return list(shared) + [1000 + rng.randrange(50000) for _ in range(n)]


def random_sessions(h, seed, steps, state_bytes):
    """Random sessions over a family of prompts with shared beginnings and two scopes.  Every restore is checked against its
    own prompt by the model; the returned log is what an implementation is compared by."""
    rng = random.Random(seed)
    family = [family_prompt(range(37 + 41 * f), 10 + f, 400) for f in range(6)]
    log = []
    for epoch in range(1, steps + 1):
        evicted = 0
        while h.free_pages() + h.pending_pages() < 24 and h.evict_lru_leaf():
            evicted += 1
        h.P("retire")(h.pool)
        p = list(family[rng.randrange(len(family))])
        p = p[:1 + rng.randrange(len(p))]
        if rng.randrange(3) == 0:
            for i in range(rng.randrange(len(p)), len(p)):
                p[i] = 90000 + rng.randrange(50)
        scope = rng.randrange(2)
        m = h.match(p, scope)
        limit = min(m[0], len(p) - 1)
        state_pos, _ = h.best_state(m, limit)
        n = limit
        if rng.randrange(4) == 0:
            n //= 2
        pg = h.pages(m, n)
        for pos in range(n):
            assert h.mem[pg[pos // PT]][pos % PT] == kv_at(p, pos), "a restore read another prompt's KV"
        if rng.randrange(2) == 0:
            h.touch(m, epoch)
        h.run(p, pg, n)
        cuts = sorted(1 + rng.randrange(len(p)) for _ in range(3))
        want = h.insert(p, len(p), cuts, epoch, scope)
        added = [bool(h.add_state(node, epoch)) for node, _ in want]
        extra = h.evict_lru_leaf() if rng.randrange(5) == 0 else -1
        if rng.randrange(7) == 0:
            h.end_session()
        log.append({"len": m[0], "path": len(m[1]), "state_pos": state_pos, "n": n, "pages": pg, "want": [w[1] for w in want],
                    "added": added, "evicted": evicted, "extra": extra, "counters": h.counters()})
    log.append({"page_lists": h.page_lists()})
    h.end_session()
    h.clear()
    log.append({"live_after_clear": h.live_pages(), "states_after_clear": len(h.states)})
    return log
