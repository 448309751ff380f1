"""Records what the reference's own PrefixKvTree (paged mode, over its own KvPool) and ArenaAlloc do on seeded random
traces, into tests/golden/prefix_kv.json.  Needs the reference's host code behind C wrappers:

    make -C oracle ref REF=/path/to/reference && python tests/golden/make_golden_prefix.py

tests/test_prefix_store.py replays the same traces (tests/prefix_trace.py) on the product's tree and compares.
"""
import ctypes as C
import json
import os
import random
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import prefix_trace as pt  # noqa: E402
from oracle import lo  # noqa: E402

STATE = 1 << 20
TREE_CASES = [{"seed": 5, "steps": 250, "states": 64}, {"seed": 11, "steps": 250, "states": 6}, {"seed": 23, "steps": 150, "states": 0}]
ARENA_CASES = [{"seed": 3, "size": 1 << 20, "align": 256, "steps": 400}, {"seed": 9, "size": 100000, "align": 64, "steps": 400}]


def arena_trace(L, prefix, case):
    """Random allocations and releases; the log is every returned offset and the bytes in use."""
    for n in ("create",):
        getattr(L, prefix + n).restype = C.c_void_p
    for n in ("size", "in_use"):
        getattr(L, prefix + n).restype = C.c_size_t
    getattr(L, prefix + "alloc").restype = C.c_longlong
    rng = random.Random(case["seed"])
    a = C.c_void_p(getattr(L, prefix + "create")(C.c_size_t(case["size"]), C.c_size_t(case["align"])))
    live, log = [], [int(getattr(L, prefix + "size")(a))]
    for _ in range(case["steps"]):
        if live and rng.randrange(5) < 2:
            off = live.pop(rng.randrange(len(live)))
            getattr(L, prefix + "release")(a, C.c_size_t(off))
            log.append(["r", off, int(getattr(L, prefix + "in_use")(a))])
        else:
            want = rng.randrange(1, case["size"] // 6)
            off = int(getattr(L, prefix + "alloc")(a, C.c_size_t(want)))
            if off >= 0:
                live.append(off)
            log.append(["a", want, off, int(getattr(L, prefix + "in_use")(a))])
    getattr(L, prefix + "release")(a, C.c_size_t(12345))  # not an allocation: ignored
    log.append(int(getattr(L, prefix + "in_use")(a)))
    getattr(L, prefix + "destroy")(a)
    return log


def main():
    R = lo.ref()
    assert R is not None, "build oracle/_ref first (make -C oracle ref REF=...)"
    out = {"tree": [], "arena": []}
    for case in TREE_CASES:
        h = pt.Host(R, True, 400, case["states"] * STATE, STATE)
        out["tree"].append({**case, "log": pt.random_sessions(h, case["seed"], case["steps"], STATE)})
        h.close()
    for case in ARENA_CASES:
        out["arena"].append({**case, "log": arena_trace(R, "ref_arena_", case)})
    with open(os.path.join(HERE, "prefix_kv.json"), "w") as f:
        json.dump(out, f, separators=(",", ":"))
    print("wrote prefix_kv.json:", os.path.getsize(os.path.join(HERE, "prefix_kv.json")), "bytes")


if __name__ == "__main__":
    main()
