"""The drafter's last stage: top-K of logit rows, the candidate selector's projection and lattice, and the whole stage on a
context feeding build_tree and a verify step.  The oracle's restatements are pinned here to numpy and, on the GPU, to the
reference's own kernels (topk_rows, selector_lattice) where those are built; the product is held to the oracle."""
import ctypes as C

import numpy as np
import pytest

from oracle import lo

BIG, NONE = np.float32(-3.4028234663852886e38), 0x7FFFFFFF


def numpy_topk(x, k):
    vals, ids = np.full((x.shape[0], k), BIG, np.float32), np.full((x.shape[0], k), NONE, np.int32)
    for r in range(x.shape[0]):
        ok = np.flatnonzero(~np.isnan(x[r]) & (x[r] > BIG))
        order = ok[np.lexsort((ok, -x[r][ok].astype(np.float64)))][:k]
        vals[r, :len(order)], ids[r, :len(order)] = x[r][order], order
    return vals, ids


def logit_rows(rng, rows, V, ties=True):
    x = rng.standard_normal((rows, V)).astype(np.float32) * 3
    if ties:  # equal maxima far apart, a plateau of equal values across a segment boundary, NaN and infinities
        x[0, [5, V - 7, V // 2]] = 20.0
        x[1 % rows, 2040:2060] = 11.5
        x[2 % rows, 17] = np.nan
        x[2 % rows, 18] = -np.inf
        x[3 % rows, 99] = np.inf
    return x


def build_tree(lb, anchor, cand, scores, chain_tokens, chain_picks, nodes, temp=1.0, width=16, max_depth=1000, chain=1000):
    fn = lb.lib().ling_b200_build_tree
    fn.argtypes = [C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_float), C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int),
                   C.c_int, C.c_double, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int),
                   C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_double)]
    E = cand.shape[0]
    cand, scores = np.ascontiguousarray(cand, np.int32), np.ascontiguousarray(scores, np.float32)
    ct, cp = (C.c_int * E)(*chain_tokens), (C.c_int * E)(*chain_picks)
    par, dep, tok, pk, mass = (C.c_int * 64)(), (C.c_int * 64)(), (C.c_int * 64)(), (C.c_int * 64)(), C.c_double()
    r = fn(anchor, cand.ctypes.data_as(C.POINTER(C.c_int)), scores.ctypes.data_as(C.POINTER(C.c_float)), E, 16, ct, cp, nodes, temp,
           width, max_depth, chain, 32, par, dep, tok, pk, C.byref(mass))
    rows = r & 0xFFFF
    return {"rows": rows, "E": r >> 16, "parent": list(par)[:rows], "token": list(tok)[:rows]}


def selector_case(rng, E, V):
    hp = rng.standard_normal((E, 256)).astype(np.float32)
    cand = np.stack([rng.choice(V, 16, replace=False) for _ in range(E)]).astype(np.int32)
    unary = np.sort(rng.standard_normal((E, 16)).astype(np.float32) * 4)[:, ::-1].copy()
    P = (rng.standard_normal((V, 256)) * 0.2).astype(np.float32)
    S = (rng.standard_normal((V, 256)) * 0.2).astype(np.float32)
    return hp, cand, unary, P, S


# ---------------------------------------------------------------------------------------------- the oracle (CPU)
def test_oracle_topk_equals_a_sort():
    rng = np.random.default_rng(1)
    for rows, V, k in ((4, 5000, 16), (3, 300, 64), (2, 10, 16), (5, 4096, 1)):
        x = logit_rows(rng, rows, V, ties=V > 3000)
        vals, ids = lo.topk_rows(x, k)
        nv, ni = numpy_topk(x, k)
        assert np.array_equal(ids, ni) and np.array_equal(vals, nv)
    x = logit_rows(rng, 3, 4096)
    assert np.array_equal(lo.topk_rows(x, 1)[1][:, 0], lo.argmax(x)[0])


def test_oracle_selector_equals_numpy():
    rng = np.random.default_rng(2)
    hp, cand, unary, P, S = selector_case(rng, 5, 700)
    got = lo.selector_lattice(hp, cand, unary, P, S, anchor=33)
    bits = lambda a: ((a.view(np.uint32) + 0x7FFF + ((a.view(np.uint32) >> 16) & 1)) & 0xFFFF0000).view(np.float32)  # noqa: E731
    Pb, Sb = bits(P.copy()).astype(np.float64), bits(S.copy()).astype(np.float64)
    for e in range(5):
        pred = np.full(16, 33) if e == 0 else cand[e - 1]
        want = unary[e][None, :] + np.einsum("pr,r,cr->pc", Pb[pred], hp[e].astype(np.float64), Sb[cand[e]])
        assert np.allclose(got[e], want, rtol=0, atol=1e-5)
    x = rng.standard_normal((3, 512)).astype(np.float32)
    W = (rng.standard_normal((256, 512)) * 0.05).astype(np.float32)
    assert np.allclose(lo.selector_project(x, W), x.astype(np.float64) @ bits(W.copy()).astype(np.float64).T, atol=1e-5)


# ---------------------------------------------------------------------------------------------- the product (GPU)
@pytest.mark.gpu
@pytest.mark.parametrize("rows,V,k", [(15, 248320, 16), (4, 248320, 64), (3, 5000, 16), (2, 2048, 1), (1, 9, 16), (31, 4096, 16)])
def test_topk_rows_equals_oracle_bit_for_bit(gpu, lb, rows, V, k):
    rng = np.random.default_rng(rows * 1000 + k)
    x = logit_rows(rng, rows, V, ties=V > 3000)
    vals, ids = lb.topk_rows(x, k)
    ov, oi = lo.topk_rows(x, k)
    assert np.array_equal(ids, oi) and np.array_equal(vals, ov)
    R = lo.refcuda()
    if R is not None:  # the reference's own kernel on the same rows
        rv, ri = np.zeros((rows, k), np.float32), np.zeros((rows, k), np.int32)
        assert R.refcuda_topk(x.ctypes.data_as(C.POINTER(C.c_float)), rows, V, k, ri.ctypes.data_as(C.POINTER(C.c_int)),
                              rv.ctypes.data_as(C.POINTER(C.c_float))) == 0
        assert np.array_equal(ri, oi) and np.array_equal(rv, ov)


@pytest.mark.gpu
def test_topk_rows_rejects_bad_arguments(gpu, lb):
    x = np.zeros((2, 100), np.float32)
    for k in (0, 65):
        with pytest.raises(lb.LingError):
            lb.topk_rows(x, k)


@pytest.mark.gpu
@pytest.mark.parametrize("E,V", [(15, 4096), (1, 300), (31, 20000)])
def test_selector_lattice_matches_oracle_and_reference_kernel(gpu, lb, E, V):
    rng = np.random.default_rng(E + V)
    hp, cand, unary, P, S = selector_case(rng, E, V)
    anchor = int(rng.integers(V))
    want = lo.selector_lattice(hp, cand, unary, P, S, anchor)
    got, _ = lb.selector_lattice(cand, unary, lb.to_bf16_bits(P), lb.to_bf16_bits(S), anchor, hp=hp)
    scale = float(np.abs(want).max())
    assert np.abs(got - want).max() <= 2e-6 * scale + 1e-5  # fp32 sums of 256 products in another order
    R = lo.refcuda()
    if R is not None:
        ref = np.zeros((E, 16, 16), np.float32)
        f = lambda a: a.ctypes.data_as(C.POINTER(C.c_float))  # noqa: E731
        assert R.refcuda_selector_lattice(f(hp), cand.ctypes.data_as(C.POINTER(C.c_int)), f(unary), f(P), f(S), V, anchor, E, f(ref)) == 0
        assert np.abs(ref - want).max() <= 2e-6 * scale + 1e-5  # the oracle against the reference's own kernel
        assert np.abs(got - ref).max() <= 4e-6 * scale + 2e-5


@pytest.mark.gpu
def test_selector_projection_and_bad_candidates(gpu, lb):
    rng = np.random.default_rng(9)
    E, V, H = 7, 1000, 1024
    hp, cand, unary, P, S = selector_case(rng, E, V)
    x = rng.standard_normal((E, H)).astype(np.float32)
    W = (rng.standard_normal((256, H)) * 0.03).astype(np.float32)
    scores, hp_dev = lb.selector_lattice(cand, unary, lb.to_bf16_bits(P), lb.to_bf16_bits(S), 5, x=x, proj_bits=lb.to_bf16_bits(W))
    hp_or = lo.selector_project(x, W)
    assert np.abs(hp_dev - hp_or).max() <= 1e-5 * float(np.abs(hp_or).max()) + 1e-6
    want = lo.selector_lattice(hp_dev, cand, unary, P, S, 5)
    assert np.abs(scores - want).max() <= 2e-6 * float(np.abs(want).max()) + 1e-5
    bad = cand.copy()
    bad[3, 4] = 0x7FFFFFFF  # a list that was shorter than 16: reported, nothing read out of range
    with pytest.raises(lb.LingError):
        lb.selector_lattice(bad, unary, lb.to_bf16_bits(P), lb.to_bf16_bits(S), 5, hp=hp)
    lb.selector_lattice(cand, unary, lb.to_bf16_bits(P), lb.to_bf16_bits(S), 5, hp=hp)  # and the device is fine afterwards


@pytest.mark.gpu
def test_draft_head_on_a_context_feeds_build_tree_and_a_verify_step(gpu, lb):
    """Rows after the drafter's final norm -> candidates, unary logits, lattice scores; equal to the oracle's FP8 head, top 16
    and lattice; the tree built from them verifies like any other."""
    cfg = lb.toy_config()
    rng = np.random.default_rng(4)
    V, H, E = cfg.vocab, cfg.hidden, 7
    ctx = lb.Context(cfg, sessions=1, max_context=256, page_tokens=16, pool_pages=17, max_seqs=1, max_rows=32)
    ctx.synth_weights(0)
    head_w = (rng.standard_normal((V, H)) * 0.05).astype(np.float32)
    ctx.set_tensor(-1, lb.T_LM_HEAD, head_w)
    W = (rng.standard_normal((256, H)) * 0.05).astype(np.float32)
    P = (rng.standard_normal((V, 256)) * 0.2).astype(np.float32)
    S = (rng.standard_normal((V, 256)) * 0.2).astype(np.float32)
    head = lb.DraftHead(ctx, lb.to_bf16_bits(W), lb.to_bf16_bits(P), lb.to_bf16_bits(S))
    x = rng.standard_normal((E, H)).astype(np.float32)
    anchor = 123
    cand, unary, scores = head.run(x, anchor)
    # the oracle's FP8 GEMM on the same head weights
    logits = lo.gemm_fp8(x, head_w)
    ov, oi = lo.topk_rows(logits, 16)
    close = np.abs(unary - ov).max() <= 1e-4 * float(np.abs(logits).std()) + 1e-5
    assert close
    # the candidate sets agree wherever the 16th and 17th logits are further apart than the GEMMs' rounding
    top17 = lo.topk_rows(logits, 17)[0]
    clear = (top17[:, 15] - top17[:, 16]) > 1e-3 * float(np.abs(logits).std())
    assert clear.sum() >= E - 2
    for e in np.flatnonzero(clear):
        assert set(cand[e]) == set(oi[e])
    want = lo.selector_lattice(lo.selector_project(x, W), cand, unary, P, S, anchor)
    assert np.abs(scores - want).max() <= 1e-4 * float(np.abs(want).max()) + 1e-5
    # build_tree over the candidates and scores, then a verify step over the tree
    tree = build_tree(lb, anchor, cand, scores, [int(cand[e, 0]) for e in range(E)], [0] * E, nodes=8)
    assert tree["rows"] >= E + 1 and tree["parent"][0] == -1 and all(p < i for i, p in enumerate(tree["parent"]))
    assert tree["token"][0] == anchor and set(tree["token"][1:]) <= set(cand.reshape(-1).tolist())
    ctx.kv_table_set(0, np.arange(16, dtype=np.int32), np.arange(1, 17, dtype=np.int32))
    ctx.synth_kv(0, 64, 0), ctx.synth_state(0, 0)
    res = ctx.verify_step([dict(slot=0, pos=64, tokens=tree["token"], parent=tree["parent"], chain=tree["E"])], lb.STEP_COMMIT)
    assert res[0].status == 0 and 1 <= res[0].n_path <= tree["rows"]
    head.close()
    ctx.close()


# ---------------------------------------------------------------------------------------------- the sparse head
def key_to_float(keys):
    """The selection's order-preserving keys back to the fp32 scores (0 = marked: NaN here)."""
    k = keys.astype(np.uint32)
    bits = np.where(k & 0x80000000, k & 0x7FFFFFFF, ~k).astype(np.uint32)
    out = bits.view(np.float32).copy()
    out[k == 0] = np.nan
    return out


def sparse_case(rng, N, M, marked_share=0.02):
    p = (rng.standard_normal((M, 256)) * 0.7).astype(np.float32)
    us = (rng.standard_normal((N, 256)) * 0.1).astype(np.float32)
    mask = (rng.random(N) < marked_share).astype(np.uint8)
    return p, us, mask


def test_sparse_select_oracle_on_a_hand_case():
    # four rows of us against one row of p: scores 3, 1, 2, -1; row 3 is marked; the best one of the others is row 0
    p = np.zeros((1, 256), np.float32)
    p[0, 0] = 1.0
    us = np.zeros((4, 256), np.float32)
    us[:, 0] = [3, 1, 2, -1]
    mask = np.array([0, 0, 0, 1], np.uint8)
    rows, approx, marked = lo.sparse_select(p, us, mask, 1, 8)
    assert list(rows) == [0, 3] and list(approx) == [3, 1, 2, -1] and list(marked) == [False, False, False, True]
    assert list(lo.sparse_select(p, us, mask, 2, 8)[0]) == [0, 2, 3]
    assert list(lo.sparse_select(p, us, mask, 3, 8)[0]) == [0, 1, 2, 3]
    assert list(lo.sparse_select(p, us, mask, 4, 8)[0]) == [3]          # fewer unmarked rows than asked for: none of them
    assert list(lo.sparse_select(p, us, mask, 3, 2)[0]) == [0, 1]       # the capacity cuts the id-ordered list
    us[1, 0] = 2                                                        # a tie at the threshold: both taken
    assert list(lo.sparse_select(p, us, mask, 2, 8)[0]) == [0, 1, 2, 3]


@pytest.mark.gpu
@pytest.mark.parametrize("N,M,dynamic,cap", [(5000, 1, 300, 4096), (40000, 7, 2048, 8192), (248320, 15, 16384, 32768), (248320, 31, 16384, 20000),
                                             (3000, 9, 2990, 4096), (3000, 9, 0, 4096)])
def test_sparse_select_matches_oracle(gpu, lb, N, M, dynamic, cap):
    rng = np.random.default_rng(N + M)
    p, us, mask = sparse_case(rng, N, M)
    rows, keys = lb.sparse_select(p, lb.to_bf16_bits(us), mask, dynamic, cap)
    want, approx, marked = lo.sparse_select(p, us, mask, dynamic, cap)
    # the scores: BF16 products, fp32 sums in the tensor core against float64 sums
    got = key_to_float(keys)
    assert np.array_equal(np.isnan(got), marked)
    free = ~marked
    assert np.abs(got[free] - approx[free]).max() <= 2e-6 * float(np.abs(approx).max()) + 1e-6
    # the selection, exactly, on the keys the device ranked: the marked rows and every key at or above the dynamic-th largest
    take = marked.copy()
    fk = keys[free]
    if dynamic > 0 and free.sum() >= dynamic:
        take[np.flatnonzero(free)[fk >= np.sort(fk)[-dynamic]]] = True
    assert np.array_equal(rows, np.flatnonzero(take)[:cap])
    # and against the oracle's own selection: the same rows but for scores within the summation error of the threshold
    if dynamic > 0 and free.sum() >= dynamic:
        thr = np.sort(approx[free])[-dynamic]
        band = np.abs(approx - thr) <= 4e-6 * float(np.abs(approx).max())
        diff = np.setxor1d(rows, want) if len(rows) < cap and len(want) < cap else np.array([], np.int64)
        assert band[diff].all()
    else:
        assert np.array_equal(rows, want)


@pytest.mark.gpu
def test_sparse_select_matches_the_reference_kernel(gpu, lb):
    R = lo.refcuda()
    if R is None or not hasattr(R, "refcuda_sparse_select"):
        pytest.skip("the reference's CUDA kernels are not built here")
    f = lambda a: a.ctypes.data_as(C.POINTER(C.c_float))
    for N, M, dynamic, cap in [(40000, 7, 2048, 8192), (248320, 15, 16384, 32768), (3000, 9, 2990, 4096)]:
        rng = np.random.default_rng(N + M)
        p, us, mask = sparse_case(rng, N, M)
        rows, keys = lb.sparse_select(p, lb.to_bf16_bits(us), mask, dynamic, cap)
        ref, n = np.zeros(N, np.int32), C.c_int(0)
        assert R.refcuda_sparse_select(f(p), M, f(us), N, mask.ctypes.data_as(C.POINTER(C.c_ubyte)), dynamic, cap,
                                       ref.ctypes.data_as(C.POINTER(C.c_int)), C.byref(n)) == 0
        ref = ref[:n.value]
        # both sum the rank in a permuted order on the tensor core; a row within that error of the threshold may fall either way
        _, approx, marked = lo.sparse_select(p, us, mask, dynamic, cap)
        free = ~marked
        if free.sum() >= dynamic:
            thr = np.sort(approx[free])[-dynamic]
            band = np.abs(approx - thr) <= 4e-6 * float(np.abs(approx).max())
            assert band[np.setxor1d(rows, ref)].all(), (N, len(rows), len(ref))
        else:
            assert np.array_equal(rows, ref)


@pytest.mark.gpu
def test_sparse_draft_head_scores_the_full_heads_bits(gpu, lb):
    """The sparse head on a context: the rows it scores are the session's mask plus the factors' choice; the logits of its 16
    candidates are bit for bit the full head's, and where the full head's top 16 lie inside the selection the candidates are
    the same."""
    cfg = lb.toy_config()
    rng = np.random.default_rng(14)
    V, H, E = cfg.vocab, cfg.hidden, 7
    ctx = lb.Context(cfg, sessions=2, max_context=256, page_tokens=16, pool_pages=17, max_seqs=1, max_rows=32)
    ctx.synth_weights(0)
    # a head with a low-rank part that the factors reproduce, plus noise they do not
    A, B = (rng.standard_normal((V, 256)) * 0.05).astype(np.float32), (rng.standard_normal((256, H)) * 0.3).astype(np.float32)
    head_w = (A @ B + rng.standard_normal((V, H)) * 0.01).astype(np.float32)
    ctx.set_tensor(-1, lb.T_LM_HEAD, head_w)
    W = (rng.standard_normal((256, H)) * 0.05).astype(np.float32)
    P = (rng.standard_normal((V, 256)) * 0.2).astype(np.float32)
    S = (rng.standard_normal((V, 256)) * 0.2).astype(np.float32)
    head = lb.DraftHead(ctx, lb.to_bf16_bits(W), lb.to_bf16_bits(P), lb.to_bf16_bits(S))
    dynamic, cap = 512, 1024
    head.enable_sparse(lb.to_bf16_bits(A), lb.to_bf16_bits(B), dynamic, cap)
    fixed = rng.choice(V, 200, replace=False).astype(np.int32)
    head.mask_reset(1, fixed)
    head.mask_mark(1, np.array([3, 5, 7], np.int32))
    x = rng.standard_normal((E, H)).astype(np.float32)
    anchor = 77
    full_c, full_u, full_s = head.run(x, anchor)
    cand, unary, scores, sel = head.run_sparse(1, x, anchor)
    marked = np.zeros(V, np.uint8)
    marked[fixed] = 1
    marked[[3, 5, 7]] = 1
    # the rows scored: the kernel-level selection on p = x . B^T (the projection kernel's own output differs from numpy's in
    # the last bits, so rows within that error of the threshold may differ: the band of the oracle test)
    want, approx, _ = lo.sparse_select(lo.selector_project(x, B), A, marked, dynamic, cap)
    assert set(np.flatnonzero(marked)) <= set(sel) and np.all(np.diff(sel) > 0) and len(sel) <= cap
    free = marked == 0
    thr = np.sort(approx[free])[-dynamic]
    band = np.abs(approx - thr) <= 1e-4 * float(np.abs(approx).max())
    assert band[np.setxor1d(sel, want)].all()
    # every candidate is a scored row, and its logit is the full head's bits for that row
    full_logits = np.full((E, V), np.nan, np.float32)
    for e in range(E):
        full_logits[e, full_c[e]] = full_u[e]
        assert set(cand[e]) <= set(sel)
        both = np.intersect1d(cand[e], full_c[e])
        assert len(both) > 0
        for t in both:
            assert unary[e][list(cand[e]).index(t)] == full_u[e][list(full_c[e]).index(t)]
        if set(full_c[e]) <= set(sel):      # the full head's top 16 all inside the selection: the same list, the same scores
            assert np.array_equal(cand[e], full_c[e]) and np.array_equal(unary[e], full_u[e])
            assert np.array_equal(scores[e], full_s[e]) or e == 0 or not set(full_c[e - 1]) <= set(sel)
    inside = sum(set(full_c[e]) <= set(sel) for e in range(E))
    print("sparse head: %d rows scored of %d; the full head's top 16 inside the selection for %d of %d positions" % (len(sel), V, inside, E))
    assert inside >= 1
    # another session's mask is its own (empty): only the dynamic rows
    _, _, _, sel0 = head.run_sparse(0, x, anchor)
    assert abs(len(sel0) - dynamic) <= 2 and not set(np.flatnonzero(marked)) <= set(sel0)
    head.close()
    ctx.close()
