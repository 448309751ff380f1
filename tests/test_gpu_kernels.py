"""Kernel-level parity on the GPU, through the C ABI: the tcgen05 block-scaled FP8 GEMM, the DeltaNet tree replay and
commit, and the argmax, each against the CPU oracle on the same seeded inputs.  Modelled on the reference's model-free
kernel tests (tests/stream_tests.cu, tests/tree_tests.cu in the reference project): a loose comparison with a host
reference plus bit-exact invariants (row invariance across M)."""
import ctypes as C

import numpy as np
import pytest

import helpers

pytestmark = pytest.mark.gpu

# GEMM tolerance: both sides multiply the same E4M3 codes; the only differences are fp32 accumulation order inside the
# tensor core and the order of the 128-wide block sums, so the bar is tight: 1e-4 of the row's rms plus 1e-5 relative.
GEMM_RTOL, GEMM_ATOL_RMS = 1e-5, 1e-4


def close_rows(y, ref, rtol, atol_rms):
    rms = np.sqrt((ref.astype(np.float64) ** 2).mean(axis=1, keepdims=True)) + 1e-30
    return bool((np.abs(y - ref) <= rtol * np.abs(ref) + atol_rms * rms).all())


SHAPES = [(24, 256, 256), (80, 1408, 256), (80, 256, 704), (1, 128, 128), (33, 640, 256), (100, 512, 512), (130, 256, 384),
          (7, 384, 1152), (24, 2048, 5120), (24, 640, 17408), (74, 1024, 6144)]


@pytest.mark.parametrize("impl", [0, 1])
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_matches_oracle(gpu, lb, lo, impl, M, N, K):
    rng = np.random.default_rng(M * 131 + N * 17 + K)
    x = rng.standard_normal((M, K)).astype(np.float32) * np.exp(rng.standard_normal((M, 1))).astype(np.float32)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    x[0, :min(K, 128)] = 0.0                       # an all-zero activation block (scale 1)
    ref = lo.gemm_fp8(x, w)
    y = lb.gemm_fp8(x, w, impl=impl)
    assert close_rows(y, ref, GEMM_RTOL, GEMM_ATOL_RMS), float(np.abs(y - ref).max())


def test_gemm_rows_are_invariant_to_the_row_count(gpu, lb):
    # the reference's central invariant (src/core/stream_gemm.cu:10-13): a row's result is bit for bit the same whatever
    # M is and whoever its batch-mates are, including across the token-tile sizes 32, 64, 96 and 128
    rng = np.random.default_rng(9)
    K, N = 1024, 768
    x = rng.standard_normal((128, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    full = lb.gemm_fp8(x, w, impl=0, splits=3)
    for M in (1, 24, 33, 80, 97):
        part = lb.gemm_fp8(x[:M], w, impl=0, splits=3)
        assert np.array_equal(part, full[:M]), M
    two_tiles = lb.gemm_fp8(np.concatenate([x, x[:40]]), w, impl=0, splits=3)
    assert np.array_equal(two_tiles[:128], full) and np.array_equal(two_tiles[128:], full[:40])


def test_gemm_k_split_changes_only_the_summation_order(gpu, lb, lo):
    rng = np.random.default_rng(10)
    x = rng.standard_normal((24, 2048)).astype(np.float32)
    w = (rng.standard_normal((256, 2048)) * 0.02).astype(np.float32)
    ref = lo.gemm_fp8(x, w)
    for splits in (1, 2, 4, 16):
        assert close_rows(lb.gemm_fp8(x, w, impl=0, splits=splits), ref, GEMM_RTOL, GEMM_ATOL_RMS)


def test_weight_and_activation_quantizers_are_bit_exact(gpu, lb, lo):
    # the product quantizes on the device, the oracle on the host: same codes, same scales
    cfg = lb.toy_config()
    ctx = lb.Context(cfg)
    opt = lb.Options(4, 2048, 16, 512, 4, 128, 0, 0, 0, 0, 0)
    m = lo.Model(cfg, opt, lb)
    helpers.load_weights_from_host(lb, lo, cfg, 0, [ctx, m])
    for layer, tensor, rows, cols in [(0, lb.T_GATE, 704, 256), (0, lb.T_UP, 704, 256), (0, lb.T_DOWN, 256, 704),
                                      (1, lb.T_IN_QKV, 512, 256), (1, lb.T_IN_Z, 256, 256), (2, lb.T_OUT, 256, 256),
                                      (3, lb.T_Q, 512, 256), (3, lb.T_K, 64, 256), (3, lb.T_V, 64, 256), (3, lb.T_O, 256, 256),
                                      (-1, lb.T_LM_HEAD, 4096, 256)]:
        a, b = ctx.get_matrix(layer, tensor, rows, cols), m.get_matrix(layer, tensor, rows, cols)
        assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1]), (layer, tensor)
    ctx.close(), m.close()


def test_device_generator_matches_host_generator(gpu, lb, lo):
    cfg = lb.toy_config()
    a, b = lb.Context(cfg), lb.Context(cfg)
    opt = lb.Options(4, 2048, 16, 512, 4, 128, 0, 0, 0, 0, 0)
    m = lo.Model(cfg, opt, lb)
    a.synth_weights(5)
    helpers.load_weights_from_host(lb, lo, cfg, 5, [b])
    m.synth_weights(5)
    for layer, tensor, rows, cols in [(0, lb.T_GATE, 704, 256), (0, lb.T_DOWN, 256, 704), (3, lb.T_Q, 512, 256),
                                      (-1, lb.T_LM_HEAD, 4096, 256)]:
        x, y, z = (t.get_matrix(layer, tensor, rows, cols) for t in (a, b, m))
        assert np.array_equal(x[0], y[0]) and np.array_equal(x[1], y[1]) and np.array_equal(x[0], z[0])
    # synthetic KV and state: device fill == host fill
    for t in (a, m):
        helpers.map_pages([t], 1, 100, 16, 7)
        t.synth_kv(1, 100, 11)
        t.synth_state(1, 11)
    for x, y in zip(a.kv_read(1, 0, 0, 100, codes=True), m.kv_read(1, 0, 0, 100, codes=True)):
        assert np.array_equal(x, y)
    for g in range(3):
        for x, y in zip(a.state_read(1, g), m.state_read(1, g)):
            assert np.array_equal(x, y)
    assert a.state_hash(1) == m.state_hash(1)
    a.close(), b.close(), m.close()


# DeltaNet tolerance: fp32 FMA chains on the device against double accumulation in the oracle, over up to 17 dependent
# steps: 2e-4 of the tensor's rms.
GDN_TOL = 2e-4


def gdn_inputs(rng, Hk, HV, Dk, Dv, n):
    Cn = 2 * Hk * Dk + HV * Dv
    return dict(pre=rng.standard_normal((n, Cn)).astype(np.float32), convw=(rng.standard_normal((Cn, 4)) * 0.3).astype(np.float32),
                g=np.log(1.0 / (1.0 + np.exp(-rng.standard_normal((n, HV))))).astype(np.float32),   # alpha = sigmoid(N(0,1))
                beta=(1.0 / (1.0 + np.exp(-rng.standard_normal((n, HV))))).astype(np.float32),
                state=(rng.standard_normal((HV, Dk, Dv)) * 0.1).astype(np.float32),
                conv=rng.standard_normal((Cn, 3)).astype(np.float32))


def fp(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


@pytest.mark.parametrize("Hk,HV,Dk,Dv", [(2, 4, 64, 64), (4, 12, 128, 128)])
@pytest.mark.parametrize("shape", ["two_branch", "chain", "random", "single"])
def test_gdn_tree_and_commit_match_oracle(gpu, lb, lo, Hk, HV, Dk, Dv, shape):
    rng = np.random.default_rng(Dk + len(shape))
    if shape == "two_branch":
        parent, chain = helpers.chain_plus_branch(16, 4), 15
    elif shape == "chain":
        parent, chain = helpers.chain_plus_branch(12, 0), 11
    elif shape == "single":
        parent, chain = [-1], 0
    else:
        parent, chain = helpers.random_tree(rng, 24, 7), 7
    n = len(parent)
    rc, td = lb.describe_tree(parent, chain)
    assert rc == 0
    d = gdn_inputs(rng, Hk, HV, Dk, Dv, n)
    d["convw"] = np.array([lo.lo().lo_bf16_round(float(v)) for v in d["convw"].ravel()], np.float32).reshape(d["convw"].shape)
    Cn, Vs = d["pre"].shape[1], HV * Dv
    post_o, core_o = np.zeros((n, Cn), np.float32), np.zeros((n, Vs), np.float32)
    lo.lo().lo_gdn_tree(Hk, HV, Dk, Dv, C.byref(td), fp(d["pre"]), fp(d["convw"]), fp(d["g"]), fp(d["beta"]), fp(d["state"]),
                        fp(d["conv"]), fp(post_o), fp(core_o))
    post_g, core_g = np.zeros_like(post_o), np.zeros_like(core_o)
    lb.check(lb.lib().ling_b200_gdn_tree_host(0, Hk, HV, Dk, Dv, C.byref(td), fp(d["pre"]), fp(d["convw"]), fp(d["g"]),
                                              fp(d["beta"]), fp(d["state"]), fp(d["conv"]), fp(post_g), fp(core_g)), "gdn_tree_host")
    # the device's `post` carries q and k already L2-normalized per head (q also times 1/sqrt(Dk)); v is the raw conv output
    post_n = post_o.copy()
    for h in range(2 * Hk):
        seg = post_o[:, h * Dk:(h + 1) * Dk].astype(np.float64)
        scale = 1.0 / np.sqrt((seg ** 2).sum(axis=1, keepdims=True) + 1e-6) / (np.sqrt(Dk) if h < Hk else 1.0)
        post_n[:, h * Dk:(h + 1) * Dk] = (seg * scale).astype(np.float32)
    assert np.abs(post_g - post_n).max() <= 1e-5 * max(1.0, np.abs(post_n).max())
    assert np.abs(core_g - core_o).max() <= GDN_TOL * np.sqrt((core_o ** 2).mean())
    # commit of an accepted path: the rows of variant 0's path up to a random length
    path = [td.path[td.nvar - 1][j] for j in range(td.depth[[r for r in range(n) if td.var[r] == td.nvar - 1][-1]] + 1)]
    path = path[:int(rng.integers(1, len(path) + 1))]
    pa = np.array(path, np.int32)
    so, wo = d["state"].copy(), d["conv"].copy()
    lo.lo().lo_gdn_commit(Hk, HV, Dk, Dv, pa.ctypes.data_as(C.POINTER(C.c_int)), len(path), n, fp(d["pre"]), fp(post_o), fp(d["g"]),
                          fp(d["beta"]), fp(so), fp(wo))
    sg, wg = d["state"].copy(), d["conv"].copy()
    lb.check(lb.lib().ling_b200_gdn_commit_host(0, Hk, HV, Dk, Dv, pa.ctypes.data_as(C.POINTER(C.c_int)), len(path), n,
                                                fp(d["pre"]), fp(post_g), fp(d["g"]), fp(d["beta"]), fp(sg), fp(wg)), "gdn_commit_host")
    assert np.array_equal(wg, wo)                                  # the window is a copy: bit-exact
    assert np.abs(sg - so).max() <= GDN_TOL * np.sqrt((so ** 2).mean())


def test_argmax_ties_nan_and_inf(gpu, lb, lo):
    # ties to the lower id, NaN skipped, inf kept, a row without a candidate comes back as (-FLT_MAX, 0x7fffffff)
    # (src/core/topk.cu:19,58 in the reference project); on the 248,320-token vocabulary like tests/stream_tests.cu:728-757
    rng = np.random.default_rng(12)
    V = 248320
    logits = rng.standard_normal((6, V)).astype(np.float32)
    logits[0, [5, 77777, 200000]] = 9.0
    logits[1, :] = np.nan
    logits[2, 1000] = np.nan
    logits[2, 123456] = np.inf
    logits[3, :] = -np.inf
    logits[4, V - 1] = 50.0
    logits[5, :] = 1.25
    ids, vals = np.zeros(6, np.int32), np.zeros(6, np.float32)
    lb.check(lb.lib().ling_b200_argmax_host(0, fp(logits), 6, V, ids.ctypes.data_as(C.POINTER(C.c_int)), fp(vals)), "argmax_host")
    oi, ov = lo.argmax(logits)
    assert np.array_equal(ids, oi) and np.array_equal(vals, ov)
    assert list(ids[:2]) == [5, 0x7fffffff] and ids[2] == 123456 and ids[4] == V - 1 and ids[5] == 0


# Attention tolerance: both sides read the same E4M3 cache; the device rounds q and the probabilities to FP16 for the
# tensor-core products (relative 2^-11 each) where the oracle keeps fp32/double: 6e-3 of a row's rms (measured: 3e-3).
ATTN_TOL = 6e-3


# impl 0: the tcgen05/TMEM kernel (the product path); impl 1: the mma.sync kernel kept as its cross-check
@pytest.mark.parametrize("impl", [0, 1])
@pytest.mark.parametrize("shape", ["toy", "toy64", "27b"])
def test_tree_attention_matches_oracle(gpu, lb, lo, shape, impl):
    if shape == "toy":     # 4 q heads / 1 kv head of 64, 16-position pages
        cfg = lb.make_config(256, 704, 1, 4096, 4, 1, 64, 16, 2, 4, 64, 64, [1])
        contexts, page_tokens = (0, 3, 37, 511, 512, 1029), 16
    elif shape == "toy64":  # 64 sequences: more work items than one wave of CTAs, so the step keeps the 512-key chunks
        cfg = lb.make_config(256, 704, 1, 4096, 4, 1, 64, 16, 2, 4, 64, 64, [1])   # (two 256-key sub-chunks per chunk,
        contexts = tuple(int(c) for c in np.random.default_rng(64).integers(520, 1900, 64))  # rows rescaled in between);
        contexts, page_tokens = contexts[:60] + (0, 511, 512, 513), 16             # the other shapes run on 256-key chunks
    else:                  # 24 q heads / 4 kv heads of 256 (six query heads per kv head), 64-position pages
        cfg = lb.make_config(5120, 128, 1, 4096, 24, 4, 256, 64, 16, 48, 128, 128, [1])
        contexts, page_tokens = (1500, 17, 530), 64
    n_seq = len(contexts)
    pool = sum((c + 48) // page_tokens + 2 for c in contexts) + 1
    ctx = lb.Context(cfg, sessions=n_seq, max_context=2048, page_tokens=page_tokens, pool_pages=pool, max_seqs=n_seq,
                     max_rows=32 * n_seq, gemm_impl=impl)
    opt = lb.Options(n_seq, 2048, page_tokens, pool, n_seq, 32 * n_seq, 0, 0, 0, 0, 0)
    m = lo.Model(cfg, opt, lb)
    rng = np.random.default_rng(len(shape))
    seqs, page = [], 1
    for s, c in enumerate(contexts):
        n = int(rng.integers(1, 33)) if s else 32
        chain = int(rng.integers(0, n))
        seqs.append({"slot": s, "pos": c, "tokens": np.zeros(n, np.int32), "parent": np.array(helpers.random_tree(rng, n, chain), np.int32),
                     "chain": chain})
        page += helpers.map_pages([ctx, m], s, c + 32, page_tokens, page)
        for t in (ctx, m):
            if c:
                t.synth_kv(s, c, 5)
            # the in-flight rows' K and V, as the step's prepare kernel would have left them
            k = rng.standard_normal((n, cfg.kv_heads, cfg.head_dim)).astype(np.float32) if t is ctx else k
            v = (rng.standard_normal((n, cfg.kv_heads, cfg.head_dim)) * 3).astype(np.float32) if t is ctx else v
            t.kv_write(s, 0, c, k, v)
    for a, b in zip(ctx.kv_read(n_seq - 1, 0, 0, contexts[-1] + 5), m.kv_read(n_seq - 1, 0, 0, contexts[-1] + 5)):
        assert np.array_equal(a, b)        # the two caches hold the same values (the V page layout differs, the content does not)
    rows = sum(len(q["tokens"]) for q in seqs)
    q = rng.standard_normal((rows, cfg.heads, cfg.head_dim)).astype(np.float32)
    out_o = m.attention(seqs, 0, q, make_steps=lb.make_steps)
    out_g = ctx.attention(seqs, 0, q)
    flat_o, flat_g = out_o.reshape(rows, -1), out_g.reshape(rows, -1)
    rms = np.sqrt((flat_o.astype(np.float64) ** 2).mean(axis=1, keepdims=True))
    assert np.isfinite(out_g).all()
    assert (np.abs(flat_g - flat_o) <= ATTN_TOL * rms).all(), float((np.abs(flat_g - flat_o) / rms).max())
    ctx.close(), m.close()


# ---------------------------------------------------------------------------------------------- the fused DeltaNet kernel
def bf16_round(a):
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    return ((u + 0x7fff + ((u >> 16) & 1)) & 0xffff0000).astype(np.uint32).view(np.float32)


def decode_fp8(lo, codes, scales):
    """codes [rows][K] and scales [rows][K/128] back to fp32."""
    return lo.e4m3_decode_table()[codes] * np.repeat(scales, 128, axis=1)[:, :codes.shape[1]]


@pytest.mark.parametrize("pdl", [0, 1])
@pytest.mark.parametrize("Hk,HV,Dk,Dv", [(2, 4, 64, 64), (16, 48, 128, 128)])
@pytest.mark.parametrize("shape", ["two_branch", "random", "single", "full32", "three_sequences"])
def test_fused_deltanet_kernel_matches_oracle(gpu, lb, lo, Hk, HV, Dk, Dv, shape, pdl):
    # the kernel the 27B-class step launches between the in and the out projection (conv over the trees, q/k normalization,
    # the delta rule along every DeltaNet path, gated RMSNorm, FP8 copy), alone on identical inputs; with dependent launch
    # on it also loads its first item's state before the packing kernel ahead of it has completed and re-checks the choice
    rng = np.random.default_rng(Dk + len(shape) + 7 * pdl)
    if shape == "two_branch":
        trees = [(helpers.chain_plus_branch(16, 8), 15)]
    elif shape == "random":
        trees = [(helpers.random_tree(rng, 24, 7), 7)]
    elif shape == "single":
        trees = [([-1], 0)]
    elif shape == "full32":
        trees = [(helpers.random_tree(rng, 32, 11), 11)]
    else:
        trees = [(helpers.chain_plus_branch(12, 5), 11), (helpers.random_tree(rng, 9, 3), 3), ([-1], 0)]
    rows, n_seqs = sum(len(p) for p, _ in trees), len(trees)
    Cn, Vs = 2 * Hk * Dk + HV * Dv, HV * Dv
    d = gdn_inputs(rng, Hk, HV, Dk, Dv, rows)
    convw = bf16_round(d["convw"])
    inp = np.concatenate([d["pre"], rng.standard_normal((rows, Vs)).astype(np.float32)], axis=1)
    state = (rng.standard_normal((n_seqs, HV, Dk, Dv)) * 0.1).astype(np.float32)
    conv = rng.standard_normal((n_seqs, Cn, 3)).astype(np.float32)
    norm_w = bf16_round(1.0 + rng.standard_normal(Dv).astype(np.float32) * 0.02)
    eps = 1e-6
    lb.lib().ling_b200_set_pdl(pdl)
    try:
        pre_g, post_g, core_g, codes_g, scales_g = lb.gdn_fused(Hk, HV, Dk, Dv, trees, inp, convw, d["g"], d["beta"], state, conv,
                                                                norm_w, eps)
    finally:
        lb.lib().ling_b200_set_pdl(0)
    # the oracle, sequence by sequence
    post_o, core_o = np.zeros((rows, Cn), np.float32), np.zeros((rows, Vs), np.float32)
    r0 = 0
    for s, (parent, chain) in enumerate(trees):
        n = len(parent)
        rc, td = lb.describe_tree(parent, chain)
        assert rc == 0
        po, co = np.zeros((n, Cn), np.float32), np.zeros((n, Vs), np.float32)
        sl = slice(r0, r0 + n)
        lo.lo().lo_gdn_tree(Hk, HV, Dk, Dv, C.byref(td), fp(np.ascontiguousarray(d["pre"][sl])), fp(convw),
                            fp(np.ascontiguousarray(d["g"][sl])), fp(np.ascontiguousarray(d["beta"][sl])),
                            fp(np.ascontiguousarray(state[s])), fp(np.ascontiguousarray(conv[s])), fp(po), fp(co))
        post_o[sl], core_o[sl] = po, co
        r0 += n
    assert np.array_equal(pre_g, d["pre"])                         # the raw inputs kept for the commit: a copy
    post_n = post_o.copy()                                         # the device's q and k are already L2-normalized
    for h in range(2 * Hk):
        seg = post_o[:, h * Dk:(h + 1) * Dk].astype(np.float64)
        scale = 1.0 / np.sqrt((seg ** 2).sum(axis=1, keepdims=True) + 1e-6) / (np.sqrt(Dk) if h < Hk else 1.0)
        post_n[:, h * Dk:(h + 1) * Dk] = (seg * scale).astype(np.float32)
    assert np.abs(post_g - post_n).max() <= 1e-5 * max(1.0, np.abs(post_n).max())
    assert np.abs(core_g - core_o).max() <= GDN_TOL * np.sqrt((core_o ** 2).mean())
    # gated RMSNorm with the plain weight times silu(z), then the FP8 copy (one scale per row per 128 columns)
    z = inp[:, Cn:].astype(np.float64)
    co = core_o.astype(np.float64).reshape(rows, HV, Dv)
    normed = (co / np.sqrt((co ** 2).mean(axis=2, keepdims=True) + eps) * norm_w.astype(np.float64)).reshape(rows, Vs)
    normed = (normed * z / (1.0 + np.exp(-z))).astype(np.float32)
    codes_o, scales_o = lo.quant_rows(normed)
    assert np.allclose(scales_g, scales_o, rtol=1e-4, atol=1e-30)
    deq_g, deq_o = decode_fp8(lo, codes_g, scales_g), decode_fp8(lo, codes_o, scales_o)
    flipped = codes_g != codes_o
    assert flipped.mean() <= 2e-3, float(flipped.mean())         # fp32-vs-double differences that straddle a rounding boundary
    step = np.maximum(np.abs(deq_o), np.repeat(scales_o, 128, axis=1)) * 0.13   # one E4M3 step is at most 12.5% of the value
    assert (np.abs(deq_g - deq_o) <= step + 1e-6).all()
    rms = np.sqrt((normed.astype(np.float64) ** 2).mean(axis=1, keepdims=True)) + 1e-30
    assert np.median(np.abs(deq_g - deq_o).max(axis=1) / rms[:, 0]) <= 0.07


# ---------------------------------------------------------------------------------------------- attn_prepare
def test_attn_prepare_matches_oracle_at_large_positions(gpu, lb, lo):
    # the prepare kernel alone (head norms with (1 + w), rotation of the first 64 of 256 dims, K and V into the paged FP8
    # cache) at positions 0 .. 131000 against the oracle's norm_rope / kv_store.  The rotation angle is position x
    # theta^(-2i/rot); the device evaluates the power with powf (as the reference's kernel does, attention_body.cuh:87-93),
    # the oracle with a correctly rounded pow, so the angles may differ by an ulp or two of position x inv_freq: the bar on the
    # rotated dims grows with the position (two ulp of the largest angle; measured against the reference's own kernel, which
    # uses the same powf: 3.7e-3 of a row's largest value at position 131000), the unrotated dims are held to FP16 rounding.
    cfg = lb.make_config(5120, 128, 1, 4096, 24, 4, 256, 64, 16, 48, 128, 128, [1])
    positions, page_tokens = (0, 1529, 8192, 60000, 131000), 16
    n_seq, max_ctx = len(positions), 131072 + 64
    ctx = lb.Context(cfg, sessions=n_seq, max_context=max_ctx, page_tokens=page_tokens, pool_pages=64, max_seqs=n_seq,
                     max_rows=32 * n_seq)
    opt = lb.Options(n_seq, max_ctx, page_tokens, 64, n_seq, 32 * n_seq, 0, 0, 0, 0, 0)
    m = lo.Model(cfg, opt, lb)
    ctx.synth_weights(2), m.synth_weights(2)
    rng = np.random.default_rng(21)
    seqs, page = [], 1
    for s, pos in enumerate(positions):
        n = (32, 24, 9, 17, 32)[s]
        chain = int(rng.integers(0, n))
        seqs.append({"slot": s, "pos": pos, "tokens": np.zeros(n, np.int32), "parent": np.array(helpers.random_tree(rng, n, chain), np.int32),
                     "chain": chain, "rope_delta": (0, 0, -5, 0, 0)[s]})
        idx = np.arange(pos // page_tokens, (pos + n - 1) // page_tokens + 1, dtype=np.int32)   # only the pages the rows land in
        pages = np.arange(page, page + len(idx), dtype=np.int32)
        page += len(idx)
        for t in (ctx, m):
            t.kv_table_set(s, idx, pages)
    rows = sum(len(q["tokens"]) for q in seqs)
    W = cfg.heads * 2 * cfg.head_dim + 2 * cfg.kv_heads * cfg.head_dim
    qkv = (rng.standard_normal((rows, W)) * np.exp(rng.standard_normal((rows, 1)))).astype(np.float32)
    q_o, k_o = m.attn_prepare(seqs, 0, qkv, make_steps=lb.make_steps)
    q_g = ctx.attn_prepare(seqs, 0, qkv)
    pk = ctx.read_packing()
    assert np.array_equal(pk["rope_pos"], m.read_packing()["rope_pos"])
    rot, ulp = cfg.rotary_dim, 2.0 ** -23
    for r in range(rows):
        # per row: the unrotated dims at FP16 precision (q is kept as FP16 for the tensor-core product) ...
        amax = np.abs(q_o[r]).max()
        assert np.abs(q_g[r, :, rot:] - q_o[r, :, rot:]).max() <= 2.0 ** -10 * amax + 1e-5
        # ... the rotated ones with the angle's uncertainty on top
        ang_tol = 2 * ulp * max(1.0, abs(float(pk["rope_pos"][r])))
        assert np.abs(q_g[r, :, :rot] - q_o[r, :, :rot]).max() <= (2.0 ** -10 + ang_tol) * amax * 1.5 + 1e-5, (r, int(pk["rope_pos"][r]))
    flips_k = total = 0
    for s, q in enumerate(seqs):
        n = len(q["tokens"])
        kc_g, ks_g, vc_g, vs_g = ctx.kv_read(s, 0, q["pos"], n, codes=True)
        kc_o, ks_o, vc_o, vs_o = m.kv_read(s, 0, q["pos"], n, codes=True)
        assert np.array_equal(vc_g, vc_o) and np.array_equal(vs_g, vs_o)      # V is stored raw: bit-exact
        assert np.allclose(ks_g, ks_o, rtol=1e-4 + 2 * ulp * max(1, q["pos"]))
        flips_k += int((kc_g != kc_o).sum())
        total += kc_o.size
        dec = lo.e4m3_decode_table()
        kg, ko = dec[kc_g] * ks_g[..., None], dec[kc_o] * ks_o[..., None]
        assert np.abs(kg - ko).max() <= 0.13 * np.abs(ko).max()              # a flipped code is one FP8 step
        if q["pos"] <= 8192:
            assert (kc_g != kc_o).mean() <= 2e-3
    assert flips_k / total <= 0.05, flips_k / total
    ctx.close(), m.close()


# ---------------------------------------------------------------------------------------------- attention: the reference's matrix
@pytest.mark.parametrize("page_tokens", [16, 64])
def test_tree_attention_at_the_reference_matrix_of_contexts(gpu, lb, lo, page_tokens):
    # contexts x rows of the reference's paged attention test (tests/paged_tests.cu:183-196: contexts around the page and
    # range boundaries and up to 131072, rows 1..32), at the 27B head shape (24 q / 4 kv heads of 256): every context is one
    # sequence of the same call, its tree a random one of the given size.  Hundreds of flash-decoding chunks per row at the
    # long end, the page window across chunk boundaries, both page sizes.
    cfg = lb.make_config(5120, 128, 1, 4096, 24, 4, 256, 64, 16, 48, 128, 128, [1])
    contexts = (1, 33, 63, 64, 65, 127, 4095, 4096, 4097, 8192, 27000, 60000, 131008)
    row_counts = (1, 12, 24, 32)
    n_seq, max_ctx = len(contexts), 131072 + 64
    pool = sum((c + 32 + page_tokens - 1) // page_tokens for c in contexts) + 1
    ctx = lb.Context(cfg, sessions=n_seq, max_context=max_ctx, page_tokens=page_tokens, pool_pages=pool, max_seqs=n_seq,
                     max_rows=32 * n_seq)
    opt = lb.Options(n_seq, max_ctx, page_tokens, pool, n_seq, 32 * n_seq, 0, 0, 0, 0, 0)
    m = lo.Model(cfg, opt, lb)
    lo.lo().lo_set_threads(16)
    rng = np.random.default_rng(100 + page_tokens)
    seqs, page = [], 1
    for s, c in enumerate(contexts):
        n = row_counts[(s + 1) % 4]
        chain = int(rng.integers(0, n))
        seqs.append({"slot": s, "pos": c, "tokens": np.zeros(n, np.int32), "parent": np.array(helpers.random_tree(rng, n, chain), np.int32),
                     "chain": chain})
        page += helpers.map_pages([ctx, m], s, c + 32, page_tokens, page)
        k = rng.standard_normal((n, cfg.kv_heads, cfg.head_dim)).astype(np.float32)
        v = (rng.standard_normal((n, cfg.kv_heads, cfg.head_dim)) * 3).astype(np.float32)
        for t in (ctx, m):
            t.synth_kv(s, c, 9)
            t.kv_write(s, 0, c, k, v)
    rows = sum(len(q["tokens"]) for q in seqs)
    q = rng.standard_normal((rows, cfg.heads, cfg.head_dim)).astype(np.float32)
    out_o = m.attention(seqs, 0, q, make_steps=lb.make_steps).reshape(rows, -1)
    out_g = ctx.attention(seqs, 0, q).reshape(rows, -1)
    rms = np.sqrt((out_o.astype(np.float64) ** 2).mean(axis=1, keepdims=True))
    err = np.abs(out_g - out_o) / rms
    assert np.isfinite(out_g).all()
    row0 = np.cumsum([0] + [len(q_["tokens"]) for q_ in seqs])
    worst = {contexts[s]: float(err[row0[s]:row0[s + 1]].max()) for s in range(n_seq)}
    assert err.max() <= ATTN_TOL, worst
    lo.lo().lo_set_threads(1)
    ctx.close(), m.close()


@pytest.mark.parametrize("shape,pos0,M", [("toy", 0, 100), ("toy", 37, 200), ("27b", 0, 70), ("27b", 530, 96)])
def test_prefill_attention_in_slices_matches_oracle(gpu, lb, lo, shape, pos0, M):
    # A prefill chunk's rows through the step's prepare / attention / combine kernels in slices of 32 query rows (several
    # slices per launch), against the oracle taking the slices one at a time through its own prepare and attention: every row
    # sees the cache up to itself, the rows of earlier slices included.  The output gate is applied in numpy on the oracle's side.
    if shape == "toy":
        cfg = lb.make_config(256, 704, 1, 4096, 4, 1, 64, 16, 2, 4, 64, 64, [1])
        page_tokens = 16
    else:
        cfg = lb.make_config(5120, 128, 1, 4096, 24, 4, 256, 64, 16, 48, 128, 128, [1])
        page_tokens = 64
    pool = (pos0 + M) // page_tokens + 3
    ctx = lb.Context(cfg, sessions=1, max_context=1024, page_tokens=page_tokens, pool_pages=pool, max_seqs=4, max_rows=128)
    opt = lb.Options(1, 1024, page_tokens, pool, 4, 128, 0, 0, 0, 0, 0)
    m = lo.Model(cfg, opt, lb)
    ctx.synth_weights(3), m.synth_weights(3)
    helpers.map_pages([ctx, m], 0, pos0 + M, page_tokens, 1)
    if pos0:
        ctx.synth_kv(0, pos0, 7), m.synth_kv(0, pos0, 7)
    rng = np.random.default_rng(pos0 + M)
    D, Hq, Hkv = cfg.head_dim, cfg.heads, cfg.kv_heads
    W = Hq * 2 * D + 2 * Hkv * D
    qkv = (rng.standard_normal((M, W)) * np.exp(0.5 * rng.standard_normal((M, 1)))).astype(np.float32)
    out = ctx.prefill_attention(0, 0, pos0, qkv)
    want = np.zeros_like(out)
    for r0 in range(0, M, 32):
        n = min(32, M - r0)
        seq = [{"slot": 0, "pos": pos0 + r0, "tokens": np.zeros(n, np.int32), "parent": np.arange(-1, n - 1, dtype=np.int32), "chain": n - 1}]
        q_o, _ = m.attn_prepare(seq, 0, qkv[r0:r0 + n], make_steps=lb.make_steps)
        o = m.attention(seq, 0, q_o, make_steps=lb.make_steps)
        gate = qkv[r0:r0 + n, :Hq * 2 * D].reshape(n, Hq, 2 * D)[:, :, D:]
        want[r0:r0 + n] = o / (1.0 + np.exp(-gate.astype(np.float64)))
    flat_o, flat_g = want.reshape(M, -1), out.reshape(M, -1)
    rms = np.sqrt((flat_o.astype(np.float64) ** 2).mean(axis=1, keepdims=True))
    assert np.isfinite(out).all()
    assert (np.abs(flat_g - flat_o) <= 2 * ATTN_TOL * rms).all(), float((np.abs(flat_g - flat_o) / rms).max())
    # the cache holds the chunk's keys and values as a verify step's prepare would have left them
    for a, b in zip(ctx.kv_read(0, 0, 0, pos0 + M), m.kv_read(0, 0, 0, pos0 + M)):
        assert np.abs(a - b).max() <= 0.13 * np.abs(b).max()  # FP8 codes may differ by a step where the norm's last bit differs
    ctx.close(), m.close()


def chunk_layer_errors(lb, ctx, m, layer, pos0, h):
    """Row errors of what a full-attention layer's chunk mixer adds to the residual rows h, device against the oracle's mixer
    taking the 32-row chains one at a time (session 0)."""
    M = h.shape[0]
    got = ctx.chunk_attention_layer(0, layer, pos0, h)
    want = np.zeros_like(h)
    for r0 in range(0, M, 32):
        n = min(32, M - r0)
        seq = [{"slot": 0, "pos": pos0 + r0, "tokens": np.zeros(n, np.int32), "parent": np.arange(-1, n - 1, dtype=np.int32), "chain": n - 1}]
        want[r0:r0 + n] = m.mixer_forward(seq, layer, h[r0:r0 + n], make_steps=lb.make_steps)
    assert np.isfinite(got).all()
    d_got, d_want = got - h, want - h
    rms = np.sqrt((d_want.astype(np.float64) ** 2).mean(axis=1, keepdims=True))
    assert (rms > 0).all()
    return np.sqrt(((d_got - d_want).astype(np.float64) ** 2).mean(axis=1, keepdims=True)) / rms


@pytest.mark.parametrize("pos0,M", [(0, 100), (37, 150)])
def test_chunk_attention_layer_matches_oracle(gpu, lb, lo, pos0, M):
    # A full-attention layer's mixer over a prefill chunk's residual rows (norm, FP8 q|k|v projection, prepare, attention, gate,
    # FP8 o projection, residual add) through the step's kernels, several 32-row chains of the session per launch, against the
    # oracle's mixer taking the chains one at a time.  Bars on what the mixer added, row by row against its rms: the o
    # projection's FP8 input rounds a last-bit difference of the attention output to the next code now and then.
    cfg = lb.make_config(256, 704, 1, 4096, 4, 1, 64, 16, 2, 4, 64, 64, [1])
    page_tokens = 16
    pool = (pos0 + M) // page_tokens + 3
    ctx = lb.Context(cfg, sessions=1, max_context=1024, page_tokens=page_tokens, pool_pages=pool, max_seqs=4, max_rows=128)
    opt = lb.Options(1, 1024, page_tokens, pool, 4, 128, 0, 0, 0, 0, 0)
    m = lo.Model(cfg, opt, lb)
    ctx.synth_weights(3), m.synth_weights(3)
    helpers.map_pages([ctx, m], 0, pos0 + M, page_tokens, 1)
    if pos0:
        ctx.synth_kv(0, pos0, 7), m.synth_kv(0, pos0, 7)
    rng = np.random.default_rng(pos0 + M)
    h = (rng.standard_normal((M, cfg.hidden)) * np.exp(0.5 * rng.standard_normal((M, 1)))).astype(np.float32)
    err = chunk_layer_errors(lb, ctx, m, 0, pos0, h)
    assert err.max() <= 2e-2 and np.median(err) <= 5e-3, (float(err.max()), float(np.median(err)))
    with pytest.raises(lb.LingError):   # the chunk's chains are not a staged step: a launch without staging again is refused
        ctx.launch()
    ctx.close(), m.close()


def test_sibling_context_works_beside_a_staged_step(gpu, lb):
    # a sibling context (own step buffers on the parent's weights, pages and state slots) runs a chunk's attention layer while the
    # parent keeps a verify step staged: the parent's step is untouched and replays to the same result, and the sibling's output is
    # bit for bit what the parent computes for the same rows
    cfg = lb.toy_config()
    ctx = lb.Context(cfg, sessions=5, max_context=2048, page_tokens=16, pool_pages=400, max_seqs=4, max_rows=128, debug_rows=128)
    ctx.synth_weights(2)
    rng = np.random.default_rng(21)
    seqs = helpers.toy_sequences(rng, cfg.vocab)
    page = helpers.setup_sessions([ctx], cfg, seqs, 16, 0)
    ctx.stage(seqs, lb.STEP_KEEP_LOGITS)
    ctx.launch()
    first, logits = ctx.fetch(), ctx.read_logits()
    sib = ctx.sibling(4, 128)
    M, layer = 100, 3
    helpers.map_pages([ctx], 4, M, 16, page)
    h = rng.standard_normal((M, cfg.hidden)).astype(np.float32)
    out_sib = sib.chunk_attention_layer(4, layer, 0, h)
    ctx.launch()    # still staged: the sibling staged its chains in its own buffers
    again = ctx.fetch()
    for a, b in zip(first, again):
        assert a.status == b.status == 0 and a.n_path == b.n_path and a.next_token == b.next_token
    assert np.array_equal(ctx.read_logits(), logits)
    out_par = ctx.chunk_attention_layer(4, layer, 0, h)
    assert np.isfinite(out_sib).all() and np.array_equal(out_sib, out_par)
    with pytest.raises(lb.LingError):
        sib.synth_weights(3)    # a sibling takes no weight uploads
    sib.close(), ctx.close()
