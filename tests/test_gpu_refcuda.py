"""The reference's OWN CUDA kernels, built for sm_100a from its sources (oracle/_ref/libling_refcuda.so, `make -C oracle
ref_cuda`), as the second oracle: on the same seeded tensors the CPU oracle's fp32 math and the product's kernels are
compared with what the reference computes on the same GPU.  Covered: the DeltaNet conv over trees, the gating, the
tree recurrence, the gated RMSNorm, the commit (conv window + state), attn_prepare (head norms + rotation, before the
cache rounding), the rows-path attention (BF16 cache in the reference, FP8 here: run on values both formats hold
exactly) and top-1.  These paths are fp32 on both sides and do not involve this build's FP8 numerics, so the bars are
tight.  What stays defined by the CPU oracle alone: the FP8 KV rounding, the 1x128 block-scaled FP8 weights and
activations, the GEMMs (the reference's rows-path GEMM does not build for sm_100a).

The reference's kernels exist for its 27B shapes only (DeltaNet dims 128, attention head dim 256, six query heads per
KV head, one sequence of at most 32 rows per call).  Skipped where the reference library was not built."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

import helpers
from test_gpu_kernels import bf16_round, fp, gdn_inputs

pytestmark = pytest.mark.gpu

REF_GDN_TOL = 5e-5    # DeltaNet recurrence and commit against the reference's kernels, of the tensor's rms
REF_ATTN_TOL = 5e-3   # attention against the reference's BF16 kernel, of a row's rms (measured 8e-4 .. 1.6e-3)


@pytest.fixture(scope="module")
def rc(gpu, lo):
    L = lo.refcuda()
    if L is None:
        pytest.skip("the reference's CUDA kernels were not built (make -C oracle ref_cuda REF=...)")
    return L


def ok(L, rc_):
    assert rc_ == 0, L.refcuda_last_error().decode()


def rel_rms(a, b):
    return float(np.abs(a.astype(np.float64) - b).max() / (np.sqrt((b.astype(np.float64) ** 2).mean()) + 1e-30))


def test_the_reference_tree_test_program_passes_on_this_gpu(gpu, lo):
    # tests/tree_tests.cu of the reference as it stands: its tree kernels equal its chain kernels by memcmp
    if not os.path.exists(lo.REF_TREE_TESTS):
        pytest.skip("the reference's tree test program was not built")
    r = subprocess.run([lo.REF_TREE_TESTS], capture_output=True, text=True, timeout=600)
    print(r.stdout[-800:])
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.parametrize("Hk,HV", [(4, 12), (16, 48)])
@pytest.mark.parametrize("shape", ["two_branch", "random", "single", "full32"])
def test_deltanet_tree_and_commit_against_the_reference_kernels(rc, lb, lo, Hk, HV, shape):
    Dk = Dv = 128
    rng = np.random.default_rng(HV + len(shape))
    if shape == "two_branch":
        parent, chain = helpers.chain_plus_branch(16, 8), 15
    elif shape == "random":
        parent, chain = helpers.random_tree(rng, 24, 7), 7
    elif shape == "single":
        parent, chain = [-1], 0
    else:
        parent, chain = helpers.random_tree(rng, 32, 11), 11
    n = len(parent)
    rcode, td = lb.describe_tree(parent, chain)
    assert rcode == 0 and rc.refcuda_tree_desc_bytes() == C.sizeof(td)
    d = gdn_inputs(rng, Hk, HV, Dk, Dv, n)
    d["convw"] = bf16_round(d["convw"])
    Cn, Vs = d["pre"].shape[1], HV * Dv
    post_r, core_r = np.zeros((n, Cn), np.float32), np.zeros((n, Vs), np.float32)
    ok(rc, rc.refcuda_gdn_tree(Hk, HV, C.byref(td), fp(d["pre"]), fp(d["convw"]), fp(d["g"]), fp(d["beta"]), fp(d["state"]), fp(d["conv"]),
                               fp(post_r), fp(core_r)))
    post_o, core_o = np.zeros_like(post_r), np.zeros_like(core_r)
    lo.lo().lo_gdn_tree(Hk, HV, Dk, Dv, C.byref(td), fp(d["pre"]), fp(d["convw"]), fp(d["g"]), fp(d["beta"]), fp(d["state"]),
                        fp(d["conv"]), fp(post_o), fp(core_o))
    # the product's fused kernel on the same inputs (z and the norm weight do not reach `core`)
    inp = np.concatenate([d["pre"], np.zeros((n, Vs), np.float32)], axis=1)
    _, _, core_g, _, _ = lb.gdn_fused(Hk, HV, Dk, Dv, [(parent, chain)], inp, d["convw"], d["g"], d["beta"], d["state"][None],
                                      d["conv"][None], np.ones(Dv, np.float32))
    e_conv, e_or, e_gr = rel_rms(post_o, post_r), rel_rms(core_o, core_r), rel_rms(core_g, core_r)
    print("conv+SiLU oracle vs reference %.1e; recurrence: oracle vs reference %.1e, product vs reference %.1e" % (e_conv, e_or, e_gr))
    assert e_conv <= 1e-5           # conv + SiLU: fp32 on both sides (the reference's __expf against the oracle's exp)
    assert e_or <= REF_GDN_TOL and e_gr <= REF_GDN_TOL   # up to 32 dependent fp32 steps (measured: 2e-6 .. 9e-6)
    # commit of the accepted path (rows of the last variant up to a random length)
    last = td.nvar - 1
    leaf = [r for r in range(n) if td.var[r] == last][-1]
    path = [td.path[last][j] for j in range(td.depth[leaf] + 1)][:int(rng.integers(1, td.depth[leaf] + 2))]
    pa = np.array(path, np.int32)
    so, wo = d["state"].copy(), d["conv"].copy()
    lo.lo().lo_gdn_commit(Hk, HV, Dk, Dv, pa.ctypes.data_as(C.POINTER(C.c_int)), len(path), n, fp(d["pre"]), fp(post_o), fp(d["g"]),
                          fp(d["beta"]), fp(so), fp(wo))
    sr, wr = d["state"].copy(), d["conv"].copy()
    take = lambda a: np.ascontiguousarray(a[path])   # noqa: E731  the reference commits the compacted rows (tree_gather first)
    ok(rc, rc.refcuda_gdn_commit(Hk, HV, len(path), fp(take(d["pre"])), fp(take(post_r)), fp(take(d["g"])), fp(take(d["beta"])),
                                 fp(d["convw"]), fp(sr), fp(wr)))
    assert np.array_equal(wr, wo)                # the window is a copy of raw inputs: bit-exact
    assert rel_rms(so, sr) <= REF_GDN_TOL, rel_rms(so, sr)


def test_gating_and_gated_norm_against_the_reference_kernels(rc, lo):
    rng = np.random.default_rng(5)
    M, HV, D = 24, 48, 128
    a, b = (rng.standard_normal((M, HV)) * 3).astype(np.float32), (rng.standard_normal((M, HV)) * 3).astype(np.float32)
    a[0, 0] = 25.0     # past the softplus switch at 20
    A_log, dt_bias = bf16_round(rng.standard_normal(HV) * 0.5), bf16_round(rng.standard_normal(HV) * 0.5)
    g, beta = np.zeros((M, HV), np.float32), np.zeros((M, HV), np.float32)
    ok(rc, rc.refcuda_gdn_gating(fp(a), fp(b), fp(A_log), fp(dt_bias), fp(g), fp(beta), M, HV))
    x = a.astype(np.float64) + dt_bias
    g_o = -np.exp(A_log.astype(np.float64)) * np.where(x <= 20.0, np.log1p(np.exp(x)), x)   # the oracle's formula (layer_forward)
    beta_o = 1.0 / (1.0 + np.exp(-b.astype(np.float64)))
    assert np.abs(g - g_o).max() <= 2e-6 * np.abs(g_o).max() and np.abs(beta - beta_o).max() <= 2e-6
    xs, z = rng.standard_normal((M * HV, D)).astype(np.float32), rng.standard_normal((M * HV, D)).astype(np.float32)
    w = bf16_round(1.0 + rng.standard_normal(D) * 0.02)
    out = np.zeros_like(xs)
    ok(rc, rc.refcuda_gated_rmsnorm(fp(xs), fp(z), fp(w), fp(out), M * HV, D, C.c_float(1e-6)))
    x64, z64 = xs.astype(np.float64), z.astype(np.float64)
    out_o = x64 / np.sqrt((x64 ** 2).mean(axis=1, keepdims=True) + 1e-6) * w * (z64 / (1.0 + np.exp(-z64)))
    assert np.abs(out - out_o).max() <= 1e-5 * np.abs(out_o).max()


@pytest.fixture(scope="module")
def attn_model(gpu, lb, lo):
    cfg = lb.make_config(5120, 128, 1, 4096, 24, 4, 256, 64, 16, 48, 128, 128, [1])
    kw = dict(sessions=1, max_context=131072 + 64, page_tokens=16, pool_pages=1100, max_seqs=1, max_rows=32)
    ctx = lb.Context(cfg, **kw)
    m = lo.Model(cfg, lb.Options(1, kw["max_context"], 16, 1100, 1, 32, 0, 0, 0, 0, 0), lb)
    ctx.synth_weights(2), m.synth_weights(2)
    rng = np.random.default_rng(77)
    qn, kn = bf16_round(rng.standard_normal(256) * 0.02), bf16_round(rng.standard_normal(256) * 0.02)
    for t in (ctx, m):
        t.set_tensor(0, lb.T_Q_NORM, qn), t.set_tensor(0, lb.T_K_NORM, kn)
    yield cfg, ctx, m, qn, kn
    ctx.close(), m.close()


@pytest.mark.parametrize("pos,rdelta", [(0, 0), (1529, 0), (8192, -7), (60000, 0), (131000, 0)])
def test_attn_prepare_against_the_reference_kernel(rc, lb, lo, attn_model, pos, rdelta):
    cfg, ctx, m, qn, kn = attn_model
    rng = np.random.default_rng(pos + 3)
    n = 24
    parent, chain = helpers.chain_plus_branch(16, 8), 15
    rcode, td = lb.describe_tree(parent, chain)
    seq = {"slot": 0, "pos": pos, "rope_delta": rdelta, "tokens": np.zeros(n, np.int32), "parent": np.array(parent, np.int32), "chain": chain}
    idx = np.arange(pos // 16, (pos + n - 1) // 16 + 1, dtype=np.int32)
    for t in (ctx, m):
        t.kv_table_set(0, idx, np.arange(1, 1 + len(idx), dtype=np.int32))
    Hq, Hkv, D = cfg.heads, cfg.kv_heads, cfg.head_dim
    qkv = (rng.standard_normal((n, Hq * 2 * D + 2 * Hkv * D)) * np.exp(rng.standard_normal((n, 1)))).astype(np.float32)
    q_gate = np.ascontiguousarray(qkv[:, :Hq * 2 * D])
    k_in = np.ascontiguousarray(qkv[:, Hq * 2 * D:Hq * 2 * D + Hkv * D])
    v_in = np.ascontiguousarray(qkv[:, Hq * 2 * D + Hkv * D:])
    q_r, gate_r = np.zeros((n, Hq, D), np.float32), np.zeros((n, Hq, D), np.float32)
    k_r, v_r = np.zeros((n, Hkv, D), np.float32), np.zeros((n, Hkv, D), np.float32)
    ok(rc, rc.refcuda_attn_prepare(fp(q_gate), fp(k_in), fp(v_in), fp(qn), fp(kn), pos, rdelta, n, Hq, Hkv, D, cfg.rotary_dim,
                                   C.c_float(cfg.rope_theta), C.c_float(cfg.eps), C.byref(td), fp(q_r), fp(gate_r), fp(k_r), fp(v_r)))
    q_o, k_o = m.attn_prepare([seq], 0, qkv, make_steps=lb.make_steps)
    q_g = ctx.attn_prepare([seq], 0, qkv)
    amax = np.abs(q_o).max(axis=(1, 2), keepdims=True)
    # product vs reference: the same formulas with the same device functions (powf, sincosf); the product keeps q as FP16
    e_gr = float((np.abs(q_g - q_r) / amax).max())
    # oracle vs reference: a correctly rounded pow on the host against powf on the device moves the angle by a few ulp of
    # position x inv_freq (the unrotated dims carry no such term)
    ang = 2.0 ** -23 * max(1, pos + 32)
    e_or_plain = float((np.abs(q_o - q_r)[:, :, cfg.rotary_dim:] / amax).max())
    e_or_rot = float((np.abs(q_o - q_r)[:, :, :cfg.rotary_dim] / amax).max())
    print("position %6d: q product vs reference %.1e; oracle vs reference: unrotated dims %.1e, rotated dims %.1e (angle bar %.1e)"
          % (pos, e_gr, e_or_plain, e_or_rot, ang))
    assert e_gr <= 2.0 ** -10 + 1e-6
    assert e_or_plain <= 1e-5 and e_or_rot <= 1e-5 + ang      # measured: 3.7e-3 at position 131000 against a bar of 1.6e-2
    assert np.array_equal(gate_r, q_gate.reshape(n, Hq, 2, D)[:, :, 1])               # the gate half is passed through
    assert np.array_equal(v_r, bf16_round(v_in).reshape(n, Hkv, D))                   # V raw, rounded to the reference's BF16 cache
    k_bar = 2.0 ** -8 * np.abs(k_o).max() + ang * np.abs(k_o).max()             # one BF16 rounding of the reference's cache
    assert np.abs(k_r - k_o).max() <= k_bar


@pytest.mark.parametrize("pos,n", [(1500, 24), (4097, 32), (8192, 24)])
def test_attention_against_the_reference_kernel_on_values_both_caches_hold_exactly(rc, lb, lo, attn_model, pos, n):
    # The reference keeps K and V in BF16, this build in E4M3 with a per-position scale.  Values of the form (E4M3 code) x
    # 2^-7 with every (position, head) vector's largest magnitude 448 x 2^-7 are exact in both: the FP8 cache stores
    # the codes with scale 2^-7, the BF16 cache the products.  Both kernels then see the same K and V, and differ in how
    # they round q and the probabilities (BF16 in the reference, FP16 here) against the oracle's fp32/double.
    cfg, ctx, m, _, _ = attn_model
    rng = np.random.default_rng(pos)
    Hq, Hkv, D = cfg.heads, cfg.kv_heads, cfg.head_dim
    dec = lo.e4m3_decode_table()
    parent, chain = (helpers.chain_plus_branch(16, 8), 15) if n == 24 else (helpers.random_tree(rng, n, 9), 9)
    rcode, td = lb.describe_tree(parent, chain)

    def exact_values(count):
        codes = rng.integers(0, 0x58, (count, Hkv, D)).astype(np.uint8) | (rng.integers(0, 2, (count, Hkv, D)).astype(np.uint8) << 7)
        codes[:, :, 0] = 0x7e                                   # 448: fixes the vector's scale at exactly 2^-7
        return (dec[codes] * np.float32(2.0 ** -7)).astype(np.float32)

    kc, vc = exact_values(pos + n), exact_values(pos + n)
    seq = {"slot": 0, "pos": pos, "tokens": np.zeros(n, np.int32), "parent": np.array(parent, np.int32), "chain": chain}
    for t in (ctx, m):
        helpers.map_pages([t], 0, pos + 32, 16, 1)
        t.kv_write(0, 0, 0, kc, vc)
    for a, b in zip(ctx.kv_read(0, 0, 0, pos + n), (kc, vc)):
        assert np.array_equal(a, b)                             # the FP8 cache holds exactly these values
    q = rng.standard_normal((n, Hq, D)).astype(np.float32)
    out_r = np.zeros_like(q)
    ok(rc, rc.refcuda_attention_rows(fp(q), fp(kc), fp(vc), pos, n, Hq, Hkv, D, C.byref(td), fp(out_r)))
    out_o = m.attention([seq], 0, q, make_steps=lb.make_steps)
    out_g = ctx.attention([seq], 0, q)
    rms = np.sqrt((out_o.astype(np.float64) ** 2).mean(axis=(1, 2), keepdims=True))
    e_ro, e_go, e_gr = (float((np.abs(a - b) / rms).max()) for a, b in ((out_r, out_o), (out_g, out_o), (out_g, out_r)))
    print("context %5d, %2d rows: reference vs oracle %.1e, product vs oracle %.1e, product vs reference %.1e (of a row's rms)"
          % (pos, n, e_ro, e_go, e_gr))
    assert e_go <= 6e-3          # the product's bar (FP16 q and probabilities)
    assert e_ro <= REF_ATTN_TOL  # BF16 q and probabilities in the reference (its own test's bar is 2e-2 absolute)
    assert e_gr <= REF_ATTN_TOL


def test_top1_against_the_reference_kernel(rc, lb, lo):
    rng = np.random.default_rng(12)
    V = 248320
    logits = rng.standard_normal((6, V)).astype(np.float32)
    logits[0, [5, 77777, 200000]] = 9.0
    logits[2, 1000] = np.nan
    logits[2, 123456] = np.inf
    logits[4, V - 1] = 50.0
    logits[5, :] = 1.25
    ids_r, vals_r = np.zeros(6, np.int32), np.zeros(6, np.float32)
    ok(rc, rc.refcuda_top1(fp(logits), 6, V, ids_r.ctypes.data_as(C.POINTER(C.c_int)), fp(vals_r)))
    ids_o, vals_o = lo.argmax(logits)
    ids_g, vals_g = np.zeros(6, np.int32), np.zeros(6, np.float32)
    lb.check(lb.lib().ling_b200_argmax_host(0, fp(logits), 6, V, ids_g.ctypes.data_as(C.POINTER(C.c_int)), fp(vals_g)), "argmax_host")
    assert np.array_equal(ids_r, ids_o) and np.array_equal(vals_r, vals_o)
    assert np.array_equal(ids_g, ids_r) and np.array_equal(vals_g, vals_r)
