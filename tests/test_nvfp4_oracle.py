"""The oracle's NVFP4 arithmetic on the CPU: the weight rounding against golden vectors recorded from the reference's own
quantize_nvfp4 (tests/golden/nvfp4_weight.json) and, where the reference was built here, against that function directly on
fresh inputs; the activation recipe and the E2M1 rounding against a written-out numpy statement of the rule the reference's
test states (tests/prefill_tests.cu:44-85 of the reference project); the GEMM against numpy in float64."""
import json
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "nvfp4_weight.json")
E2M1 = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6], np.float32)


def bf16_bits(x):
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_round(x):
    return (bf16_bits(x).astype(np.uint32) << 16).view(np.float32)


def e2m1_rne(v):
    """E2M1 codes of an fp32 array: nearest, ties to the even code, saturating; the sign bit is kept for values that round to 0."""
    a = np.abs(v).astype(np.float32)
    mags = E2M1[:8]
    d = np.abs(a[..., None] - mags)
    best = np.zeros(a.shape, np.int64)
    for i in range(1, 8):
        db = np.take_along_axis(d, best[..., None], -1)[..., 0]
        better = (d[..., i] < db) | ((d[..., i] == db) & (i % 2 == 0))
        best = np.where(better, i, best)
    best = np.where(a > 6, 7, best)
    return (best | (np.signbit(v) * 8)).astype(np.uint8)


def unpack(q):
    """[rows][K/2] bytes -> [rows][K] codes (low nibble first)."""
    return np.stack([q & 15, q >> 4], -1).reshape(q.shape[0], -1)


def test_weight_rounding_matches_the_reference_golden_vectors(lo):
    golden = json.load(open(GOLDEN))
    assert len(golden) >= 7
    for case in golden:
        N, K = case["N"], case["K"]
        w = np.array(case["w_bf16"], np.uint16).reshape(N, K)
        q, sf, s2 = lo.nvfp4_quantize_weight(w)
        assert q.ravel().tolist() == case["values"], case["name"]
        assert sf.ravel().tolist() == case["scales"], case["name"]
        assert int(np.float32(s2).view(np.uint32)) == case["scale2_bits"], case["name"]


def test_golden_midpoints_take_the_smaller_magnitude():
    case = next(c for c in json.load(open(GOLDEN)) if c["name"] == "midpoints")
    codes = unpack(np.array(case["values"], np.uint8).reshape(case["N"], case["K"] // 2))
    # every row holds midpoints 0.25 .. 5 (and their negatives) of its block scale: codes 0,1,2,3,4,5,6 then 7 for the maximum
    want = [0, 1, 2, 3, 4, 5, 6, 7, 0, 9, 10, 11, 12, 13, 14, 0]
    for r in range(1, case["N"]):
        assert codes[r, :16].tolist() == want
    assert np.float32(np.array(case["scale2_bits"], np.uint32).view(np.float32)) == 1.0


def test_weight_rounding_matches_the_reference_on_fresh_inputs(lo):
    if lo.refquant() is None:
        pytest.skip("the reference's quantize_nvfp4 was not built here (make -C oracle ref_quant REF=...)")
    rng = np.random.default_rng(5)
    for N, K, std in [(96, 512, 0.02), (33, 5120, 0.02), (7, 48, 3.0)]:
        w = (rng.standard_normal((N, K)) * std).astype(np.float32)
        w[rng.random((N, K)) < 0.005] *= 25
        bits = bf16_bits(w)
        a, b = lo.nvfp4_quantize_weight(bits), lo.nvfp4_quantize_weight(bits, use_reference=True)
        assert (a[0] == b[0]).all() and (a[1] == b[1]).all() and a[2] == b[2]


def test_activation_recipe(lo):
    rng = np.random.default_rng(6)
    M, K, in_scale = 67, 512, 0.0019763766
    x = (rng.standard_normal((M, K)) * 0.003).astype(np.float32)
    x.ravel()[::97] *= 40
    x[3, 16:32] = 0          # an all-zero block: scale 0, codes 0
    x[4, :16] = -1e-30       # negative values that round to zero keep their sign bit
    dec = lo.e4m3_decode_table()
    q, sf = lo.nvfp4_quant_act(x, in_scale)
    g = np.float32(1) / np.float32(in_scale)
    v = bf16_round(x).reshape(M, K // 16, 16)
    amax = np.abs(v).max(-1)
    want_sf = np.array([[lo.lo().lo_e4m3_encode(float(np.float32(g * np.float32(a * np.float32(1.0 / 6.0))))) for a in row] for row in amax], np.uint8)
    assert (sf == want_sf).all()
    sv = dec[want_sf]
    with np.errstate(divide="ignore"):
        os_ = np.where(sv != 0, np.float32(1) / (sv * (np.float32(1) / g)), np.float32(0)).astype(np.float32)
    codes = e2m1_rne((v * os_[..., None]).astype(np.float32)).reshape(M, K)
    assert (unpack(q) == codes).all()
    assert (unpack(q)[3, 16:32] == 0).all() and sf[3, 1] == 0
    assert (unpack(q)[4, :16] == 8).all()
    # silu(x) * up fused = the plain recipe on the product computed in fp32
    up = rng.standard_normal((M, K)).astype(np.float32)
    prod = (x / (np.float32(1) + np.exp(-x, dtype=np.float32))).astype(np.float32) * up
    q2, sf2 = lo.nvfp4_quant_act(x, in_scale, up=up)
    q3, sf3 = lo.nvfp4_quant_act(prod, in_scale)
    assert (q2 != q3).mean() < 1e-3 and (sf2 != sf3).mean() < 1e-3   # expf rounding may move a value across a boundary


def test_e2m1_ties_go_to_the_even_code(lo):
    # one block: amax 6 under gscale 1 gives scale 1; the other values sit on midpoints
    x = np.array([[0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, 7.5]], np.float32)
    x[0, 15] = 6.0
    q, sf = lo.nvfp4_quant_act(x, 1.0)
    assert sf[0, 0] == 0x38   # E4M3 code of 1.0
    assert unpack(q)[0].tolist() == [0, 2, 2, 4, 4, 6, 6, 7, 8, 10, 10, 12, 12, 14, 14, 7]


def test_gemm_and_dequant(lo):
    rng = np.random.default_rng(7)
    M, N, K = 9, 24, 64
    xq, wq = rng.integers(0, 256, (M, K // 2), np.uint8), rng.integers(0, 256, (N, K // 2), np.uint8)
    xs, ws = rng.integers(0x28, 0x41, (M, K // 16), np.uint8), rng.integers(0x28, 0x41, (N, K // 16), np.uint8)
    dec = lo.e4m3_decode_table()
    xa = E2M1[unpack(xq)].astype(np.float64) * np.repeat(dec[xs], 16, axis=1)
    wa = E2M1[unpack(wq)].astype(np.float64) * np.repeat(dec[ws], 16, axis=1)
    assert np.array_equal(lo.nvfp4_dequant(xq, xs).astype(np.float64), xa)
    y0 = rng.standard_normal((M, N + 8)).astype(np.float32)
    want = y0.astype(np.float64).copy()
    want[:, :N] += 0.37 * (xa @ wa.T)
    got = lo.nvfp4_gemm(xq, xs, wq, ws, 0.37, y=y0, ldy=N + 8, accumulate=True)
    assert np.array_equal(got[:, N:], y0[:, N:])
    assert np.abs(got - want).max() <= 1e-6 * np.abs(want).max()
    plain = lo.nvfp4_gemm(xq, xs, wq, ws, 0.37)
    assert np.abs(plain - 0.37 * (xa @ wa.T)).max() <= 1e-6 * np.abs(want).max()


def test_entry_points_refuse_bad_shapes_before_touching_a_device(lb):
    """Argument errors come back as LING_B200_ERR_ARG with nothing launched: N and K must be multiples of 128 (the
    reference's rule, prefill_gemm.cu:596), K of 16 for the quantizers, scales positive; M = 0 is an empty success."""
    import ctypes as C
    L = lb.lib()
    b = (C.c_ubyte * 64)()
    f = (C.c_float * 64)()
    h = (C.c_uint16 * 64)()
    s2 = C.c_float()
    assert L.ling_b200_quantize_nvfp4_host(0, h, 2, 24, b, b, C.byref(s2)) == lb.ERR_ARG          # K % 16
    assert L.ling_b200_quant_act_nvfp4_host(0, f, None, 1, 40, C.c_float(1.0), b, b) == lb.ERR_ARG
    assert L.ling_b200_quant_act_nvfp4_host(0, f, None, 1, 32, C.c_float(0.0), b, b) == lb.ERR_ARG  # input_scale
    assert L.ling_b200_rmsnorm_quant_nvfp4_host(0, f, h, None, 1, 24, C.c_float(1e-6), C.c_float(1.0), b, b) == lb.ERR_ARG
    gemm = L.ling_b200_prefill_gemm_nvfp4_host
    assert gemm(0, b, b, 1, b, b, C.c_float(1.0), f, 192, 192, 128, 0) == lb.ERR_ARG      # N % 128
    assert gemm(0, b, b, 1, b, b, C.c_float(1.0), f, 128, 128, 192, 0) == lb.ERR_ARG      # K % 128
    assert gemm(0, b, b, 1, b, b, C.c_float(1.0), f, 64, 128, 128, 0) == lb.ERR_ARG       # ldy < N
    assert gemm(0, b, b, 0, b, b, C.c_float(1.0), f, 128, 128, 128, 0) == lb.OK           # no rows: nothing to do
    sw = L.ling_b200_prefill_swiglu_nvfp4_host
    assert sw(0, b, b, 1, b, b, C.c_float(1.0), b, b, C.c_float(1.0), 100, 128, C.c_float(1.0), b, b) == lb.ERR_ARG
    assert sw(0, b, b, 1, b, b, C.c_float(1.0), b, b, C.c_float(1.0), 128, 128, C.c_float(0.0), b, b) == lb.ERR_ARG
    out = C.c_void_p()
    L.ling_b200_nvfp4_ffn_create.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_uint64, C.POINTER(C.c_void_p)]
    assert L.ling_b200_nvfp4_ffn_create(0, 1, 100, 512, 8, 0, C.byref(out)) == lb.ERR_ARG   # hidden % 256
    assert L.ling_b200_nvfp4_ffn_create(0, 0, 256, 512, 8, 0, C.byref(out)) == lb.ERR_ARG   # no layers
    tf = C.c_float()
    assert L.ling_b200_fp4_tensor_peak(0, 0, 0, C.byref(tf), None) == lb.ERR_ARG
    assert L.ling_b200_fp4_tensor_peak(0, 10, 7, C.byref(tf), None) == lb.ERR_ARG
