"""The NVFP4 prefill-chunk path on the GPU through the C ABI, against the oracle: the weight rounding and the activation
quantizer byte for byte, the tcgen05 block-scaled GEMM against a float64 product of the same quantized operands at the
reference's own bar (tests/prefill_tests.cu:206 of the reference project: max error <= 1e-4 of the output's rms), the fused
gate|up GEMM byte for byte against the two plain GEMMs followed by the quantizer (the reference's test_swiglu), the
norm + quantize kernel, and the chunk's feed-forward stack against the same chain of oracle calls."""
import json
import os

import numpy as np
import pytest

from test_nvfp4_oracle import E2M1, GOLDEN, bf16_bits, unpack

pytestmark = pytest.mark.gpu

GEMM_TOL = 1e-4        # of the output's rms, plus 1e-6 (the reference's bar for prefill_gemm_nvfp4)
NORM_TOL = 2e-6        # normalized rows against the oracle's double-precision sum of squares, relative to the row's largest value
FFN_TOL = 2e-2         # residual after the stack, rel-L2: a sum that rounds differently can move an activation to the next E2M1 code


def random_operand(rng, rows, K, scale_lo=0x28, scale_hi=0x40):
    """Every nibble pattern, block scales in [2^-2, 2] as the reference's test draws them."""
    return rng.integers(0, 256, (rows, K // 2), dtype=np.uint8), rng.integers(scale_lo, scale_hi + 1, (rows, K // 16), dtype=np.uint8)


def dequant64(lo, q, s):
    dec = lo.e4m3_decode_table().astype(np.float64)
    return E2M1[unpack(q)].astype(np.float64) * np.repeat(dec[s], 16, axis=1)


def test_weight_rounding_is_the_references(gpu, lb, lo):
    for case in json.load(open(GOLDEN)):
        w = np.array(case["w_bf16"], np.uint16).reshape(case["N"], case["K"])
        q, sf, s2 = lb.quantize_nvfp4(w)
        assert q.ravel().tolist() == case["values"], case["name"]
        assert sf.ravel().tolist() == case["scales"], case["name"]
        assert int(np.float32(s2).view(np.uint32)) == case["scale2_bits"], case["name"]
    rng = np.random.default_rng(11)
    w = (rng.standard_normal((300, 5120)) * 0.02).astype(np.float32)
    w[rng.random(w.shape) < 0.003] *= 20
    bits = bf16_bits(w)
    got, want = lb.quantize_nvfp4(bits), lo.nvfp4_quantize_weight(bits)
    assert (got[0] == want[0]).all() and (got[1] == want[1]).all() and got[2] == want[2]


def test_activation_quantizer_byte_for_byte(gpu, lb, lo):
    rng = np.random.default_rng(12)
    for M, K, in_scale, amp in [(67, 512, 0.0019763766, 0.003), (130, 5120, 0.05, 1.0), (1, 16, 1.0, 3.0)]:
        x = (rng.standard_normal((M, K)) * amp).astype(np.float32)
        x.ravel()[::97] *= 40
        if K >= 32:
            x[0, 16:32] = 0
        got, want = lb.quant_act_nvfp4(x, in_scale), lo.nvfp4_quant_act(x, in_scale)
        assert (got[0] == want[0]).all() and (got[1] == want[1]).all()
    # silu(x) * up: the device's __expf and the host's exp differ in the last bits, so a value can land on the other side of
    # a rounding boundary; the fused GEMM test below holds the device to its own unfused path byte for byte
    x, up = rng.standard_normal((64, 1024)).astype(np.float32), rng.standard_normal((64, 1024)).astype(np.float32)
    got, want = lb.quant_act_nvfp4(x, 0.02, up=up), lo.nvfp4_quant_act(x, 0.02, up=up)
    assert (got[0] != want[0]).mean() < 2e-3 and (got[1] != want[1]).mean() < 2e-3


@pytest.mark.parametrize("M,N,K,extra,accumulate", [
    (67, 256, 512, 128, False),     # the reference test's shape class: ragged rows, a wider output row
    (200, 384, 1024, 128, True),    # N % 256 == 128: the last tile's upper half is past the matrix
    (128, 128, 128, 0, False),      # one MMA row block, K shorter than a pipeline stage
    (1, 128, 256, 0, False),
    (300, 640, 384, 64, True),      # K % 256 == 128: the last stage is half past the rows' end
    (513, 2560, 2048, 0, False),    # more tiles than one wave of a small grid, several K stages
])
def test_gemm_against_float64(gpu, lb, lo, M, N, K, extra, accumulate):
    rng = np.random.default_rng(M * 7 + N)
    x = rng.standard_normal((M, K)).astype(np.float32)
    xq, xs = lo.nvfp4_quant_act(x, 0.05)
    wq, ws = random_operand(rng, N, K)
    ldy, alpha = N + extra, 0.37
    y0 = rng.standard_normal((M, ldy)).astype(np.float32)
    got = lb.prefill_gemm_nvfp4(xq, xs, wq, ws, alpha, y=y0, ldy=ldy, accumulate=accumulate)
    ref = alpha * (dequant64(lo, xq, xs) @ dequant64(lo, wq, ws).T) + (y0[:, :N] if accumulate else 0.0)
    rms = np.sqrt((ref ** 2).mean())
    assert np.array_equal(got[:, N:], y0[:, N:]), "columns past N were written"
    assert np.abs(got[:, :N] - ref).max() <= GEMM_TOL * rms + 1e-6
    if M <= 200:  # the oracle's own GEMM agrees with the numpy statement
        want = lo.nvfp4_gemm(xq, xs, wq, ws, alpha, y=y0, ldy=ldy, accumulate=accumulate)
        assert np.abs(want[:, :N] - ref).max() <= 1e-6 * rms + 1e-7


def test_gemm_rows_do_not_depend_on_their_neighbours(gpu, lb, lo):
    rng = np.random.default_rng(3)
    N, K = 512, 1024
    xq, xs = random_operand(rng, 300, K, 0x30, 0x3c)
    wq, ws = random_operand(rng, N, K)
    whole = lb.prefill_gemm_nvfp4(xq, xs, wq, ws, 0.01)
    for r0, r1 in [(0, 1), (5, 70), (128, 300), (299, 300)]:
        part = lb.prefill_gemm_nvfp4(xq[r0:r1], xs[r0:r1], wq, ws, 0.01)
        assert np.array_equal(part, whole[r0:r1])


@pytest.mark.parametrize("M,N,K", [(67, 256, 512), (200, 384, 1024), (300, 1152, 640)])
def test_fused_swiglu_equals_the_unfused_path_byte_for_byte(gpu, lb, lo, M, N, K):
    rng = np.random.default_rng(M + N + K)
    x = rng.standard_normal((M, K)).astype(np.float32)
    xq, xs = lo.nvfp4_quant_act(x, 0.05)
    gq, gs = random_operand(rng, N, K)
    uq, us = random_operand(rng, N, K)
    ag, au, out_in = 0.013, 0.017, 0.3
    g = lb.prefill_gemm_nvfp4(xq, xs, gq, gs, ag)
    u = lb.prefill_gemm_nvfp4(xq, xs, uq, us, au)
    want_q, want_s = lb.quant_act_nvfp4(g, out_in, up=u)
    got_q, got_s = lb.prefill_swiglu_nvfp4(xq, xs, gq, gs, ag, uq, us, au, out_in)
    assert (got_q == want_q).all() and (got_s == want_s).all()
    assert got_q.any() and got_s.any()
    # and the unfused path is the oracle's, up to values that the device's __expf moves across a rounding boundary
    oq, os_ = lo.nvfp4_quant_act(lo.nvfp4_gemm(xq, xs, gq, gs, ag), out_in, up=lo.nvfp4_gemm(xq, xs, uq, us, au))
    assert (oq != got_q).mean() < 5e-3 and (os_ != got_s).mean() < 5e-3


def test_rmsnorm_quant(gpu, lb, lo):
    rng = np.random.default_rng(14)
    M, H, eps, in_scale = 70, 5120, 1e-6, 16.0 / 2688.0
    x = (rng.standard_normal((M, H)) * rng.uniform(0.1, 30, (M, 1))).astype(np.float32)
    w = bf16_bits((rng.standard_normal(H) * 0.02).astype(np.float32))
    out, q, sf = lb.rmsnorm_quant_nvfp4(x, w, eps, in_scale)
    want = lo.rmsnorm_rows(x, w, eps)
    assert np.abs(out - want).max() <= NORM_TOL * np.abs(want).max()
    # the codes are the quantizer's over the kernel's own fp32 output, byte for byte
    wq, ws = lo.nvfp4_quant_act(out, in_scale)
    assert (q == wq).all() and (sf == ws).all()
    _, q2, sf2 = lb.rmsnorm_quant_nvfp4(x, w, eps, in_scale, want_out=False)
    assert (q2 == q).all() and (sf2 == sf).all()


def test_chunk_ffn_stack_against_the_oracle_chain(gpu, lb, lo):
    layers, H, I, rows = 3, 256, 512, 200
    ffn = lb.Nvfp4Ffn(layers, H, I, 256, seed=9)
    rng = np.random.default_rng(15)
    h0 = rng.standard_normal((rows, H)).astype(np.float32)
    got = ffn.forward(h0)
    assert np.array_equal(ffn.forward(h0), got)          # the same inputs give the same bits
    ffn.set_residual(h0)
    ffn.launch(rows)
    assert ffn.wait() > 0
    h = h0.copy()
    for l in range(layers):
        L = ffn.read_layer(l)
        # the stack's weights are the reference rounding of the generator's BF16 values
        n = lo.rmsnorm_rows(h, L["norm"], 1e-6)
        xq, xs = lo.nvfp4_quant_act(n, L["in_scale"])
        g = lo.nvfp4_gemm(xq, xs, *L["gate"], L["in_scale"] * L["s_gate"])
        u = lo.nvfp4_gemm(xq, xs, *L["up"], L["in_scale"] * L["s_up"])
        mq, ms = lo.nvfp4_quant_act(g, L["mid_scale"], up=u)
        h = lo.nvfp4_gemm(mq, ms, *L["down"], L["mid_scale"] * L["s_down"], y=h, accumulate=True)
    assert np.isfinite(got).all()
    delta = np.sqrt(((got - h0) ** 2).sum())
    assert delta > 0.01 * np.sqrt((h0 ** 2).sum()), "the stack must change the residual for the comparison to mean anything"
    assert np.sqrt(((got - h) ** 2).sum()) <= FFN_TOL * delta


def test_ffn_weights_are_the_reference_rounding_of_the_generator(gpu, lb, lo):
    H, I = 256, 512
    ffn = lb.Nvfp4Ffn(1, H, I, 128, seed=4)
    L = ffn.read_layer(0)
    for name, tensor, shape in (("gate", lb.T_GATE, (I, H)), ("up", lb.T_UP, (I, H)), ("down", lb.T_DOWN, (H, I))):
        w = lo.synth(4, lo.weight_stream(0, tensor), 0, shape[0] * shape[1], 0.02).reshape(shape)
        q, s, s2 = lo.nvfp4_quantize_weight(bf16_bits(w))
        assert (L[name][0] == q).all() and (L[name][1] == s).all(), name
        assert L["s_" + name] == s2


def test_down_projection_at_the_27b_shape_sampled(gpu, lb, lo):
    """4096 rows x 5120 x 17408 (the chunk's down projection): 4000 sampled outputs against float64 dot products."""
    rng = np.random.default_rng(16)
    M, N, K = 4096, 5120, 17408
    xq, xs = random_operand(rng, M, K, 0x30, 0x3c)
    wq, ws = random_operand(rng, N, K)
    y = lb.prefill_gemm_nvfp4(xq, xs, wq, ws, 1e-3)
    rows, cols = rng.integers(0, M, 64), rng.integers(0, N, 64)
    rows[:2], cols[:2] = (0, M - 1), (0, N - 1)
    ref = 1e-3 * (dequant64(lo, xq[rows], xs[rows]) @ dequant64(lo, wq[cols], ws[cols]).T)
    rms = np.sqrt((ref ** 2).mean())
    assert np.abs(y[np.ix_(rows, cols)] - ref).max() <= GEMM_TOL * rms + 1e-6
    assert np.isfinite(y).all()


@pytest.mark.parametrize("M,N,K", [(67, 256, 512), (300, 640, 384), (513, 2560, 2048), (128, 128, 128), (257, 384, 1024)])
def test_two_cta_form_gives_the_same_bits(gpu, lb, lo, M, N, K):
    """The cta_group::2 form (a pair of CTAs per 256 x 256 tile) against the one-CTA form: plain, accumulating and fused."""
    rng = np.random.default_rng(M + 3 * N + K)
    xq, xs = lo.nvfp4_quant_act(rng.standard_normal((M, K)).astype(np.float32), 0.05)
    wq, ws = random_operand(rng, N, K)
    uq, us = random_operand(rng, N, K)
    y0 = rng.standard_normal((M, N + 64)).astype(np.float32)

    def run():
        return (lb.prefill_gemm_nvfp4(xq, xs, wq, ws, 0.37, y=y0, ldy=N + 64, accumulate=True),
                lb.prefill_gemm_nvfp4(xq, xs, uq, us, 0.11),
                lb.prefill_swiglu_nvfp4(xq, xs, wq, ws, 0.013, uq, us, 0.017, 0.3))
    prev = lb.nvfp4_pair_mode(0)
    try:
        one = run()
        lb.nvfp4_pair_mode(1)
        two = run()
    finally:
        lb.nvfp4_pair_mode(prev)
    assert np.array_equal(one[0], two[0]) and np.array_equal(one[1], two[1])
    assert np.array_equal(one[2][0], two[2][0]) and np.array_equal(one[2][1], two[2][1])
    ref = 0.11 * (dequant64(lo, xq, xs) @ dequant64(lo, uq, us).T)
    assert np.abs(two[1] - ref).max() <= GEMM_TOL * np.sqrt((ref ** 2).mean()) + 1e-6


def test_chunk_ffn_layer_at_the_27b_width_on_sampled_rows(gpu, lb, lo):
    """One layer of the chunk's stack at the named shape (4096 rows, hidden 5120, FFN 17408).  Every operation of the stack is
    row-wise or a GEMM whose rows are independent, so the oracle chain on a handful of rows checks those rows of the full pass."""
    H, I, rows = 5120, 17408, 4096
    ffn = lb.Nvfp4Ffn(1, H, I, rows, seed=21)
    rng = np.random.default_rng(22)
    h0 = rng.standard_normal((rows, H)).astype(np.float32)
    got = ffn.forward(h0)
    L = ffn.read_layer(0)
    pick = np.array([0, 1, 127, 128, 2049, rows - 1])
    h = h0[pick]
    n = lo.rmsnorm_rows(h, L["norm"], 1e-6)
    xq, xs = lo.nvfp4_quant_act(n, L["in_scale"])
    g = lo.nvfp4_gemm(xq, xs, *L["gate"], L["in_scale"] * L["s_gate"])
    u = lo.nvfp4_gemm(xq, xs, *L["up"], L["in_scale"] * L["s_up"])
    mq, ms = lo.nvfp4_quant_act(g, L["mid_scale"], up=u)
    want = lo.nvfp4_gemm(mq, ms, *L["down"], L["mid_scale"] * L["s_down"], y=h, accumulate=True)
    assert np.isfinite(got).all()
    for i, r in enumerate(pick):
        delta = np.sqrt(((want[i] - h0[r]) ** 2).sum())
        assert delta > 0
        assert np.sqrt(((got[r] - want[i]) ** 2).sum()) <= FFN_TOL * delta, "row %d" % r


def test_gemm_edge_cases(gpu, lb, lo):
    """All-zero activations (block scale 0) give exact zeros and leave an accumulated-into output as it was; 8192 rows (more than
    one pass of the persistent grid over the row tiles) agree with the same rows computed 300 at a time."""
    rng = np.random.default_rng(31)
    N, K = 256, 512
    wq, ws = random_operand(rng, N, K)
    xq, xs = lo.nvfp4_quant_act(np.zeros((40, K), np.float32), 0.05)
    assert not xs.any() and not xq.any()
    assert not lb.prefill_gemm_nvfp4(xq, xs, wq, ws, 0.5).any()
    y0 = rng.standard_normal((40, N)).astype(np.float32)
    assert np.array_equal(lb.prefill_gemm_nvfp4(xq, xs, wq, ws, 0.5, y=y0, accumulate=True), y0)
    xq, xs = random_operand(rng, 8192, K, 0x30, 0x3c)
    whole = lb.prefill_gemm_nvfp4(xq, xs, wq, ws, 0.01)
    for r0 in (0, 4000, 7892):
        assert np.array_equal(lb.prefill_gemm_nvfp4(xq[r0:r0 + 300], xs[r0:r0 + 300], wq, ws, 0.01), whole[r0:r0 + 300])
