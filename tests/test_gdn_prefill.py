"""The prefill path's DeltaNet core: the conv over many rows and the gated delta rule in 32-token chunks on tensor cores,
against the oracle's token-by-token rule and, where it is built, against the reference's own prefill kernels."""
import ctypes as C

import numpy as np
import pytest

from oracle import lo

DK = DV = 128
# The chunked form multiplies FP16 copies of q^, k^, beta v, the state and the intermediate matrices (fp32 accumulation), so it
# differs from the fp32 token rule by FP16 operand rounding (2^-11 relative per operand, sums of 128 products): measured
# root-mean-square errors of 3e-4 .. 1e-3 of the tensor's rms and worst elements up to 1.6e-2 of it, the reference's own
# prefill kernel the same.  Bars: rms error <= 2e-3, worst element <= 3e-2, both relative to the tensor's rms.
RMS_TOL, MAX_TOL = 2e-3, 3e-2


def case(seed, Hk, HV, M, decay):
    rng = np.random.default_rng(seed)
    Cc = 2 * Hk * DK + HV * DV
    pre = rng.standard_normal((M, Cc)).astype(np.float32)
    convw = (rng.standard_normal((Cc, 4)) * 0.5).astype(np.float32)
    alpha = 1.0 / (1.0 + np.exp(-rng.standard_normal((M, HV)) - decay))  # decay 0: alpha = sigma(N(0,1)); 3: close to 1
    g = np.log(alpha).astype(np.float32)
    beta = (1.0 / (1.0 + np.exp(-rng.standard_normal((M, HV))))).astype(np.float32)
    state = (rng.standard_normal((HV, DK, DV)) * 0.1).astype(np.float32)
    conv = rng.standard_normal((Cc, 3)).astype(np.float32)
    return pre, convw, g, beta, state, conv


def rel(a, b):
    return float(np.abs(a - b).max() / (np.sqrt(np.mean(np.square(b.astype(np.float64)))) + 1e-30))


def rms_rel(a, b):
    d = a.astype(np.float64) - b.astype(np.float64)
    return float(np.sqrt(np.mean(d * d)) / (np.sqrt(np.mean(np.square(b.astype(np.float64)))) + 1e-30))


def close(a, b):
    return rms_rel(a, b) <= RMS_TOL and rel(a, b) <= MAX_TOL


def bf16_values(lb, w):
    bits = lb.to_bf16_bits(w)
    return bits, (bits.astype(np.uint32) << 16).view(np.float32).reshape(w.shape)


def test_oracle_prefill_does_not_depend_on_the_split():
    pre, convw, g, beta, state, conv = case(1, 1, 2, 70, 0.0)
    post, core, s1, c1 = lo.gdn_prefill(1, 2, DK, DV, pre, convw, g, beta, state, conv)
    pa, ca, sa, wa = lo.gdn_prefill(1, 2, DK, DV, pre[:32], convw, g[:32], beta[:32], state, conv)
    pb, cb, sb, wb = lo.gdn_prefill(1, 2, DK, DV, pre[32:], convw, g[32:], beta[32:], sa, wa)
    assert np.array_equal(np.vstack([pa, pb]), post) and np.array_equal(np.vstack([ca, cb]), core)
    assert np.array_equal(sb, s1) and np.array_equal(wb, c1) and np.array_equal(c1, pre[-3:].T)


@pytest.mark.gpu
@pytest.mark.parametrize("Hk,HV,M,decay", [(2, 4, 1, 0.0), (2, 4, 31, 0.0), (2, 4, 32, 3.0), (2, 4, 33, 0.0), (1, 2, 96, 3.0), (2, 6, 200, 0.0),
                                            (16, 48, 64, 3.0), (2, 4, 1000, 3.0)])
def test_chunked_delta_rule_matches_the_token_rule(gpu, lb, Hk, HV, M, decay):
    pre, convw, g, beta, state, conv = case(M + HV, Hk, HV, M, decay)
    bits, convw = bf16_values(lb, convw)
    post, core, s1, c1 = lb.gdn_prefill(Hk, HV, DK, DV, pre, bits, g, beta, state, conv)
    opost, ocore, os1, oc1 = lo.gdn_prefill(Hk, HV, DK, DV, pre, convw, g, beta, state, conv)
    assert rel(post, opost) <= 1e-5 and np.array_equal(c1, oc1)  # fp32 either side, __expf in the SiLU
    assert close(core, ocore), (rms_rel(core, ocore), rel(core, ocore))
    assert close(s1, os1), (rms_rel(s1, os1), rel(s1, os1))
    R = lo.refcuda()
    if R is not None and hasattr(R, "refcuda_gdn_prefill"):  # the reference's own chunked kernel on the same inputs
        f = lambda a: a.ctypes.data_as(C.POINTER(C.c_float))  # noqa: E731
        rs, rc = state.copy(), conv.copy()
        rpost, rcore = np.zeros_like(post), np.zeros_like(core)
        assert R.refcuda_gdn_prefill(Hk, HV, M, f(pre), f(convw), f(g), f(beta), f(rs), f(rc), f(rpost), f(rcore)) == 0
        assert close(rcore, ocore) and close(rs, os1)  # the oracle against the reference's kernel: the same bars
        assert np.array_equal(rc, oc1) and rel(rpost, opost) <= 1e-5
        # and this kernel is no further from the token rule than the reference's is
        assert rms_rel(core, ocore) <= 1.5 * rms_rel(rcore, ocore) + 2e-4, (rms_rel(core, ocore), rms_rel(rcore, ocore))
        assert rms_rel(s1, os1) <= 1.5 * rms_rel(rs, os1) + 2e-4, (rms_rel(s1, os1), rms_rel(rs, os1))
        print("M=%d HV=%d: core rms %.1e (reference kernel %.1e), state rms %.1e (%.1e)" %
              (M, HV, rms_rel(core, ocore), rms_rel(rcore, ocore), rms_rel(s1, os1), rms_rel(rs, os1)))


@pytest.mark.gpu
def test_chunks_at_multiples_of_32_make_the_split_invisible(gpu, lb):
    pre, convw, g, beta, state, conv = case(5, 2, 4, 96, 3.0)
    bits, _ = bf16_values(lb, convw)
    post, core, s1, c1 = lb.gdn_prefill(2, 4, DK, DV, pre, bits, g, beta, state, conv)
    pa, ca, sa, wa = lb.gdn_prefill(2, 4, DK, DV, pre[:64], bits, g[:64], beta[:64], state, conv)
    pb, cb, sb, wb = lb.gdn_prefill(2, 4, DK, DV, pre[64:], bits, g[64:], beta[64:], sa, wa)
    assert np.array_equal(np.vstack([pa, pb]), post) and np.array_equal(np.vstack([ca, cb]), core)
    assert np.array_equal(sb, s1) and np.array_equal(wb, c1)


@pytest.mark.gpu
def test_gdn_prefill_rejects_other_head_sizes(gpu, lb):
    pre, convw, g, beta, state, conv = case(1, 1, 1, 4, 0.0)
    with pytest.raises(lb.LingError):
        lb.gdn_prefill(1, 1, 64, 64, pre, lb.to_bf16_bits(convw), g, beta, state, conv)


def bf(bits):
    return (np.asarray(bits).astype(np.uint32) << 16).view(np.float32).reshape(np.shape(bits))


@pytest.mark.gpu
@pytest.mark.parametrize("M", [70, 128])
def test_prefill_gdn_layer_matches_the_oracle_stage_by_stage(gpu, lb, M):
    """One DeltaNet layer's mixer on the prefill path: norm -> NVFP4 in projections -> conv, gating, chunked delta rule -> gated
    norm -> NVFP4 out projection.  Each stage is held to the oracle on the inputs the device fed it (so that a block-scale or
    4-bit code that flips on a last-bit difference upstream does not blur the stages behind it); the whole chain to a looser bar."""
    H, Hk, HV = 512, 2, 4
    layer = lb.PrefillGdnLayer(H, Hk, HV, 128, seed=3)
    w = layer.weights()
    rng = np.random.default_rng(M)
    h = rng.standard_normal((M, H)).astype(np.float32)
    state = (rng.standard_normal((HV, DK, DV)) * 0.1).astype(np.float32)
    conv = rng.standard_normal((layer.C, 3)).astype(np.float32)
    layer.set_state(state, conv)
    out = layer.forward(h)
    st = layer.stages(M)
    s1, c1 = layer.get_state()
    layer.close()

    def gemm(x, scale, q, s, wscale):
        xq, xs = lo.nvfp4_quant_act(x, scale)
        return lo.nvfp4_gemm(xq, xs, q, s, scale * wscale)

    def gating(xn):
        a = xn.astype(np.float64) @ bf(w["wa"]).astype(np.float64).T + bf(w["dt_bias"]).astype(np.float64)
        b = xn.astype(np.float64) @ bf(w["wb"]).astype(np.float64).T
        sp = np.where(a <= 20, np.log1p(np.exp(np.minimum(a, 20))), a)  # softplus (src/core/kernels.cu:385-395)
        return (-np.exp(bf(w["A_log"]).astype(np.float64)) * sp).astype(np.float32), (1 / (1 + np.exp(-b))).astype(np.float32)

    def gated(core, z):  # rmsnorm over each head of 128 with the plain weight, times silu(z) (src/core/kernels.cu:543-554)
        c = core.astype(np.float64).reshape(M, HV, 128)
        rstd = 1.0 / np.sqrt((c * c).mean(-1, keepdims=True) + 1e-6)
        zz = z.astype(np.float64).reshape(M, HV, 128)
        return (c * rstd * bf(w["lin_norm"]).astype(np.float64) * (zz / (1 + np.exp(-zz)))).reshape(M, HV * 128).astype(np.float32)

    # stage by stage, each from the device's own inputs
    xn = lo.rmsnorm_rows(h, w["norm"], 1e-6)
    assert rel(st["xn"], xn) <= 1e-5
    assert rel(st["pre"], gemm(st["xn"], w["in_scale"], w["qkv_q"], w["qkv_s"], w["s_qkv"])) <= 1e-4
    assert rel(st["z"], gemm(st["xn"], w["in_scale"], w["z_q"], w["z_s"], w["s_z"])) <= 1e-4
    g, beta = gating(st["xn"])
    assert np.abs(st["g"] - g).max() <= 1e-5 * max(1.0, float(np.abs(g).max())) and np.abs(st["beta"] - beta).max() <= 1e-5
    post, core, os1, oc1 = lo.gdn_prefill(Hk, HV, DK, DV, st["pre"], bf(w["convw"]), st["g"], st["beta"], state, conv)
    assert close(st["core"], core), (rms_rel(st["core"], core), rel(st["core"], core))
    assert close(s1, os1) and np.array_equal(c1, oc1)
    mixed = gemm(gated(st["core"], st["z"]), w["mid_scale"], w["out_q"], w["out_s"], w["s_out"])
    assert rms_rel(out - h, mixed) <= 2e-3 and rel(out - h, mixed) <= 1e-1  # (a 4-bit code may flip on the last bit of the norm)
    # the whole chain from the oracle's own stages
    pre_o = gemm(xn, w["in_scale"], w["qkv_q"], w["qkv_s"], w["s_qkv"])
    z_o = gemm(xn, w["in_scale"], w["z_q"], w["z_s"], w["s_z"])
    g_o, b_o = gating(xn)
    _, core_o, _, _ = lo.gdn_prefill(Hk, HV, DK, DV, pre_o, bf(w["convw"]), g_o, b_o, state, conv)
    chain = gemm(gated(core_o, z_o), w["mid_scale"], w["out_q"], w["out_s"], w["s_out"])
    assert rms_rel(out - h, chain) <= 3e-2, rms_rel(out - h, chain)
