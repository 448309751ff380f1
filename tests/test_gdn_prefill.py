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
