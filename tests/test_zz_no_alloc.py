"""The GEMM entry point that allocates nothing (ling_b200_gemm_fp8_noalloc), through the C ABI.

Who needs it: a host that cannot call cudaMalloc where it needs the GEMM -- a serving loop that handed the whole device to
its own arena at start-up, a real-time thread that cannot take an allocation's implicit synchronization, a plugin that is
given buffers but may not create them.  The K splits' partial-sum planes live in a 16 MiB __device__ array inside the
library instead of a per-call allocation.

The check: its output against the regular entry point (ling_b200_gemm_fp8_host, which allocates its scratch) on the same
operands, within the GEMM tolerance of tests/test_gpu_kernels.py, on two calls in a row with different shapes -- the
second call finds the first call's planes still in the shared array and must not be affected by them.  Both entry points
see the same FP8 codes: the operands are quantized once on the host (bit-identical to the device quantizer, as
test_weight_and_activation_quantizers_are_bit_exact shows) and laid out as the library's device layouts.
This file sorts last so that a run that stops at the first failure has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

GEMM_RTOL, GEMM_ATOL_RMS = 1e-5, 1e-4   # the bars of tests/test_gpu_kernels.py


def device_operands(torch, lo, x, w):
    """Host quantization (scale = amax/448 per row per 128 columns, E4M3 codes) into the padded device layouts."""
    M, K = x.shape
    N = w.shape[0]
    n_pad, k_pad = (N + 127) // 128 * 128, (K + 127) // 128 * 128
    wc, ws = lo.quant_rows(w, bf16_first=True)
    xc, xs = lo.quant_rows(x, bf16_first=False)
    w_codes = np.zeros((n_pad, k_pad), np.uint8)
    w_codes[:N, :K] = wc
    w_scales = np.ones((k_pad // 128, n_pad), np.float32)
    w_scales[:, :N] = ws.T
    x_codes = np.zeros((128, k_pad), np.uint8)
    x_codes[:M, :K] = xc
    x_scales = np.ones((k_pad // 128, 128), np.float32)
    x_scales[:, :M] = xs.T
    return [torch.from_numpy(a).cuda() for a in (w_codes, w_scales, x_codes, x_scales)]


def test_noalloc_gemm_matches_the_allocating_entry_point_twice_in_a_row(gpu, lb, lo):
    torch = pytest.importorskip("torch")
    fn = lb.lib().ling_b200_gemm_fp8_noalloc
    fn.argtypes = [C.c_void_p] * 5 + [C.c_int] * 3 + [C.c_void_p]
    rng = np.random.default_rng(42)
    # first a wide matrix that fills many planes of the shared array, then a smaller one that reuses its beginning
    for M, N, K in ((24, 5120, 2048), (7, 384, 704)):
        x = rng.standard_normal((M, K)).astype(np.float32)
        w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
        w = np.array([lo.lo().lo_bf16_round(float(v)) for v in w.ravel()], np.float32).reshape(w.shape) if w.size < 1 << 19 else \
            (w.view(np.uint32) + 0x7fff + ((w.view(np.uint32) >> 16) & 1) & 0xffff0000).view(np.float32)   # round to BF16 once, here
        ref = lb.gemm_fp8(x, w, impl=0)
        dev = device_operands(torch, lo, x, w)
        y = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = fn(dev[0].data_ptr(), dev[1].data_ptr(), dev[2].data_ptr(), dev[3].data_ptr(), y.data_ptr(), M, N, K, None)
        assert rc == 0, lb.last_error()
        assert torch.cuda.memory_allocated() == before
        got = y.cpu().numpy()
        rms = np.sqrt((ref.astype(np.float64) ** 2).mean(axis=1, keepdims=True)) + 1e-30
        assert np.isfinite(got).all()
        assert (np.abs(got - ref) <= GEMM_RTOL * np.abs(ref) + GEMM_ATOL_RMS * rms).all(), float(np.abs(got - ref).max())


def test_noalloc_gemm_rejects_sizes_beyond_its_scratch(gpu, lb):
    fn = lb.lib().ling_b200_gemm_fp8_noalloc
    fn.argtypes = [C.c_void_p] * 5 + [C.c_int] * 3 + [C.c_void_p]
    one = C.c_void_p(16)   # never dereferenced: the size check comes first
    assert fn(one, one, one, one, one, 129, 256, 256, None) == lb.ERR_ARG and "beyond the built-in scratch" in lb.last_error()
    assert fn(one, one, one, one, one, 8, 40000, 256, None) == lb.ERR_ARG and "beyond the built-in scratch" in lb.last_error()
