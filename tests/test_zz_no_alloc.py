"""The GEMM entry point that allocates nothing (ling_b200_gemm_fp8_noalloc), through the C ABI.

Who needs it: a host that cannot call cudaMalloc where it needs the GEMM -- a serving loop that handed the whole device to
its own arena at start-up, a real-time thread that cannot take an allocation's implicit synchronization, a plugin that is
given buffers but may not create them.  The K splits' partial-sum planes live in a 16 MiB __device__ array inside the
library instead of a per-call allocation.

The check: its output against the regular entry point (ling_b200_gemm_fp8_host, which allocates its scratch) and against
the CPU oracle on the same operands, within the GEMM tolerance of tests/test_gpu_kernels.py, on two shapes in a row -- the
second finds the first one's planes still in the shared array and must not be affected by them -- and the device's free
memory (cudaMemGetInfo, which sees an allocation whoever makes it) is the same before and after a call.  Both entry points
see the same FP8 codes: the operands are quantized once on the host (bit-identical to the device quantizer, as
test_weight_and_activation_quantizers_are_bit_exact shows) and laid out as the library's device layouts.
This file sorts last so that a run that stops at the first failure has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

GEMM_RTOL, GEMM_ATOL_RMS = 1e-5, 1e-4   # the bars of tests/test_gpu_kernels.py


class Cuda:
    """The CUDA runtime through ctypes, for the caller's side of the call: device buffers for the operands and the
    device-wide free-memory figure (cudaMemGetInfo), which sees an allocation whoever makes it.  The library under test
    links its own static copy of the runtime; both use the device's primary context, so pointers are interchangeable."""

    def __init__(self):
        self.rt = None
        for name in ("libcudart.so.12", "/usr/local/cuda/lib64/libcudart.so.12", "libcudart.so", "/usr/local/cuda/lib64/libcudart.so"):
            try:
                self.rt = C.CDLL(name)
                break
            except OSError:
                continue
        if self.rt is None:
            pytest.fail("no CUDA runtime library (libcudart) found to allocate the caller's buffers with")
        self.ptrs = []

    def ok(self, rc):
        assert rc == 0, "CUDA runtime call failed with error %d" % rc

    def put(self, a):
        a = np.ascontiguousarray(a)
        p = C.c_void_p()
        self.ok(self.rt.cudaMalloc(C.byref(p), C.c_size_t(max(a.nbytes, 1))))
        self.ok(self.rt.cudaMemcpy(p, a.ctypes.data_as(C.c_void_p), C.c_size_t(a.nbytes), 1))
        self.ptrs.append(p)
        return p

    def get(self, p, shape, dtype):
        out = np.zeros(shape, dtype)
        self.ok(self.rt.cudaMemcpy(out.ctypes.data_as(C.c_void_p), p, C.c_size_t(out.nbytes), 2))
        return out

    def free_bytes(self):
        free, total = C.c_size_t(), C.c_size_t()
        self.ok(self.rt.cudaDeviceSynchronize())
        self.ok(self.rt.cudaMemGetInfo(C.byref(free), C.byref(total)))
        return free.value

    def close(self):
        for p in self.ptrs:
            self.rt.cudaFree(p)
        self.ptrs = []


def device_operands(cu, lo, x, w):
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
    return [cu.put(a) for a in (w_codes, w_scales, x_codes, x_scales)]


def test_noalloc_gemm_matches_the_allocating_entry_point_twice_in_a_row(gpu, lb, lo):
    cu = Cuda()
    fn = lb.lib().ling_b200_gemm_fp8_noalloc
    fn.argtypes = [C.c_void_p] * 5 + [C.c_int] * 3 + [C.c_void_p]
    rng = np.random.default_rng(42)
    # first a wide matrix that fills many planes of the shared array, then a smaller one that reuses its beginning
    for M, N, K in ((24, 5120, 2048), (7, 384, 704)):
        x = rng.standard_normal((M, K)).astype(np.float32)
        w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
        u = w.view(np.uint32)
        w = ((u + 0x7fff + ((u >> 16) & 1)) & 0xffff0000).astype(np.uint32).view(np.float32)   # round to BF16 once, here
        ref = lb.gemm_fp8(x, w, impl=0)        # the existing entry point (allocates its scratch per call)
        oracle = lo.gemm_fp8(x, w)             # the CPU oracle on the same operands
        dev = device_operands(cu, lo, x, w)
        y = cu.put(np.full((M, N), np.nan, np.float32))
        rc = fn(dev[0], dev[1], dev[2], dev[3], y, M, N, K, None)    # the first call on the device also looks the array up
        assert rc == 0, lb.last_error()
        cu.ok(cu.rt.cudaMemcpy(y, np.full((M, N), np.nan, np.float32).ctypes.data_as(C.c_void_p), C.c_size_t(M * N * 4), 1))
        before = cu.free_bytes()
        rc = fn(dev[0], dev[1], dev[2], dev[3], y, M, N, K, None)
        assert rc == 0, lb.last_error()
        assert cu.free_bytes() == before       # nobody allocated device memory during the call: not the library, not its runtime
        got = cu.get(y, (M, N), np.float32)
        assert np.isfinite(got).all()
        for want in (ref, oracle):
            rms = np.sqrt((want.astype(np.float64) ** 2).mean(axis=1, keepdims=True)) + 1e-30
            assert (np.abs(got - want) <= GEMM_RTOL * np.abs(want) + GEMM_ATOL_RMS * rms).all(), float(np.abs(got - want).max())
    cu.close()


def test_noalloc_gemm_rejects_sizes_beyond_its_scratch(gpu, lb):
    fn = lb.lib().ling_b200_gemm_fp8_noalloc
    fn.argtypes = [C.c_void_p] * 5 + [C.c_int] * 3 + [C.c_void_p]
    one = C.c_void_p(16)   # never dereferenced: the size check comes first
    assert fn(one, one, one, one, one, 129, 256, 256, None) == lb.ERR_ARG and "beyond the built-in scratch" in lb.last_error()
    assert fn(one, one, one, one, one, 8, 40000, 256, None) == lb.ERR_ARG and "beyond the built-in scratch" in lb.last_error()
