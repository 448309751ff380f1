// noalloc.cu -- the block-scaled FP8 weight GEMM for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc on the path where they need a GEMM: a serving loop that has handed
// every byte of the device to its own arena at start-up and treats a later allocation as a bug (the reference engine
// allocates nothing while serving), a real-time thread on which an allocation's implicit device synchronization is not
// acceptable, or a sandboxed plugin that is given buffers but not the right to create them.  The regular GEMM needs
// scratch: its K splits write partial-sum planes that are added afterwards.  Here that scratch is a file-scope __device__
// array of a fixed, modest size (16 MiB) that every GPU which loads the library carries until the process exits; the caller
// passes only the operands and the output.
//
// The array's name is a host-side stand-in in host code, not a device address, so its address is taken once per device
// with cudaGetSymbolAddress (with that device current) and cached; the first call on a device does this.  Every call waits
// for its stream before it returns.  Every call uses the same array: two calls that overlap on the GPU (different streams, or
// two host threads) race on it.  The planes need no clearing (a call reads back only what it wrote); the error word is
// cleared at the start of every call.
#include <mutex>

#include "gemm.h"
#include "kernels.h"

namespace lb {
namespace {

constexpr size_t kNoAllocScratchFloats = size_t(LING_B200_NOALLOC_SCRATCH_BYTES) / 4;
static __device__ __align__(256) float g_noalloc_planes[kNoAllocScratchFloats];
static __device__ __align__(256) int g_noalloc_err[64];

struct PerDevice {
  float* planes = nullptr;
  int* err = nullptr;
  int sms = 0;
  bool ready = false;
};
PerDevice g_per_device[64];
std::mutex g_setup_mutex;

// y[m][n] = sum over the K splits' planes, in plane order (the order every consumer of the step uses).
__global__ void __launch_bounds__(256)
    planes_reduce_kernel(const float* __restrict__ planes, int splits, size_t stride, int ld, float* __restrict__ y, int M, int N) {
  pdl_sync();  // first statement: see common.cuh
  const int m = blockIdx.y;
  for (int n = blockIdx.x * blockDim.x + threadIdx.x; n < N; n += gridDim.x * blockDim.x) {
    float v = 0.f;
    for (int p = 0; p < splits; ++p) v += planes[size_t(p) * stride + size_t(m) * ld + n];
    y[size_t(m) * N + n] = v;
  }
}

int setup_device(PerDevice** out) {
  int dev = 0;
  LB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) {
    set_error("gemm_fp8_noalloc: device ordinal out of range");
    return LING_B200_ERR_ARG;
  }
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  PerDevice& p = g_per_device[dev];
  if (!p.ready) {
    cudaDeviceProp prop;
    LB_CUDA(cudaGetDeviceProperties(&prop, dev));
    if (prop.major != 10) {
      set_error(std::string("this library is built for sm_100a (B200) only; device is ") + prop.name);
      return LING_B200_ERR_UNSUPPORTED;
    }
    if (const int r = gemm_init()) return r;  // opts the kernels into their shared memory; allocates nothing
    // In host code the arrays' names are stand-ins: the device addresses come from the runtime, for the current device.
    LB_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&p.planes), g_noalloc_planes));
    LB_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&p.err), g_noalloc_err));
    p.sms = prop.multiProcessorCount;
    p.ready = true;
  }
  *out = &p;
  return LING_B200_OK;
}

}  // namespace
}  // namespace lb

using namespace lb;

extern "C" int ling_b200_gemm_fp8_noalloc(const uint8_t* w_codes, const float* w_scales, const uint8_t* x_codes,
                                          const float* x_scales, float* y, int M, int N, int K, void* stream) {
  if (!w_codes || !w_scales || !x_codes || !x_scales || !y || M < 1 || N < 1 || K < 1) {
    set_error("gemm_fp8_noalloc: bad argument");
    return LING_B200_ERR_ARG;
  }
  const int N_pad = round_up(N, kTileN), K_pad = round_up(K, kBlockK), KB = K_pad / kBlockK;
  const size_t plane = size_t(LING_B200_NOALLOC_MAX_ROWS) * N_pad;  // floats of one K split's plane
  if (M > LING_B200_NOALLOC_MAX_ROWS || plane > kNoAllocScratchFloats) {
    set_error("gemm_fp8_noalloc: beyond the built-in scratch: at most " + std::to_string(LING_B200_NOALLOC_MAX_ROWS) + " rows and " +
              std::to_string(kNoAllocScratchFloats / LING_B200_NOALLOC_MAX_ROWS) + " (padded) output columns; got M = " +
              std::to_string(M) + ", N = " + std::to_string(N));
    return LING_B200_ERR_ARG;
  }
  PerDevice* dev = nullptr;
  if (const int r = setup_device(&dev)) return r;
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  Fp8Matrix W;
  W.codes = const_cast<uint8_t*>(w_codes), W.scales = const_cast<float*>(w_scales);
  W.N = N, W.K = K, W.N_pad = N_pad, W.K_pad = K_pad, W.KB = KB;
  W.splits = int(std::min<size_t>(size_t(choose_splits(N_pad, KB, dev->sms)), kNoAllocScratchFloats / plane));  // as many K splits as the scratch holds
  Fp8Acts X;
  X.codes = const_cast<uint8_t*>(x_codes), X.scales = const_cast<float*>(x_scales);
  X.rows_alloc = LING_B200_NOALLOC_MAX_ROWS, X.K = K, X.K_pad = K_pad, X.KB = KB;
  if (const int r = make_weight_map(W)) return r;  // tensor maps are encoded on the host into these structs
  if (const int r = make_acts_maps(X)) return r;

  LB_CUDA(cudaMemsetAsync(dev->err, 0, sizeof(int), s));  // the error word must start at zero; the planes need not
  GemmCall c;
  c.W = &W, c.X = &X, c.M = M, c.out = dev->planes, c.ld = N_pad, c.split_stride = plane, c.impl = 0, c.err_flag = dev->err;
  if (const int r = gemm_launch(c, s)) return r;
  LB_CUDA(launch_kernel(planes_reduce_kernel, dim3(ceil_div(N, 256), M), dim3(256), size_t(0), s, (const float*)dev->planes, W.splits,
                        plane, N_pad, y, M, N));
  int err = 0;
  LB_CUDA(cudaMemcpyAsync(&err, dev->err, sizeof(int), cudaMemcpyDeviceToHost, s));
  LB_CUDA(cudaStreamSynchronize(s));
  if (err != 0) {
    set_error("gemm_fp8_noalloc: device error word = " + std::to_string(err) + " (a bounded wait of the GEMM ran out)");
    return LING_B200_ERR_DEVICE_FLAG;
  }
  return LING_B200_OK;
}
