// Shared device/host helpers of the B200 verify-step library: error plumbing, number formats, the counter-based
// generator, warp reductions.  sm_100a only.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <cstdlib>

#include <cstdint>
#include <cstdio>
#include <string>
#include <utility>

namespace lb {

// ---------------------------------------------------------------------------------------------- errors
void set_error(const std::string& what);  // thread-local text behind ling_b200_last_error()
inline bool cuda_ok(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return true;
  set_error(std::string(what) + ": " + cudaGetErrorString(e));
  return false;
}
#define LB_CUDA(call)                                   \
  do {                                                  \
    if (!::lb::cuda_ok((call), #call)) return LING_B200_ERR_CUDA; \
  } while (0)
// LING_B200_SYNC_LAUNCHES (debugging aid, eager launches only -- not under graph capture): the device is synchronized after
// every launch, so an asynchronous fault is reported with the name of the kernel that raised it.
inline bool sync_launches() {
  static const bool on = std::getenv("LING_B200_SYNC_LAUNCHES") != nullptr;
  return on;
}
#define LB_LAUNCH(name)                                                 \
  do {                                                                  \
    if (!::lb::cuda_ok(cudaGetLastError(), name)) return LING_B200_ERR_CUDA; \
    if (::lb::sync_launches() && !::lb::cuda_ok(cudaDeviceSynchronize(), name)) return LING_B200_ERR_CUDA; \
  } while (0)

// Device-side error word: kernels never trap; a bounded wait that runs out or a bounds check that trips records a
// code here (first writer wins) and the kernel returns.  The host reads it after the step.
enum DeviceError : int {
  kDevOk = 0,
  kDevWaitFull = 1,       // GEMM consumer: a TMA stage never arrived
  kDevWaitEmpty = 2,      // GEMM producer: a stage was never released
  kDevWaitTmemFull = 3,   // GEMM epilogue: the accumulator never completed
  kDevWaitTmemEmpty = 4,  // GEMM issuer: the accumulator buffer was never drained
  kDevBadPage = 5,        // a position maps to page 0 or past the pool
  kDevBadTree = 6,        // a parent index is not below its row, or too many leaves/paths
  kDevBadToken = 7        // a token id outside the vocabulary
};
__device__ __forceinline__ void dev_fail(int* flag, int code) {
  if (flag) atomicCAS(flag, 0, code);
}

// ---------------------------------------------------------------------------------------------- formats
// E4M3 with saturation, round to nearest even (the one conversion used for weights, activations and the KV cache).
__device__ __forceinline__ uint8_t to_e4m3(float x) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ float from_e4m3(uint8_t c) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(c), __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}
// Two packed E4M3 codes (low byte first) to two halves.
__device__ __forceinline__ uint32_t e4m3x2_to_h2(uint16_t pair) {
  const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(pair), __NV_E4M3);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__host__ __device__ __forceinline__ float bf16_round(float x) {
  uint32_t u;
  memcpy(&u, &x, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return x;
  u += 0x7fffu + ((u >> 16) & 1u);
  u &= 0xffff0000u;
  float r;
  memcpy(&r, &u, 4);
  return r;
}
__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float sigmoidf(float x) { return 1.f / (1.f + __expf(-x)); }

// ---------------------------------------------------------------------------------------------- generator
// Element i of stream s under a seed is a function of (seed, s, i) alone; z is the centred sum of twelve 16-bit
// uniforms scaled to unit variance, in integer arithmetic, so host and device agree bit for bit.
__host__ __device__ __forceinline__ uint64_t mix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}
__host__ __device__ __forceinline__ uint64_t stream_key(uint64_t seed, uint64_t stream) {
  return mix64(seed ^ mix64(stream));
}
__host__ __device__ __forceinline__ float synth_z(uint64_t key, uint64_t i) {
  int s = 0;
#pragma unroll
  for (int j = 0; j < 3; ++j) {
    const uint64_t h = mix64(key + 3 * i + j);
    s += int(h & 0xffff) + int((h >> 16) & 0xffff) + int((h >> 32) & 0xffff) + int((h >> 48) & 0xffff);
  }
  return float(2 * s - 786420) * (1.0f / 131072.0f);
}
constexpr uint64_t kStreamKv = 1ull << 32, kStreamState = 2ull << 32, kStreamConv = 3ull << 32;
inline uint64_t weight_stream(int layer, int tensor) { return uint64_t(layer + 1) * 64 + uint64_t(tensor); }

// ---------------------------------------------------------------------------------------------- reductions
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Sum over the block; `red` holds 32 floats.  Every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < warps ? red[lane] : 0.f;
  return warp_sum(t);
}

// ---------------------------------------------------------------------------------------------- dependent launch
// Programmatic dependent launch (the reference's launch.cuh:1-98 discipline, here for every kernel of the step): a kernel
// launched with the attribute may start while its predecessor is still running.  Every kernel's first statement is
// pdl_sync(): it lets its own successor be scheduled (griddepcontrol.launch_dependents) and then waits until the
// predecessor has completed and its writes are visible (griddepcontrol.wait).  Because every kernel waits, completion is
// transitive along the stream.  Only loads of data that no kernel of the step writes (weights) are issued before the
// wait: the weight GEMM prefetches its first tiles there, the norm kernel its weight row.  Without the launch attribute
// both instructions are no-ops.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_sync() {
  pdl_trigger();
  pdl_wait();
}
void set_pdl(bool on);  // the calling host thread's switch (the reference's kernels::set_pdl, src/core/kernels.cuh:82-83, is process-wide)
bool pdl_enabled();

// cluster_x > 1: the grid's x dimension is grouped into thread-block clusters of that many CTAs (distributed shared memory).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, int cluster_x,
                                         cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = stream;
  cudaLaunchAttribute at[2];
  int n = 0;
  if (pdl_enabled()) {
    at[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_x > 1) {
    at[n].id = cudaLaunchAttributeClusterDimension;
    at[n].val.clusterDim.x = unsigned(cluster_x), at[n].val.clusterDim.y = 1, at[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = at;
  cfg.numAttrs = unsigned(n);
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...);
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  return launch_kernel_cluster(kernel, grid, block, smem, 1, stream, std::forward<Args>(args)...);
}

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline int round_up(int a, int b) { return ceil_div(a, b) * b; }

}  // namespace lb
