// abi_util.h -- helpers shared by the kernel-level entry points of the C ABI (kernel_abi.cu, nvfp4_abi.cu): scoped device
// scratch, the device check, early-return macros.
#pragma once

#include <algorithm>
#include <vector>

#include "../../include/ling_b200.h"
#include "gemm.h"
#include "kernels.h"

namespace lb {

struct Scratch {  // device allocations freed on scope exit
  std::vector<void*> p;
  ~Scratch() {
    for (void* q : p) cudaFree(q);
  }
  template <typename T>
  T* get(size_t n, bool zero = true) {
    void* q = nullptr;
    if (cudaMalloc(&q, std::max<size_t>(n, 1) * sizeof(T)) != cudaSuccess) return nullptr;
    if (zero) cudaMemset(q, 0, std::max<size_t>(n, 1) * sizeof(T));
    p.push_back(q);
    return static_cast<T*>(q);
  }
  template <typename T>
  T* put(const T* host, size_t n) {
    T* q = get<T>(n, false);
    if (q && cudaMemcpy(q, host, n * sizeof(T), cudaMemcpyHostToDevice) != cudaSuccess) return nullptr;
    return q;
  }
};

inline int check_device(int device) {
  LB_CUDA(cudaSetDevice(device));
  cudaDeviceProp prop;
  LB_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10) {
    set_error(std::string("this library is built for sm_100a (B200) only; device is ") + prop.name);
    return LING_B200_ERR_UNSUPPORTED;
  }
  if (const int r = gemm_init()) return r;
  return kernels_init();
}
#define LB_TRY(call)                      \
  do {                                    \
    const int rc__ = (call);              \
    if (rc__ != LING_B200_OK) return rc__; \
  } while (0)
#define LB_PTR(p)                          \
  do {                                     \
    if (!(p)) {                            \
      set_error("device allocation failed"); \
      return LING_B200_ERR_CUDA;           \
    }                                      \
  } while (0)


}  // namespace lb
