// ref_quant_shim.cpp -- C wrapper around the REFERENCE's own host-side NVFP4 weight rounding (quantize_nvfp4,
// src/core/model.cu:188-249 of dreamference/ling-engine), compiled from where the source lies into
// oracle/_ref/libling_refquant.so (see oracle/Makefile, target ref_quant).  TEST INFRASTRUCTURE ONLY; nothing of the
// reference is copied into this repository.  model.cu also holds the checkpoint loader, whose callees (the tiled-weight
// kernels) are not built here: the library is linked with unresolved symbols allowed and must be opened with lazy binding;
// only the function below is ever called.
#include <cstdint>
#include <cstring>
#include <exception>
#include <string>

#include "core/model.hpp"

namespace {
std::string g_err;
}

extern "C" {

const char* refquant_last_error() { return g_err.c_str(); }

// w: BF16 bit patterns [N][K]; q [N][K/2]; sf [N][K/16].
int refquant_nvfp4(const uint16_t* w, int N, int K, uint8_t* q, uint8_t* sf, float* scale2, double* rel_sq_error) {
  try {
    const ling::Nvfp4Host h = ling::quantize_nvfp4(reinterpret_cast<const __nv_bfloat16*>(w), N, K);
    std::memcpy(q, h.values.data(), h.values.size());
    std::memcpy(sf, h.scales.data(), h.scales.size());
    *scale2 = h.scale2;
    if (rel_sq_error) *rel_sq_error = h.rel_sq_error;
    return 0;
  } catch (const std::exception& e) {
    g_err = e.what();
    return 1;
  }
}

}  // extern "C"
