// A layer segment as one persistent kernel (chain.cu): up to three block-scaled FP8 weight GEMMs and the row-wise work
// between them, for steps of at most 32 packed rows.  Stands in for the reference's persistent per-layer kernels
// (ffn_persistent, gdn_persistent: src/core/kernels.cuh:331-383, src/core/stream_gemm.cu:841-851,1074-1086 in the
// reference project), rebuilt around this library's tcgen05 GEMM.
#pragma once

#include "gemm.h"
#include "kernels.h"

namespace lb {

constexpr int kChainGemms = 3;
constexpr int kChainRows = 32;          // packed rows a chain covers (one 32-row token tile)
constexpr int kChainCounterWords = 2368;  // unsigned words of one chain's dependency counters (zeroed before the step)

struct ChainGemm {
  CUtensorMap mapW, mapX;   // weights {K_pad, N_pad} box 128 x 128; activations {K_pad, rows_alloc} box 128 x 32
  const float* ws;          // [KB][N_pad]
  const float* xs;          // [KB][xrows]
  float* out;               // [splits][rows_alloc][N_pad] partial planes
  size_t split_stride;
  int N, N_pad, KB, splits, xrows;
};

// h (+= planes, or = embedding rows) -> RMSNorm (1 + w) -> fp32 copy (optional) and FP8 copy: norm_quant_kernel's work.
struct ChainNorm {
  float* h;
  Planes add;
  const int* ids;
  const __nv_bfloat16* embed;
  const __nv_bfloat16* w;
  float* xn;
  QuantOut q;
  int H;
  float eps;
};
// a = xn . W_a^T, b = xn . W_b^T, then the gating: ab_gating_kernel's work.
struct ChainAb {
  const float* xn;
  const __nv_bfloat16 *wa, *wb, *A_log, *dt_bias;
  float *g, *beta;
  int H, HV;
};
// silu(gate) * up and its FP8 copy: silu_mul_quant_kernel's work.
struct ChainSilu {
  int I, up_col0;
  QuantOut q;
};

// GEMM 0 .. n_gemm-1 in order.  GEMM norm_gemm reads the norm's output (the norm adds the planes of GEMM norm_gemm - 1, or
// of the kernel before when norm_gemm is 0); with has_silu, GEMM norm_gemm is gate|up and GEMM norm_gemm + 1 reads the
// activation's output; every other GEMM reads an input the kernel before left.
struct ChainProgram {
  int n_gemm = 0, norm_gemm = 0, has_ab = 0, has_silu = 0;
  ChainGemm g[kChainGemms];
  ChainNorm norm;
  ChainAb ab;
  ChainSilu silu;
  const int* n_rows = nullptr;  // real packed rows (device)
  int rows_grid = 0;            // the step's row class (<= 32): rows every unit is laid out for
  unsigned* counters = nullptr; // kChainCounterWords words, zero on entry
  float* ssq = nullptr;         // [32 rows][8 chunks][8] partial sums of squares
  int* err_flag = nullptr;
  int l2_ahead = 0;             // K blocks of weights each CTA keeps requested into L2 ahead of its loads
  unsigned long long* stamps = nullptr;  // nine %globaltimer stamps of this launch (debugging aid), or nullptr
};

int chain_init();
bool chain_supported(const ChainProgram& P, int sm_count);
int chain_launch(const ChainProgram& P, int sm_count, cudaStream_t stream);

}  // namespace lb
