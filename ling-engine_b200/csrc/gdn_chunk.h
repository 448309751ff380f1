// The DeltaNet mixer core of the prefill path (gdn_chunk.cu): the causal conv over many rows and the gated delta rule in its
// chunked form.
#pragma once

#include "../../include/ling_b200.h"
#include "common.cuh"

namespace lb {

int gdn_chunk_init();
// The DeltaNet gating of many rows on tensor cores: g, beta [M][HV] from the normalized rows xn [M][H] (fp32, split into two BF16
// terms) and the BF16 projections wa, wb [HV][H] (src/core/kernels.cu:200-253,385-395); H a multiple of 128.
int ab_gating_mma_launch(const float* xn, const __nv_bfloat16* wa, const __nv_bfloat16* wb, const __nv_bfloat16* A_log, const __nv_bfloat16* dt_bias,
                         float* g, float* beta, int M, int H, int HV, cudaStream_t s);
// post [M][C] = silu(conv(pre [M][C])) with the taps before row 0 from window [C][3], which then advances to the last three
// raw inputs (gdn_conv_prefill, src/core/kernels.cuh:445-449).
int conv_rows_launch(const float* pre, const __nv_bfloat16* w, float* window, int M, int C, float* post, cudaStream_t s);
// The gated delta rule over the M rows of one sequence in 32-token chunks (gdn_recurrent_prefill, kernels.cuh:450-456):
// post [M][C] (q | k | v channels, C = 2 Hk Dk + HV Dv), g and beta [M][HV], state [HV][Dk][Dv] updated in place,
// core [M][HV Dv].  Dk = Dv = 128.
// scratch: gdn_chunk_scratch_bytes(M, HV) bytes on the device (what the state-independent half leaves for the other: 46 KB per
// chunk and value head).
size_t gdn_chunk_scratch_bytes(int M, int HV);
int gdn_chunk_launch(const float* post, const float* g, const float* beta, int M, int Hk, int HV, int Dk, int Dv, float* state, float* core,
                     void* scratch, cudaStream_t s);

}  // namespace lb
