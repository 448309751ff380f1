// NVFP4 GEMMs of the prefill chunk: y[m][n] = alpha * sum over blocks of 16 along K of
// sfx[m][blk] * sfw[n][blk] * dot(x4[m][blk], w4[n][blk]), values E2M1 (two a byte, the first in the low nibble),
// block scales E4M3 (one per 16 values), the two tensor scales folded into alpha.
//
// Stands in for the reference's prefill GEMMs over NVFP4 operands (src/core/prefill_gemm.cu:138-380,593-603,685-715 in the
// reference project: mma.sync kind::mxf4nvf4 with cp.async stages, which does not build for sm_100a), rebuilt for
// sm_100a: tcgen05.mma kind::mxf4nvf4.block_scale with the block scales in tensor memory (tcgen05.cp), operands by TMA
// into 128B-swizzled shared memory, a 128 x 256 accumulator tile in TMEM, one persistent CTA per SM.
#pragma once

#include "common.cuh"

namespace lb {

constexpr int kFp4TileM = 128;   // token rows per tile (the MMA's M)
constexpr int kFp4TileN = 256;   // weight rows per tile (the MMA's N); gate|up of 128 features in the fused form
constexpr int kFp4StageK = 256;  // K elements per pipeline stage: 128 bytes a row, four MMAs of K = 64

// Block scales on the device are kept in the order the tensor core's scale copy reads them: for every group of 128 rows
// and every 64 values of K (four blocks of 16) one 512-byte atom, byte (r % 32) * 16 + (r / 32) * 4 + j for row r of
// the group and block j of the four.  Atoms of one row group are consecutive along K; K is padded to whole stages.
__host__ __device__ inline size_t fp4_sf_offset(int row, int blk16, int k_atoms) {
  return (size_t(row >> 7) * k_atoms + size_t(blk16 >> 2)) * 512 + size_t(row & 31) * 16 + size_t((row & 127) >> 5) * 4 + size_t(blk16 & 3);
}
inline int fp4_k_atoms(int K) { return round_up(K, kFp4StageK) / 64; }
inline size_t fp4_sf_bytes(int rows, int K) { return size_t(round_up(rows, kFp4TileN) / 128) * fp4_k_atoms(K) * 512; }

// One NVFP4 operand on the device: a weight matrix [rows = N][K] or quantized activations [rows = M][K].
struct Fp4Operand {
  uint8_t* codes = nullptr;  // [rows][K / 2]
  uint8_t* sf = nullptr;     // fp4_sf_bytes(rows_alloc, K), layout above; rows and K blocks past the extent hold zero
  int rows = 0, K = 0;
  CUtensorMap map;           // {K / 2 bytes, rows}, box {128 bytes, 128 rows}, 128B swizzle; rows past the extent read zero
  CUtensorMap sf_map;        // the scales as [row groups][k_atoms * 512 bytes], box = one row group's 2 KiB of a stage
};
int make_fp4_map(Fp4Operand& o);

struct Fp4GemmCall {
  const Fp4Operand* X = nullptr;   // activations, M = X->rows
  const Fp4Operand* W = nullptr;   // plain: the weight [N][K]; fused: the gate projection
  const Fp4Operand* W2 = nullptr;  // fused: the up projection (same shape), else nullptr
  float alpha = 1.f, alpha2 = 1.f;
  // plain: y[m * ldy + n] = alpha * acc (or += with accumulate)
  float* y = nullptr;
  int ldy = 0;
  bool accumulate = false;
  // fused: NVFP4(bf16(silu(alpha * gate) * (alpha2 * up))) under the global scale gscale_out, codes [M][N / 2], block
  // scales in the layout above for an operand of N columns (sf_out_tiled) or row-major [M][N / 16]
  uint8_t* q_out = nullptr;
  uint8_t* sf_out = nullptr;
  bool sf_out_tiled = true;
  float gscale_out = 1.f;
  int* err_flag = nullptr;
  int ctas = 0;  // 0: one per SM
  int pair = -1; // 1: the two-CTA form (cta_group::2, 256 x 256 tiles per pair); 0: one CTA per tile; -1: the library's choice
  unsigned long long* stats = nullptr;  // optional, 4 zeroed words: cycle sums over the CTAs (issuer waiting for stages,
                                        // issuer waiting for the epilogue, one epilogue warp busy, whole CTA)
};
int fp4_init();
// The form used by calls that leave Fp4GemmCall::pair at -1 (process-wide): 0 one CTA per tile, 1 the two-CTA form.  Returns the
// previous setting.
int fp4_set_pair_mode(int mode);
int fp4_gemm_launch(const Fp4GemmCall& c, cudaStream_t stream);

// x (and, with up, silu(x) * up) [M][K] fp32 -> NVFP4 under the global scale gscale (= 1 / input_scale): values rounded
// to BF16 first, block scale E4M3(gscale * amax / 6), codes E2M1(x * gscale / scale) to nearest even (the reference's
// put_nvfp4, src/core/prefill_gemm.cu:383-394,408-420).  sf in the layout above (tiled) or row-major [M][K / 16].
int fp4_quant_act_launch(const float* x, const float* up, int M, int K, float gscale, uint8_t* q, uint8_t* sf, bool tiled,
                         cudaStream_t stream);
// Gemma RMSNorm of each row, x * rstd * (1 + w), into NVFP4 as above and, when out is given, into fp32 too
// (src/core/prefill_gemm.cu:426-459).
int fp4_rmsnorm_quant_launch(const float* x, const __nv_bfloat16* w, float* out, int M, int H, float eps, float gscale, uint8_t* q,
                             uint8_t* sf, bool tiled, cudaStream_t stream);
// The DeltaNet mixer's gated RMSNorm per head of 128 (src/core/kernels.cu:543-554), core [M][K] and z [M][K] fp32, the plain
// weight w [128], into NVFP4 as above: the out projection's input on the prefill path.
int fp4_gated_norm_quant_launch(const float* core, const float* z, const __nv_bfloat16* w, int M, int K, float eps, float gscale,
                                uint8_t* q, uint8_t* sf, bool tiled, cudaStream_t stream);
// BF16 weights [N][K] on the device -> NVFP4 in the checkpoints' rounding (the reference's host-side quantize_nvfp4,
// src/core/model.cu:188-249): tensor scale g = amax / (448 * 6) into *scale2 (device), block scales
// max(amax16 / 6 / g, 2^-9) as E4M3, codes nearest with ties to the smaller magnitude.  `amax_bits` is one zeroed word.
int fp4_quant_weight_launch(const __nv_bfloat16* w, int N, int K, uint8_t* q, uint8_t* sf, bool tiled, float* scale2,
                            unsigned* amax_bits, cudaStream_t stream);
// `ctas` CTAs each issue `iters` groups of four 128 x 256 x 64 NVFP4 MMAs on resident operands (the tensor pipe's rate).
// mode 0: MMAs only; 1: with the GEMM's twelve scale copies per group into one TMEM region; 2: into two regions in turn; 3: the
// copies issued by a second thread into a region the MMAs do not read; 4: the same 48 columns by six 128x256b copies.
int fp4_tensor_peak_launch(int ctas, int iters, int mode, int* err_flag, cudaStream_t stream);
// Row-major block scales [rows][K / 16] <-> the layout above.
int fp4_sf_tile_launch(const uint8_t* rowmajor, uint8_t* tiled, int rows, int K, cudaStream_t stream);
int fp4_sf_untile_launch(const uint8_t* tiled, uint8_t* rowmajor, int rows, int K, cudaStream_t stream);

}  // namespace lb
