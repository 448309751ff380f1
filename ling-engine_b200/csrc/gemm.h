// Block-scaled FP8 weight GEMM of the verify step: y[m][n] = sum over 128-wide K blocks of
// dot(x8[m][blk], w8[n][blk]) * xs[blk][m] * ws[blk][n].
//
// Stands in for the reference's weight-streaming rows GEMM (src/core/stream_gemm.cu:181-349,674-703 in the
// reference project), rebuilt for sm_100a: weights are the MMA's M dimension (128 rows a tile), the packed token
// rows its N dimension, operands arrive by TMA into 128B-swizzled shared memory, each 128-wide K block is one
// tcgen05.mma group into a TMEM accumulator that four epilogue warps drain and promote with the two block scales.
#pragma once

#include "common.cuh"

namespace lb {

constexpr int kTileN = 128;   // weight rows per tile (the MMA's M)
constexpr int kBlockK = 128;  // K per block scale and per pipeline stage (bytes: E4M3)

// One FP8 weight matrix on the device, padded to whole tiles (padding rows/columns are zero codes).
struct Fp8Matrix {
  uint8_t* codes = nullptr;  // [N_pad][K_pad]
  float* scales = nullptr;   // [KB][N_pad]   (block-major: one stage reads 128 consecutive floats)
  int N = 0, K = 0, N_pad = 0, K_pad = 0, KB = 0;
  int splits = 1;            // fixed K split of this shape (never depends on the row count: row invariance)
  CUtensorMap map;           // {K_pad, N_pad}, box {128, 128}, 128B swizzle
  size_t bytes() const { return size_t(N_pad) * K_pad + size_t(KB) * N_pad * 4; }
};

// Quantized activations: codes [rows_alloc][K_pad], scales [KB][rows_alloc].
struct Fp8Acts {
  uint8_t* codes = nullptr;
  float* scales = nullptr;
  int rows_alloc = 0, K = 0, K_pad = 0, KB = 0;
  CUtensorMap map[4];  // box rows 32, 64, 96, 128
};

// Optional fused epilogue of the LM head: per (tile, row) the best (value, vocabulary id), ties to the lower id,
// NaN skipped (reference rule: src/core/topk.cu:19,58).
struct HeadEpilogue {
  float* tile_val = nullptr;  // [N_pad/128][rows_alloc]
  int* tile_idx = nullptr;
  int rows_alloc = 0;
  bool store_logits = false;
};

// The gate|up projection with its activation fused in: the CTA that finishes a (gate tile, up tile) pair last adds the K
// splits' planes, applies silu(gate) * up and writes the FP8 copy the down projection reads (what silu_mul_quant_kernel
// does as a launch of its own, bit for bit).  tickets: one zeroed word per (token tile, gate tile); they return to zero.
struct SwigluEpilogue {
  unsigned* tickets = nullptr;
  int I = 0, up_col0 = 0;
  uint8_t* codes = nullptr;
  float* scales = nullptr;
  int K_pad = 0, rows_alloc = 0;
};

struct GemmCall {
  const Fp8Matrix* W = nullptr;
  const Fp8Acts* X = nullptr;
  int M = 0;                // real rows
  float* out = nullptr;     // [splits][M][ld]; column n of the matrix lands at out[m * ld + n]
  int ld = 0;
  size_t split_stride = 0;  // floats between split planes
  const HeadEpilogue* head = nullptr;
  const SwigluEpilogue* swiglu = nullptr;  // tcgen05 path only
  int impl = 0;             // 0 tcgen05, 1 CUDA cores
  int force_tile = 0;       // 0: token_tile(M); else the token tile to use (32, 64, 96 or 128): results do not depend on it
  int* err_flag = nullptr;
  unsigned long long* timeline = nullptr;  // four stamps of this launch (debugging aid), or nullptr
};

// Tensor map of a row-major byte matrix [rows][row_bytes] read in boxes of 128 bytes x box_rows under the 128B swizzle
// (row_bytes a multiple of 16; rows and bytes past the extent read zero).
int encode_tile_map(CUtensorMap* map, void* base, uint64_t row_bytes, uint64_t rows, uint32_t box_rows);
// Tensor map of a row-major byte matrix read in unswizzled boxes of box_bytes (at most 2048, a multiple of 16) of one row:
// the box lands as box_bytes consecutive bytes.  Coordinates count 8-byte words.
int encode_linear_map(CUtensorMap* map, void* base, uint64_t row_bytes, uint64_t rows, uint32_t box_bytes);
// Creates the tensor maps (driver entry point fetched at run time; no link against libcuda).
int make_weight_map(Fp8Matrix& w);
int make_acts_maps(Fp8Acts& x);
// The K split used for a shape: enough tiles x splits to cover the SMs about twice, at least 4 K blocks a split.
int choose_splits(int N_pad, int KB, int sm_count);
int gemm_init();
int gemm_launch(const GemmCall& c, cudaStream_t stream);
// `ctas` CTAs each issue `iters` 128 x 256 x 128 FP8 MMA groups on resident operands (the tensor pipe's sustained rate).
int tensor_peak_launch(int ctas, int iters, int* err_flag, cudaStream_t stream);
// One CTA waits, with the kernels' bounded wait and the given limit, on a barrier that nobody arrives at: records
// kDevWaitFull in *err_flag and the nanoseconds it waited, and returns.
int wait_probe_launch(unsigned long long limit_ns, int* err_flag, unsigned long long* waited_ns, cudaStream_t stream);
// Token rows per MMA (the N of the instruction) used for M rows: 32, 64, 96 or 128 (beyond 128 rows: the one with the least
// padding over ceil(M / tile) tiles).
int token_tile(int M);

}  // namespace lb
