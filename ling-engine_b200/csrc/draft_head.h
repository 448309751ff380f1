// The drafter's last stage (draft_head.cu): top-K of logit rows, the candidate selector's projection and its lattice.
#pragma once

#include "../../include/ling_b200.h"
#include "common.cuh"

namespace lb {

constexpr int kTopMaxK = 64;   // topk_rows takes K <= 64 (src/core/kernels.cuh:400-410)
constexpr int kSelTop = 16;    // candidates per drafted position (DraftConfig::selector_top_k)
constexpr int kSelRank = 256;  // width of the selector's projection and of its two codebooks (draft_kernels.cu:330)

// Top-K of each row of x [rows][V]: values descending, ties to the lower index; a row with fewer than K rankable values
// (NaN never ranks) ends in (-FLT_MAX, 0x7fffffff) pairs.  scratch: topk_scratch_floats(rows, V, K) floats.
size_t topk_scratch_floats(int rows, int V, int K);
int topk_rows_launch(const float* x, int rows, int V, int K, float* scratch, float* vals, int* ids, cudaStream_t s);
// hp [E][256] = x [E][H] . W^T, W [256][H] BF16, H a multiple of 256.
int selector_project_launch(const float* x, const __nv_bfloat16* W, int E, int H, float* hp, cudaStream_t s);
// scores [E][16][16] from hp [E][256], cand / unary [E][16] and the predecessor / successor codebooks [vocab][256] BF16.
// anchor_dev, when given, is read instead of `anchor`.  An id outside [0, vocab) sets the error word (code 7) and is clamped.
int selector_lattice_launch(const float* hp, const int* cand, const float* unary, const __nv_bfloat16* P, const __nv_bfloat16* S,
                            int vocab, int anchor, const int* anchor_dev, int E, float* scores, int* err, cudaStream_t s);


// ---- the sparse head (draft_sparse.cu)
constexpr int kSparseMasks = 4;  // masks one selection joins (kMaxSeqs, src/core/kernels.cuh:52,300-303)
struct SparseMasks {
  const uint8_t* m[kSparseMasks];  // [vocab] bytes each, non-zero = the row is always scored
  int n;
};
size_t sparse_scratch_bytes(int N);
// rows [cap] = the ids every mask marks and the `dynamic` best of the others under approx[n] = max_m p[m] . us[n] (ties at the
// threshold all taken), ascending; *nrows their count, at most cap.  p [M][256] fp32, us [N][256] BF16 (16-byte aligned), 1 <= M <= 32.
// err: the device error word a bounded wait that runs out records its code in (may be null).
int sparse_select_launch(const float* p, int M, const __nv_bfloat16* us, int N, const SparseMasks& masks, int dynamic, int cap, void* scratch,
                         int sm_count, int* rows, int* nrows, int* err, cudaStream_t s, bool scores_only = false);  // scores_only: the keys alone (a timing aid)
// the selected rows' codes [cap][K_pad] and block scales [KB][cap_pad] out of an FP8 matrix (codes [N_pad][K_pad], scales [KB][N_pad])
int sparse_gather_launch(const uint8_t* codes, const float* scales, int N_pad, int K_pad, int KB, const int* rows, const int* nrows, int cap,
                         uint8_t* out_codes, float* out_scales, int cap_pad, cudaStream_t s);
int sparse_tail_launch(float* logits, int E, int ld, int cap, const int* nrows, cudaStream_t s);   // columns >= *nrows := -inf
int sparse_ids_launch(const int* rows, const int* nrows, int* ids, int n, cudaStream_t s);         // ids[i] = rows[ids[i]]
int sparse_mark_launch(uint8_t* mask, const int* ids, int n, int vocab, cudaStream_t s);           // mask[ids[i]] = 1

}  // namespace lb
