// Launchers of the verify step's non-GEMM kernels (sm_100a).  Raw device pointers + a stream, like the reference's
// kernel layer (src/core/kernels.cuh:82-578 in the reference project); shapes come from the structs below.
#pragma once

#include "../../include/ling_b200.h"
#include "common.cuh"

namespace lb {

constexpr int kTreeRows = LING_B200_MAX_TREE_ROWS;
constexpr int kAttnChunk = 512;    // context keys per flash-decoding chunk
constexpr int kAttnChunkShort = 256;  // ... of a step with so few sequences that the shorter chunks still fit one wave of CTAs
constexpr int kAttnTcRows = 128;   // query rows per work item of the tcgen05 attention (the MMA's M)
constexpr int kAttnKeyTile = 64;   // keys per shared-memory tile
constexpr int kAttnRowTile = 48;   // query rows (token rows x q heads of one kv head) per CTA: three m16 tiles
constexpr float kPScale = 256.f;   // attention: p * v_scale is carried in FP16 times this power of two (clear of subnormals)
constexpr int kMaxPlanes = 8;      // most K splits of one GEMM (partial-sum planes a consumer adds)

// One sequence of the staged step as the device sees it.
struct SeqDev {
  int slot, pos, rope_delta, n_rows, chain, has_force;
};

// The step's device-resident description.  Host-written parts arrive with one copy from pinned memory; the packed
// arrays are built by pack_kernel.
// Per sequence, built by pack_kernel beside the tree description for the fused DeltaNet kernel: of every DeltaNet path
// its distinct rows in step order (a row's conv taps are its ancestors, which the path contains), their count and the
// rows the path writes; of every row its three conv taps (the ancestors at depths d-3 .. d-1, or -3 .. -1 for the
// session's window entries 0 .. 2 before depth 0; src/core/kernels.cu:365-383).
struct GdnAux {
  int np[LING_B200_MAX_TREE_VARIANTS];
  uint32_t wmask[LING_B200_MAX_TREE_VARIANTS];
  uint8_t prow[LING_B200_MAX_TREE_VARIANTS][LING_B200_MAX_TREE_ROWS];
  signed char tap[LING_B200_MAX_TREE_ROWS][4];
};

// Weights that a long glue kernel's idle CTAs ask into L2 for the GEMMs behind it (HBM is idle while such a kernel runs):
// up to four byte ranges, requested `delay_ns` after the kernel's dependency wait so that the kernel's own first loads
// are not queued behind them.  Ranges are 16-byte aligned; bytes = 0 skips a range.
struct PrefetchPlan {
  static constexpr int kRanges = 4;
  const void* p[kRanges] = {nullptr, nullptr, nullptr, nullptr};
  unsigned long long bytes[kRanges] = {0, 0, 0, 0};
  int delay_ns = 0;
};

struct StepBuffers {
  // host-written (one contiguous block, see Context::stage)
  int* n_seqs = nullptr;      // [1]
  SeqDev* seqs = nullptr;     // [max_seqs]
  int* in_parent = nullptr;   // [max_seqs][32]
  int* in_token = nullptr;    // [max_seqs][32]
  int* in_force = nullptr;    // [max_seqs][32]
  // built on the device
  int* row0 = nullptr;        // [max_seqs + 1]
  int* n_rows_total = nullptr;  // [1]
  int* token = nullptr;       // [rows]
  int* seq_of = nullptr;      // [rows]
  int* local = nullptr;       // [rows] row index inside its sequence
  int* depth = nullptr;       // [rows]
  int* rope_pos = nullptr;    // [rows]
  int* cache_slot = nullptr;  // [rows]
  uint32_t* anc = nullptr;    // [rows]
  ling_b200_tree_desc* trees = nullptr;  // [max_seqs]
  GdnAux* gdn_aux = nullptr;             // [max_seqs]
  // results
  int* argmax_id = nullptr;   // [rows]
  float* argmax_val = nullptr;
  ling_b200_seq_result* results = nullptr;  // [max_seqs]
  int* err = nullptr;         // [1] device error word
};

#ifdef __CUDACC__
// What a CTA without work does with a PrefetchPlan: its share (CTA `me` of `idle`) of every range, as 4 KB bulk prefetches.
__device__ __forceinline__ void prefetch_plan_share(const PrefetchPlan& plan, int me, int idle) {
  if (plan.delay_ns > 0) asm volatile("nanosleep.u32 %0;" ::"r"(unsigned(plan.delay_ns)));
  for (int r = 0; r < PrefetchPlan::kRanges; ++r) {
    const unsigned long long pieces = plan.bytes[r] / 4096ull;
    const char* base = static_cast<const char*>(plan.p[r]);
    for (unsigned long long i = (unsigned long long)me * blockDim.x + threadIdx.x; i < pieces; i += (unsigned long long)idle * blockDim.x)
      asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base + i * 4096ull), "r"(4096u) : "memory");
  }
}
// Keys per flash-decoding chunk of the staged step.  A step with few sequences has too few (sequence, kv head, 512-key
// chunk) items to occupy the SMs, and its attention time is one item's latency: when the items of 256-key chunks still fit
// one wave of `budget` CTAs the step uses those.  The attention kernel (tile_rows query rows per item) and the combine
// behind it evaluate the same rule on the same device-resident extents.
__device__ __forceinline__ int attn_chunk_keys(const StepBuffers& sb, int nseq, int Hkv, int G, int tile_rows, int budget) {
  if (nseq * Hkv * 2 > budget) return kAttnChunk;
  int items = 0;
  for (int s = 0; s < nseq; ++s) {
    const int nch = (sb.seqs[s].pos + kAttnChunkShort - 1) / kAttnChunkShort + 1;
    const int nrg = (sb.seqs[s].n_rows * G + tile_rows - 1) / tile_rows;
    items += Hkv * nch * nrg;
  }
  return items <= budget ? kAttnChunkShort : kAttnChunk;
}
#endif

struct ModelDims {
  int H, I, V, Hq, Hkv, D, rot, Hk, HV, Dk, Dv, C, Vs;
  float theta, eps;
  int n_attn, n_gdn;
  int page_tokens, pool_pages, max_pages;  // max_pages: entries of one slot's page table
  int rows_alloc;                          // allocated packed rows (multiple of 128)
  int max_seqs;
};

// The paged FP8 KV pool.  Codes: [attn layer][K|V][kv head][page] pages of page_tokens * D bytes; a K page is [token][D]
// (a key's D bytes contiguous: the score product reduces over D), a V page is [D][token] (one dim's tokens contiguous: the
// value product reduces over tokens), so both land in shared memory by 16-byte copies in the order the MMA fragments
// read them.  Scales: [..][page][token] fp32, one per (position, head).
struct KvPoolDev {
  uint8_t* codes = nullptr;
  float* scales = nullptr;
  int* tables = nullptr;  // [sessions][max_pages] page ids, 0 = unmapped
};
__host__ __device__ __forceinline__ size_t kv_slot_index(const ModelDims& d, int al, int kv, int h, int page, int tok) {
  return (((size_t(al) * 2 + kv) * d.Hkv + h) * size_t(d.pool_pages + 1) + page) * d.page_tokens + tok;
}

// Byte offset of element (position token `tok` of page `page`, dim dd) of K (kv = 0) or V (kv = 1).
__host__ __device__ __forceinline__ size_t kv_code_index(const ModelDims& d, int al, int kv, int h, int page, int tok, int dd) {
  const size_t page_base = kv_slot_index(d, al, kv, h, page, 0) * d.D;
  return kv ? page_base + size_t(dd) * d.page_tokens + tok : page_base + size_t(tok) * d.D + dd;
}

// A GEMM output as its consumers see it: `planes` partial sums (the K splits) to be added in order.
struct Planes {
  const float* p = nullptr;
  int n = 1;
  size_t stride = 0;  // floats between planes
  int ld = 0;         // floats between rows
};

// Quantized activation destination.
struct QuantOut {
  uint8_t* codes;
  float* scales;
  int K, K_pad, rows_alloc;
};

int kernels_init();
int pack_launch(const StepBuffers& sb, const ModelDims& d, cudaStream_t s);
// h (+= planes) -> h; xn = rmsnorm(h) (1 + w); xq = quant(xn).  ids != nullptr: h = embedding rows instead.
int norm_quant_launch(float* h, const Planes& add, const int* ids, const __nv_bfloat16* embed, const __nv_bfloat16* w,
                      float* xn, const QuantOut& q, const int* n_rows, int rows_grid, int H, float eps, cudaStream_t s);
// tap[m][:] = h[m][:] + planes (debug copy of the residual after a layer)
// h[m][:] += planes, in place
int add_planes_launch(float* h, const Planes& add, const int* n_rows, int rows_grid, int H, cudaStream_t s);
int tap_launch(const float* h, const Planes& add, float* out, const int* n_rows, int rows_grid, int H, cudaStream_t s);
int copy_rows_launch(const float* src, float* out, const int* n_rows, int rows_grid, int H, cudaStream_t s);
int kernels_norm_stamps(unsigned long long* stamps);  // debugging aid: five %globaltimer stamps of norm_quant's block (0, 0), or nullptr
// the same for the many rows of a prefill chunk (four rows x four heads a block)
int ab_gating_rows_launch(const float* xn, const __nv_bfloat16* wa, const __nv_bfloat16* wb, const __nv_bfloat16* A_log,
                          const __nv_bfloat16* dt_bias, float* g, float* beta, int M, int H, int HV, cudaStream_t s);
int ab_gating_launch(const float* xn, const __nv_bfloat16* wa, const __nv_bfloat16* wb, const __nv_bfloat16* A_log,
                     const __nv_bfloat16* dt_bias, float* g, float* beta, const int* n_rows, int rows_grid, int H, int HV,
                     cudaStream_t s);
int conv_tree_launch(const Planes& in, const StepBuffers& sb, const ModelDims& d, const __nv_bfloat16* convw,
                     const float* conv_state, size_t conv_slot_stride, float* pre, float* post, int rows_grid, cudaStream_t s);
int gdn_tree_launch(const float* post, const float* g, const float* beta, const StepBuffers& sb, const ModelDims& d,
                    const float* state, size_t state_slot_stride, float* core, int grid, cudaStream_t s);
// conv + recurrence + gated norm + FP8 copy in one launch (shapes: gdn_fused_supported); also stores pre and post
bool gdn_fused_supported(const ModelDims& d);
int gdn_fused_launch(const Planes& in, const StepBuffers& sb, const ModelDims& d, const __nv_bfloat16* convw, const float* conv_state,
                     size_t conv_slot_stride, const float* g, const float* beta, const float* state, size_t state_slot_stride,
                     const __nv_bfloat16* norm_w, const QuantOut& q, float* pre, float* post, float* core_out, int n_slots, int grid,
                     const PrefetchPlan& plan, unsigned long long* stamps, cudaStream_t s);  // core_out: [rows][HV * Dv] the recurrence's output before the gated norm, or nullptr; n_slots: sessions the state holds; stamps: seven %globaltimer values of block 0's first item (debugging aid) or nullptr
int gated_norm_quant_launch(const float* core, const Planes& z, int z_col, const __nv_bfloat16* w, const QuantOut& q,
                            const int* n_rows, int rows_grid, int HV, int Dv, float eps, cudaStream_t s);
int attn_prepare_launch(const Planes& qkv, const StepBuffers& sb, const ModelDims& d, int al, const __nv_bfloat16* q_norm,
                        const __nv_bfloat16* k_norm, __half* q, const KvPoolDev& kv, int rows_grid, cudaStream_t s);
int attention_launch(const __half* q, const StepBuffers& sb, const ModelDims& d, int al, const KvPoolDev& kv, float* part_o,
                     float* part_ml, int chunk_slots, int grid, cudaStream_t s);
// raw != nullptr: also the merged rows before the output gate, [rows][Hq * D] (the gate is then not applied: qkv.p may be null)
// The tcgen05/TMEM form of the same attention (attention_tc.cu): same inputs, same partial outputs.
int attention_tc_init();
bool attention_tc_supported(const ModelDims& d);
int attention_tc_launch(const __half* q, const StepBuffers& sb, const ModelDims& d, int al, const KvPoolDev& kv, float* part_o,
                        float* part_ml, int chunk_slots, int grid, const PrefetchPlan& plan, unsigned long long* stamps,
                        cudaStream_t s);  // plan: what CTAs without an item prefetch; stamps: see the kernel
// max_chunks: the most flash-decoding chunks one sequence can have (context capacity / kAttnChunkShort + 2);
// tile_rows, budget: the query rows per item and the grid of the attention kernel whose partials are merged (attn_chunk_keys)
int attn_combine_launch(const float* part_o, const float* part_ml, const Planes& qkv, const StepBuffers& sb,
                        const ModelDims& d, const QuantOut& q, float* raw, int rows_grid, int max_chunks, int tile_rows, int budget,
                        int chunk_slots, cudaStream_t s);  // chunk_slots: the partial buffers' capacity (slots past it are not read)
int f32_to_half_launch(const float* src, __half* dst, size_t n, cudaStream_t s);
int silu_mul_quant_launch(const Planes& gu, int I, int up_col0, const QuantOut& q, const int* n_rows, int rows_grid, cudaStream_t s);
int argmax_reduce_launch(const float* tile_val, const int* tile_idx, int tiles, int rows_alloc, int* ids, float* vals,
                         const int* n_rows, int rows_grid, cudaStream_t s);
int argmax_rows_launch(const float* logits, int rows, int vocab, int* ids, float* vals, cudaStream_t s);
int accept_launch(const StepBuffers& sb, const ModelDims& d, int commit, cudaStream_t s);
int kv_compact_launch(const StepBuffers& sb, const ModelDims& d, const KvPoolDev& kv, cudaStream_t s);
int conv_commit_launch(const StepBuffers& sb, const ModelDims& d, const float* pre, size_t layer_stride, float* conv_state,
                       size_t conv_slot_stride, size_t conv_layer_stride, cudaStream_t s);
int gdn_commit_launch(const StepBuffers& sb, const ModelDims& d, const float* post, const float* g, const float* beta,
                      size_t post_layer_stride, size_t g_layer_stride, float* state, size_t state_slot_stride,
                      size_t state_layer_stride, int grid, cudaStream_t s);
// weights and synthetic data
int quant_weight_launch(const float* src_f32, uint64_t key, float std_, int from_generator, uint8_t* codes, float* scales,
                        int row_off, int rows, int K, int N_pad, int K_pad, cudaStream_t s);
int quant_acts_launch(const float* x, int rows, const QuantOut& q, cudaStream_t s);
int fill_bf16_launch(const float* src_f32, uint64_t key, float std_, float bias, int from_generator, __nv_bfloat16* dst,
                     size_t n, cudaStream_t s);
int fill_f32_launch(uint64_t key, float std_, float* dst, size_t n, cudaStream_t s);
int kv_write_launch(const float* k, const float* v, uint64_t key_k, uint64_t key_v, int from_generator, const ModelDims& d,
                    int al, int slot, int from, int n, const KvPoolDev& kv, int* err, cudaStream_t s);
int kv_page_copy_launch(const ModelDims& d, const KvPoolDev& kv, int src, int dst, cudaStream_t s);
int flush_launch(float* buf, size_t n, cudaStream_t s);

}  // namespace lb
