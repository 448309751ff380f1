// draft_sparse.cu -- the drafter's sparse LM head: which rows of the target's head a draft step scores
// (src/core/sparse_head.cu; Engine::draft_launch's head, src/core/speculate.cpp:598-610).
//
// Instead of all of the vocabulary a draft step scores (1) the rows its session's mask marks (a fixed list of frequent
// tokens joined with every token id of the session's prompt and output) and (2) the `dynamic` rows that a rank-256 factor of
// the head rates best for this step's rows: approx[n] = max over the step's rows m of p[m] . us[n], p = x . Vt^T (the
// selector_project kernel), us [vocab][256] BF16.  The selected rows, in id order, are gathered into a compact FP8
// matrix which the head GEMM then multiplies like any other: a selected row's logit is the full head's, bit for bit.
//
//   sparse_scores_kernel   HBM-bound: reads us once (vocab x 512 bytes) by TMA into a swizzled ring in shared memory; BF16 mma.sync
//                          m16n8k16 with ldmatrix fragments; writes an order-preserving 32-bit key per row, 0 = marked
//   sparse_level_kernel    radix select of the `dynamic`-th largest key, 11 + 11 + 10 bits: per level one histogram launch whose
//                          last block (a ticket) finds the bin the threshold falls in
//   sparse_count / _scan / _scatter   the ids of (marked or key >= threshold) in ascending order, at most `cap`
//   sparse_gather_kernel   the selected rows' FP8 codes and 1 x 128 block scales into the compact matrix
#include <cfloat>

#include "draft_head.h"
#include "gemm.h"
#include "tc.cuh"

namespace lb {
namespace {
using tc::smem_u32;

constexpr int kRank = kSelRank;
constexpr int kBins = 2048;

__device__ __forceinline__ uint32_t order_key(float f) {  // larger float, larger key; never 0 for a number
  const uint32_t b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ bool any_mask(const SparseMasks& ms, int n) {
  bool on = false;
#pragma unroll
  for (int i = 0; i < kSparseMasks; ++i)
    if (i < ms.n) on |= ms.m[i][n] != 0;
  return on;
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// keys[n] = marked ? 0 : order_key(max_m p[m] . us[n]).  One block per SM streams its share of us through a three-stage ring
// in shared memory, 128 rows (64 KB) a stage, as four TMA tiles of 128 rows x 128 bytes under the 128-byte swizzle (a
// byte-typed map of the factor, plain loads: this CTA's shared memory only), completing on the stage's mbarrier; warp w of the
// block then owns rows 16 w .. 16 w + 15 of the stage: A fragments by ldmatrix.x4 with the swizzle's XOR in the address (the
// eight rows of a matrix fall in different banks), the step's rows (BF16, converted once, rows padded) as the B operand by
// ldmatrix as well, sixteen k-steps of mma.sync m16n8k16 a column tile.  Every wait is bounded: one that runs out records a
// code in the error word, and the block makes no further waits and writes no further keys.
// (Earlier forms: fragments loaded straight from global memory, a lane per 128-byte quarter of a row -- 32 lines an
// instruction, load-unit bound at a third of the copy bandwidth; the ring filled by 16-byte cp.async -- 0.44; by one 512-byte
// bulk copy a row into padded rows -- 0.49: 128 small copies a stage.)
constexpr int kScoreRows = 128, kScoreStages = 3, kScoreLd = kRank + 8;  // (halves per padded row of the step's rows)
constexpr int kScoreStageBytes = kScoreRows * kRank * 2;                  // 64 KB: [k quarter][row][128 B]
template <int NT>
constexpr size_t score_smem() { return size_t(kScoreStages) * kScoreStageBytes + size_t(NT * 8) * kScoreLd * 2 + 1024 /* alignment */; }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x2(uint32_t (&r)[2], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(smem_u32(p)));
}
template <int NT>
__global__ void __launch_bounds__(256, 1) sparse_scores_kernel(const float* __restrict__ p, int M, const __grid_constant__ CUtensorMap map_us,
                                                               int N, SparseMasks masks, uint32_t* __restrict__ keys, int* err) {
  pdl_sync();  // first statement: see common.cuh
  extern __shared__ uint8_t score_raw[];
  uint8_t* ring = score_raw + ((1024u - (smem_u32(score_raw) & 1023u)) & 1023u);  // swizzled tiles: 1024-byte aligned
  __nv_bfloat16* ps = reinterpret_cast<__nv_bfloat16*>(ring + size_t(kScoreStages) * kScoreStageBytes);  // [NT * 8][264]
  __shared__ __align__(8) uint64_t full[kScoreStages];
  __shared__ volatile int failed;
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_us)) : "memory");
    for (int i = 0; i < kScoreStages; ++i) tc::mbar_init(&full[i], 1);
    failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int tiles = (N + kScoreRows - 1) / kScoreRows;
  const int mine = blockIdx.x < tiles ? (tiles - 1 - int(blockIdx.x)) / int(gridDim.x) + 1 : 0;  // tiles blockIdx.x, + gridDim.x, ...
  // stage i % 3 of the ring <- this block's i-th tile: four tiles of 128 bytes x 128 rows (rows past N arrive as zeros)
  auto send = [&](int i) {
    if (i >= mine || failed || threadIdx.x != 0) return;
    const int row0 = (int(blockIdx.x) + i * int(gridDim.x)) * kScoreRows;
    uint64_t* bar = &full[i % kScoreStages];
    uint8_t* dst = ring + size_t(i % kScoreStages) * kScoreStageBytes;
    const uint64_t pol = tc::policy_evict_first();  // the factor is read once
    tc::mbar_expect_tx(bar, uint32_t(kScoreStageBytes));
#pragma unroll
    for (int kq = 0; kq < 4; ++kq) tc::tma_load_2d(dst + kq * (kScoreRows * 128), &map_us, bar, kq * 128, row0, pol);
  };
  send(0), send(1);
  for (int i = threadIdx.x; i < NT * 8 * kRank; i += blockDim.x) {
    const int m = i / kRank, r = i % kRank;
    ps[m * kScoreLd + r] = __float2bfloat16(m < M ? p[size_t(m) * kRank + r] : 0.f);
  }
  for (int i = 0; i < mine; ++i) {
    send(i + 2);  // into the stage that iteration i - 1 read: every warp is past it (the barrier that ended that iteration)
    if (i == 0) __syncthreads();  // ps is written
    if (!failed && !tc::mbar_wait(&full[i % kScoreStages], uint32_t(i / kScoreStages) & 1u, &failed)) {
      dev_fail(err, kDevWaitFull);
      failed = 1;
    }
    if (failed) {  // block-uniform once the barrier below has been passed; until then a thread that saw it only skips work
      __syncthreads();
      continue;
    }
    const int row0 = (int(blockIdx.x) + i * int(gridDim.x)) * kScoreRows + warp * 16;
    // lanes t = 0 write the keys of rows g and g + 8: their mask bytes are asked for now, needed after the products
    bool m0 = false, m1 = false;
    if (t == 0) {
      if (row0 + g < N) m0 = any_mask(masks, row0 + g);
      if (row0 + g + 8 < N) m1 = any_mask(masks, row0 + g + 8);
    }
    const uint8_t* stage = ring + size_t(i % kScoreStages) * kScoreStageBytes;
    const int arow = warp * 16 + (lane & 15);  // this lane's row of the stage for the A fragments
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
#pragma unroll 4
    for (int ks = 0; ks < kRank / 16; ++ks) {
      // A: rows 0-15 x k 16 ks .. + 15 as four 8 x 8 matrices (rows 0-7 / 8-15, k low / high): lane l addresses row l % 16 and the
      // 16-byte chunk 2 ks + l / 16 of its 512 bytes = chunk c % 8 of k quarter c / 8, at the swizzled position (c % 8) ^ (row % 8)
      uint32_t a[4];
      const int c = 2 * ks + (lane >> 4);
      ldsm_x4(a, stage + (c >> 3) * (kScoreRows * 128) + arow * 128 + (((c & 7) ^ (arow & 7)) << 4));
      if constexpr (NT == 1) {
        uint32_t b[2];  // step rows 0-7: k low / high; lanes 0-15 give the addresses
        ldsm_x2(b, ps + size_t(lane & 7) * kScoreLd + ks * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16_16816(acc[0], a[0], a[1], a[2], a[3], b[0], b[1]);
      } else {
#pragma unroll
        for (int j = 0; j < NT; j += 2) {
          uint32_t b[4];  // step rows 8 j .. 8 j + 15: (rows low, k low), (rows low, k high), (rows high, k low), (rows high, k high)
          ldsm_x4(b, ps + size_t(j * 8 + (lane & 7) + ((lane >> 4) & 1) * 8) * kScoreLd + ks * 16 + ((lane >> 3) & 1) * 8);
          mma_bf16_16816(acc[j], a[0], a[1], a[2], a[3], b[0], b[1]);
          mma_bf16_16816(acc[j + 1], a[0], a[1], a[2], a[3], b[2], b[3]);
        }
      }
    }
    // acc[j][e]: us row g (e = 0, 1) / g + 8 (e = 2, 3) against the step's row 8 j + 2 t + (e & 1)
    float top0 = -INFINITY, top1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e)
        if (j * 8 + 2 * t + e < M) top0 = fmaxf(top0, acc[j][e]), top1 = fmaxf(top1, acc[j][2 + e]);
    top0 = fmaxf(top0, __shfl_xor_sync(0xffffffffu, top0, 1)), top0 = fmaxf(top0, __shfl_xor_sync(0xffffffffu, top0, 2));
    top1 = fmaxf(top1, __shfl_xor_sync(0xffffffffu, top1, 1)), top1 = fmaxf(top1, __shfl_xor_sync(0xffffffffu, top1, 2));
    if (t == 0) {
      if (row0 + g < N) keys[row0 + g] = m0 ? 0u : order_key(top0);
      if (row0 + g + 8 < N) keys[row0 + g + 8] = m1 ? 0u : order_key(top1);
    }
    __syncthreads();  // every warp is done with the stage before iteration i + 1 sends tile i + 3 into it
  }
}

// One level of the radix select.  state: [0] the key prefix found so far, [1] how many keys at or above the threshold are
// still wanted below that prefix, [2] the tickets of this level, [3] the threshold (after level 2).  hist: kBins words of
// this level, zero on entry.  Every block histograms its share of the keys that carry the prefix; the block that takes the
// last ticket walks the bins from the top until `want` keys are covered.  If the keys run out first the walk ends in bin 0
// of every level and the threshold is 0, which selects no unmarked row at all (the reference's rule, sparse_head.cu:150-171).
__device__ __forceinline__ int level_shift(int level) { return level == 0 ? 21 : level == 1 ? 10 : 0; }
__device__ __forceinline__ uint32_t level_bins(int level) { return level == 2 ? 1024u : 2048u; }
__global__ void __launch_bounds__(512) sparse_level_kernel(const uint32_t* __restrict__ keys, int N, uint32_t* __restrict__ hist,
                                                           uint32_t* __restrict__ state, int level, int dynamic) {
  pdl_sync();  // first statement: see common.cuh
  __shared__ uint32_t h[kBins];
  __shared__ uint32_t part[512];
  __shared__ bool last;
  for (int i = threadIdx.x; i < kBins; i += blockDim.x) h[i] = 0;
  __syncthreads();
  const int shift = level_shift(level);
  const uint32_t bins = level_bins(level);
  const uint32_t keep = level == 0 ? 0u : level == 1 ? 0xffe00000u : 0xfffffc00u;
  const uint32_t prefix = level ? state[0] : 0u;
  for (int n = blockIdx.x * blockDim.x + threadIdx.x; n < N; n += gridDim.x * blockDim.x) {
    const uint32_t k = keys[n];
    if (k != 0 && (k & keep) == prefix) atomicAdd(&h[(k >> shift) & (bins - 1)], 1u);
  }
  __syncthreads();
  for (uint32_t i = threadIdx.x; i < bins; i += blockDim.x)
    if (h[i]) atomicAdd(&hist[i], h[i]);
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last = atomicAdd(&state[2], 1u) == gridDim.x - 1;
  __syncthreads();
  if (!last) return;
  __threadfence();
  // the last block: thread i sums bins [per i, per i + per); thread 0 walks the sums from the top, then the bins of the group
  const uint32_t per = bins / 512;
  uint32_t sum = 0;
  for (uint32_t b = threadIdx.x * per; b < (threadIdx.x + 1) * per; ++b) sum += __ldcg(hist + b);
  part[threadIdx.x] = sum;
  __syncthreads();
  if (threadIdx.x != 0) return;
  const uint32_t want = level ? state[1] : uint32_t(dynamic);
  uint32_t above = 0;
  int c = 511;
  for (; c > 0 && above + part[c] < want; --c) above += part[c];
  int b = c * int(per) + int(per) - 1;
  for (; b > c * int(per) && above + __ldcg(hist + b) < want; --b) above += __ldcg(hist + b);
  const uint32_t found = prefix | (uint32_t(b) << shift);
  state[0] = found;
  state[1] = want > above ? want - above : 0u;
  state[2] = 0u;
  if (level == 2) state[3] = found;
}

__device__ __forceinline__ bool selected(const uint32_t* keys, const SparseMasks& masks, int n, uint32_t thr) {
  const uint32_t k = keys[n];  // 0: marked by the scores kernel (the same masks)
  return k == 0 ? any_mask(masks, n) : (thr != 0 && k >= thr);
}
// per block of 1024 rows the number of selected ones
__global__ void __launch_bounds__(256) sparse_count_kernel(const uint32_t* __restrict__ keys, SparseMasks masks, int N,
                                                           const uint32_t* __restrict__ state, int* __restrict__ counts) {
  pdl_sync();  // first statement: see common.cuh
  __shared__ int red[8];
  const uint32_t thr = state[3];
  int c = 0;
  for (int i = 0; i < 4; ++i) {
    const int n = blockIdx.x * 1024 + i * 256 + threadIdx.x;
    c += n < N && selected(keys, masks, n, thr);
  }
  c = __reduce_add_sync(0xffffffffu, c);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0;
    for (int w = 0; w < 8; ++w) t += red[w];
    counts[blockIdx.x] = t;
  }
}
// exclusive prefix over the blocks' counts (one block), and the row count, bounded by the capacity
__global__ void __launch_bounds__(1024) sparse_scan_kernel(int* __restrict__ counts, int blocks, int cap, int* __restrict__ nrows) {
  pdl_sync();  // first statement: see common.cuh
  __shared__ int warp_tot[32];
  __shared__ int carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int b0 = 0; b0 < blocks; b0 += 1024) {
    const int b = b0 + threadIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int v = b < blocks ? counts[b] : 0;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += up;
    }
    if (lane == 31) warp_tot[warp] = inc;
    __syncthreads();
    int before = carry;
    for (int w = 0; w < warp; ++w) before += warp_tot[w];
    if (b < blocks) counts[b] = before + inc - v;
    __syncthreads();
    if (threadIdx.x == 1023) carry = before + inc;
    __syncthreads();
  }
  if (threadIdx.x == 0) *nrows = min(carry, cap);
}
// rows[rank] = n for every selected n, in ascending order; ranks at or past the capacity are dropped
__global__ void __launch_bounds__(256) sparse_scatter_kernel(const uint32_t* __restrict__ keys, SparseMasks masks, int N,
                                                             const uint32_t* __restrict__ state, const int* __restrict__ offsets, int cap,
                                                             int* __restrict__ rows) {
  pdl_sync();  // first statement: see common.cuh
  __shared__ int warp_tot[8];
  const uint32_t thr = state[3];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int base = offsets[blockIdx.x];
  for (int i = 0; i < 4; ++i) {
    const int n = blockIdx.x * 1024 + i * 256 + threadIdx.x;
    const bool on = n < N && selected(keys, masks, n, thr);
    const uint32_t ballot = __ballot_sync(0xffffffffu, on);
    if (lane == 0) warp_tot[warp] = __popc(ballot);
    __syncthreads();
    int before = base;
    for (int w = 0; w < warp; ++w) before += warp_tot[w];
    const int rank = before + __popc(ballot & ((1u << lane) - 1u));
    if (on && rank < cap) rows[rank] = n;
    int total = 0;
    for (int w = 0; w < 8; ++w) total += warp_tot[w];
    base += total;
    __syncthreads();
  }
}

// Row i of the compact matrix = row rows[i] of the head for i < *nrows: a block copies one row's codes sixteen bytes a thread
// and its block scales (scales are [K block][row], both matrices).  Rows past *nrows keep what an earlier step left there
// (zero at first): the logits of those columns are overwritten with -inf before anything reads them.
__global__ void __launch_bounds__(128) sparse_gather_kernel(const uint8_t* __restrict__ codes, const float* __restrict__ scales, int N_pad,
                                                            int K_pad, int KB, const int* __restrict__ rows, const int* __restrict__ nrows,
                                                            uint8_t* __restrict__ out_codes, float* __restrict__ out_scales, int cap_pad) {
  pdl_sync();  // first statement: see common.cuh
  const int i = blockIdx.x;
  if (i >= *nrows) return;
  const int src = rows[i];
  const uint4* from = reinterpret_cast<const uint4*>(codes + size_t(src) * K_pad);
  uint4* to = reinterpret_cast<uint4*>(out_codes + size_t(i) * K_pad);
  for (int c = threadIdx.x; c < K_pad / 16; c += blockDim.x) to[c] = __ldg(from + c);
  for (int kb = threadIdx.x; kb < KB; kb += blockDim.x) out_scales[size_t(kb) * cap_pad + i] = scales[size_t(kb) * N_pad + src];
}

// logits [E][ld]: columns at or past *nrows become -inf (the compact matrix's unused rows are zero, not absent)
__global__ void sparse_tail_kernel(float* __restrict__ logits, int E, int ld, int cap, const int* __restrict__ nrows) {
  pdl_sync();  // first statement: see common.cuh
  const int n = *nrows;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < E * cap; i += gridDim.x * blockDim.x) {
    const int col = i % cap;
    if (col >= n) logits[size_t(i / cap) * ld + col] = -INFINITY;
  }
}
// ids[i] = rows[ids[i]]: the compact matrix's columns back to token ids (an id past the rows there are stays as it is)
__global__ void sparse_ids_kernel(const int* __restrict__ rows, const int* __restrict__ nrows, int* __restrict__ ids, int n) {
  pdl_sync();  // first statement: see common.cuh
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n && ids[i] >= 0 && ids[i] < *nrows) ids[i] = rows[ids[i]];
}
__global__ void sparse_mark_kernel(uint8_t* __restrict__ mask, const int* __restrict__ ids, int n, int vocab) {
  pdl_sync();  // first statement: see common.cuh
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n && ids[i] >= 0 && ids[i] < vocab) mask[ids[i]] = 1;
}

}  // namespace

size_t sparse_scratch_bytes(int N) {
  // keys [N] u32, state (16 words), three levels' histograms, the per-block counts
  return size_t(N) * 4 + 64 + 3 * size_t(kBins) * 4 + size_t((N + 1023) / 1024) * 4 + 64;
}

int sparse_select_launch(const float* p, int M, const __nv_bfloat16* us, int N, const SparseMasks& masks, int dynamic, int cap, void* scratch,
                         int sm_count, int* rows, int* nrows, int* err, cudaStream_t s, bool scores_only) {
  if (M < 1 || M > 32 || N < 1 || masks.n < 1 || masks.n > kSparseMasks || dynamic < 0 || cap < 1) {
    set_error("sparse_select: 1 to 32 rows, 1 to 4 masks, a positive capacity");
    return LING_B200_ERR_ARG;
  }
  if (N < kScoreRows || (reinterpret_cast<uintptr_t>(us) & 15u) != 0) {
    set_error("sparse_select: the factor must have at least 128 rows and start on a 16-byte boundary (it is read by TMA tiles)");
    return LING_B200_ERR_ARG;
  }
  uint8_t* base = static_cast<uint8_t*>(scratch);
  uint32_t* keys = reinterpret_cast<uint32_t*>(base);
  uint32_t* state = reinterpret_cast<uint32_t*>(base + ((size_t(N) * 4 + 63) & ~size_t(63)));
  uint32_t* hist = state + 16;
  int* counts = reinterpret_cast<int*>(hist + 3 * kBins);
  const int blocks = (N + 1023) / 1024;
  LB_CUDA(cudaMemsetAsync(state, 0, (16 + 3 * size_t(kBins)) * 4, s));
  static bool attr_set = false;
  if (!attr_set) {
    LB_CUDA(cudaFuncSetAttribute(sparse_scores_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(score_smem<1>())));
    LB_CUDA(cudaFuncSetAttribute(sparse_scores_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(score_smem<2>())));
    LB_CUDA(cudaFuncSetAttribute(sparse_scores_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(score_smem<4>())));
    attr_set = true;
  }
  CUtensorMap map_us;  // the factor as bytes: rows of 512, tiles of 128 bytes x 128 rows, 128-byte swizzle
  if (const int rc = encode_tile_map(&map_us, const_cast<__nv_bfloat16*>(us), uint64_t(kRank) * 2, uint64_t(N), kScoreRows)) return rc;
  const dim3 grid(sm_count);
  if (M <= 8) LB_CUDA(launch_kernel(sparse_scores_kernel<1>, grid, dim3(256), score_smem<1>(), s, p, M, map_us, N, masks, keys, err));
  else if (M <= 16) LB_CUDA(launch_kernel(sparse_scores_kernel<2>, grid, dim3(256), score_smem<2>(), s, p, M, map_us, N, masks, keys, err));
  else LB_CUDA(launch_kernel(sparse_scores_kernel<4>, grid, dim3(256), score_smem<4>(), s, p, M, map_us, N, masks, keys, err));
  LB_LAUNCH("sparse_scores_kernel");
  if (scores_only) return LING_B200_OK;
  for (int level = 0; level < 3; ++level) {
    LB_CUDA(launch_kernel(sparse_level_kernel, dim3(sm_count), dim3(512), size_t(0), s, (const uint32_t*)keys, N, hist + level * kBins, state, level,
                          dynamic));
    LB_LAUNCH("sparse_level_kernel");
  }
  LB_CUDA(launch_kernel(sparse_count_kernel, dim3(blocks), dim3(256), size_t(0), s, (const uint32_t*)keys, masks, N, (const uint32_t*)state, counts));
  LB_LAUNCH("sparse_count_kernel");
  LB_CUDA(launch_kernel(sparse_scan_kernel, dim3(1), dim3(1024), size_t(0), s, counts, blocks, cap, nrows));
  LB_LAUNCH("sparse_scan_kernel");
  LB_CUDA(launch_kernel(sparse_scatter_kernel, dim3(blocks), dim3(256), size_t(0), s, (const uint32_t*)keys, masks, N, (const uint32_t*)state,
                        (const int*)counts, cap, rows));
  LB_LAUNCH("sparse_scatter_kernel");
  return LING_B200_OK;
}

int sparse_gather_launch(const uint8_t* codes, const float* scales, int N_pad, int K_pad, int KB, const int* rows, const int* nrows, int cap,
                         uint8_t* out_codes, float* out_scales, int cap_pad, cudaStream_t s) {
  LB_CUDA(launch_kernel(sparse_gather_kernel, dim3(cap), dim3(128), size_t(0), s, codes, scales, N_pad, K_pad, KB, rows, nrows, out_codes, out_scales,
                        cap_pad));
  LB_LAUNCH("sparse_gather_kernel");
  return LING_B200_OK;
}

int sparse_tail_launch(float* logits, int E, int ld, int cap, const int* nrows, cudaStream_t s) {
  LB_CUDA(launch_kernel(sparse_tail_kernel, dim3(ceil_div(E * cap, 256)), dim3(256), size_t(0), s, logits, E, ld, cap, nrows));
  LB_LAUNCH("sparse_tail_kernel");
  return LING_B200_OK;
}

int sparse_ids_launch(const int* rows, const int* nrows, int* ids, int n, cudaStream_t s) {
  LB_CUDA(launch_kernel(sparse_ids_kernel, dim3(ceil_div(n, 256)), dim3(256), size_t(0), s, rows, nrows, ids, n));
  LB_LAUNCH("sparse_ids_kernel");
  return LING_B200_OK;
}

int sparse_mark_launch(uint8_t* mask, const int* ids, int n, int vocab, cudaStream_t s) {
  if (n <= 0) return LING_B200_OK;
  LB_CUDA(launch_kernel(sparse_mark_kernel, dim3(ceil_div(n, 256)), dim3(256), size_t(0), s, mask, ids, n, vocab));
  LB_LAUNCH("sparse_mark_kernel");
  return LING_B200_OK;
}

}  // namespace lb
