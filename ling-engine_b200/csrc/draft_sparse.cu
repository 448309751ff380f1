// draft_sparse.cu -- the drafter's sparse LM head: which rows of the target's head a draft step scores
// (src/core/sparse_head.cu; Engine::draft_launch's head, src/core/speculate.cpp:598-610).
//
// Instead of all of the vocabulary a draft step scores (1) the rows its session's mask marks (a fixed list of frequent
// tokens joined with every token id of the session's prompt and output) and (2) the `dynamic` rows that a rank-256 factor of
// the head rates best for this step's rows: approx[n] = max over the step's rows m of p[m] . us[n], p = x . Vt^T (the
// selector_project kernel), us [vocab][256] BF16.  The selected rows, in id order, are gathered into a compact FP8
// matrix which the head GEMM then multiplies like any other: a selected row's logit is the full head's, bit for bit.
//
//   sparse_scores_kernel   HBM-bound: reads us once (vocab x 512 bytes); BF16 mma.sync m16n8k16 with the K index permuted so
//                          that a lane's fragments are 16-byte loads; writes an order-preserving 32-bit key per row, 0 = marked
//   sparse_level_kernel    radix select of the `dynamic`-th largest key, 11 + 11 + 10 bits: per level one histogram launch whose
//                          last block (a ticket) finds the bin the threshold falls in
//   sparse_count / _scan / _scatter   the ids of (marked or key >= threshold) in ascending order, at most `cap`
//   sparse_gather_kernel   the selected rows' FP8 codes and 1 x 128 block scales into the compact matrix
#include <cfloat>

#include "draft_head.h"

namespace lb {
namespace {

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

// keys[n] = marked ? 0 : order_key(max_m p[m] . us[n]).  A warp takes 16 rows of us at a time as the MMA's A tile and the
// step's rows (BF16, in shared memory) as B, eight rows per MMA column tile.  The sum over the rank runs in a permuted
// order: lane (g, t) of the fragment layout supplies, at k-step s, the rank indices 64 t + 4 s .. + 3 of rows g and g + 8 --
// a lane's 64 values of a row are then four 16-byte loads per half row, and B's matching four values are 8 contiguous bytes.
template <int NT>
__global__ void __launch_bounds__(256) sparse_scores_kernel(const float* __restrict__ p, int M, const __nv_bfloat16* __restrict__ us,
                                                            int N, SparseMasks masks, uint32_t* __restrict__ keys) {
  pdl_sync();  // first statement: see common.cuh
  constexpr int LD = kRank + 8;  // padded: the eight rows g of a B fragment read fall in different banks
  __shared__ __align__(16) __nv_bfloat16 ps[NT * 8 * LD];
  for (int i = threadIdx.x; i < NT * 8 * kRank; i += blockDim.x) {
    const int m = i / kRank, r = i % kRank;
    ps[m * LD + r] = __float2bfloat16(m < M ? p[size_t(m) * kRank + r] : 0.f);
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int n_warps = gridDim.x * (blockDim.x >> 5), warp = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  for (int n0 = warp * 16; n0 < N; n0 += n_warps * 16) {
    uint4 lo[8], hi[8];  // rows n0 + g and n0 + g + 8: rank indices 64 t .. 64 t + 63
    {
      const uint4* a = reinterpret_cast<const uint4*>(us + size_t(min(n0 + g, N - 1)) * kRank + t * 64);
      const uint4* b = reinterpret_cast<const uint4*>(us + size_t(min(n0 + g + 8, N - 1)) * kRank + t * 64);
#pragma unroll
      for (int q = 0; q < 8; ++q) lo[q] = __ldg(a + q), hi[q] = __ldg(b + q);
    }
    // the two rows' mask bytes travel with the rows (lanes t = 0 write the keys): asked for now, needed after the products
    bool m0 = false, m1 = false;
    if (t == 0) {
      if (n0 + g < N) m0 = any_mask(masks, n0 + g);
      if (n0 + g + 8 < N) m1 = any_mask(masks, n0 + g + 8);
    }
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
#pragma unroll
    for (int s = 0; s < 16; ++s) {
      const uint4 &x = lo[s >> 1], &y = hi[s >> 1];
      const uint32_t a0 = (s & 1) ? x.z : x.x, a2 = (s & 1) ? x.w : x.y;
      const uint32_t a1 = (s & 1) ? y.z : y.x, a3 = (s & 1) ? y.w : y.y;
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const uint2 b = *reinterpret_cast<const uint2*>(ps + (j * 8 + g) * LD + t * 64 + 4 * s);
        mma_bf16_16816(acc[j], a0, a1, a2, a3, b.x, b.y);
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
      if (n0 + g < N) keys[n0 + g] = m0 ? 0u : order_key(top0);
      if (n0 + g + 8 < N) keys[n0 + g + 8] = m1 ? 0u : order_key(top1);
    }
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
                         int sm_count, int* rows, int* nrows, cudaStream_t s, bool scores_only) {
  if (M < 1 || M > 32 || N < 1 || masks.n < 1 || masks.n > kSparseMasks || dynamic < 0 || cap < 1) {
    set_error("sparse_select: 1 to 32 rows, 1 to 4 masks, a positive capacity");
    return LING_B200_ERR_ARG;
  }
  uint8_t* base = static_cast<uint8_t*>(scratch);
  uint32_t* keys = reinterpret_cast<uint32_t*>(base);
  uint32_t* state = reinterpret_cast<uint32_t*>(base + ((size_t(N) * 4 + 63) & ~size_t(63)));
  uint32_t* hist = state + 16;
  int* counts = reinterpret_cast<int*>(hist + 3 * kBins);
  const int blocks = (N + 1023) / 1024;
  LB_CUDA(cudaMemsetAsync(state, 0, (16 + 3 * size_t(kBins)) * 4, s));
  const dim3 grid(sm_count * 2);
  if (M <= 8) LB_CUDA(launch_kernel(sparse_scores_kernel<1>, grid, dim3(256), size_t(0), s, p, M, us, N, masks, keys));
  else if (M <= 16) LB_CUDA(launch_kernel(sparse_scores_kernel<2>, grid, dim3(256), size_t(0), s, p, M, us, N, masks, keys));
  else LB_CUDA(launch_kernel(sparse_scores_kernel<4>, grid, dim3(256), size_t(0), s, p, M, us, N, masks, keys));
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
