// draft_head.cu -- the last stage of the drafter, the part that turns its hidden rows into what build_tree takes: the top
// 16 tokens of every drafted position under the target's LM head, the candidate selector's projection, and the selector's
// 16 x 16 transition scores between consecutive positions' candidates (Engine::draft_launch from its final norm on,
// src/core/speculate.cpp:598-617; topk_rows, src/core/topk.cu:83-129; selector_lattice, src/core/draft_kernels.cu:328-351).
// The drafter's transformer body, which produces the hidden rows, is not part of this library.
#include <cfloat>

#include "draft_head.h"

namespace lb {
namespace {

__device__ __forceinline__ bool ahead(float v, int i, float v2, int i2) { return v > v2 || (v == v2 && i < i2); }

// The K best of the (value, index) pairs spread over the block's threads, kTopPer + 1 each in registers: K rounds, each a
// block-wide argmax (value descending, ties to the lower index) whose winner is then struck out by the thread that holds
// it.  The winners go to win_v / win_i [K] in shared memory (past the pairs there are: -FLT_MAX, 0x7fffffff).  The extra
// slot carries the winners of the previous chunk when a list is longer than the block's registers.
constexpr int kTopThreads = 256, kTopPer = 8, kTopChunk = kTopThreads * kTopPer;
__device__ void block_topk(float (&v)[kTopPer + 1], int (&idx)[kTopPer + 1], int K, float* win_v, int* win_i, float* sv, int* si) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int round = 0; round < K; ++round) {
    float bv = -FLT_MAX;
    int bi = 0x7fffffff;
#pragma unroll
    for (int k = 0; k <= kTopPer; ++k)
      if (ahead(v[k], idx[k], bv, bi)) bv = v[k], bi = idx[k];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ahead(ov, oi, bv, bi)) bv = ov, bi = oi;
    }
    if (lane == 0) sv[warp] = bv, si[warp] = bi;
    __syncthreads();
    bv = sv[0], bi = si[0];
#pragma unroll
    for (int w = 1; w < kTopThreads / 32; ++w)
      if (ahead(sv[w], si[w], bv, bi)) bv = sv[w], bi = si[w];
    if (tid == 0) win_v[round] = bv, win_i[round] = bi;
#pragma unroll
    for (int k = 0; k <= kTopPer; ++k)
      if (idx[k] == bi) v[k] = -FLT_MAX, idx[k] = 0x7fffffff;  // an index occurs once
    __syncthreads();
  }
}

// The K best of a list of n pairs read through `get(e, value, index)`, chunk by chunk.
template <class Get>
__device__ void list_topk(Get get, int n, int K, float* out_v, int* out_i) {
  __shared__ float sv[kTopThreads / 32], win_v[kTopMaxK];
  __shared__ int si[kTopThreads / 32], win_i[kTopMaxK];
  const int tid = threadIdx.x;
  for (int c0 = 0; c0 == 0 || c0 < n; c0 += kTopChunk) {
    float v[kTopPer + 1];
    int idx[kTopPer + 1];
#pragma unroll
    for (int k = 0; k < kTopPer; ++k) {
      const int e = c0 + tid + k * kTopThreads;
      float val = -FLT_MAX;
      int id = 0x7fffffff;
      if (e < n) get(e, val, id);
      const bool real = val == val && val > -FLT_MAX && id != 0x7fffffff;  // a NaN never ranks
      v[k] = real ? val : -FLT_MAX, idx[k] = real ? id : 0x7fffffff;
    }
    const bool carry = c0 > 0 && tid < K;
    v[kTopPer] = carry ? win_v[tid] : -FLT_MAX, idx[kTopPer] = carry ? win_i[tid] : 0x7fffffff;
    block_topk(v, idx, K, win_v, win_i, sv, si);  // (its first barrier comes before its first write to win_*)
  }
  if (tid < K) out_v[tid] = win_v[tid], out_i[tid] = win_i[tid];
}

// Stage 1: block (segment, row) keeps the K best of its segment of the row.
__global__ void __launch_bounds__(kTopThreads)
    topk_segments_kernel(const float* __restrict__ x, int V, int K, int per, float* __restrict__ pv, int* __restrict__ pi) {
  pdl_sync();  // first statement: see common.cuh
  const int seg = blockIdx.x, row = blockIdx.y, start = seg * per, n = max(0, min(V, start + per) - start);
  const float* r = x + size_t(row) * V + start;
  const size_t o = (size_t(row) * gridDim.x + seg) * K;
  list_topk([&](int e, float& val, int& id) { val = r[e], id = start + e; }, n, K, pv + o, pi + o);
}

// Stage 2: one block per row merges the segments' lists.
__global__ void __launch_bounds__(kTopThreads)
    topk_merge_kernel(const float* __restrict__ pv, const int* __restrict__ pi, int n, int K, float* __restrict__ vals,
                      int* __restrict__ ids) {
  pdl_sync();  // first statement: see common.cuh
  const int row = blockIdx.x;
  const float* rv = pv + size_t(row) * n;
  const int* ri = pi + size_t(row) * n;
  list_topk([&](int e, float& val, int& id) { val = rv[e], id = ri[e]; }, n, K, vals + size_t(row) * K, ids + size_t(row) * K);
}

// hp[e][j] = x[e] . W[j]: W [kSelRank][H] in BF16, fp32 accumulation.  A warp owns an output column j and walks the weight
// row once for all the rows (kSelRows at a time in registers); lane l takes the elements 8 l .. 8 l + 7 of every 256.
constexpr int kSelRows = 8;
__global__ void __launch_bounds__(256)
    selector_project_kernel(const float* __restrict__ x, const __nv_bfloat16* __restrict__ W, int E, int H, float* __restrict__ hp) {
  pdl_sync();  // first statement: see common.cuh
  const int j = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (j >= kSelRank) return;
  for (int e0 = 0; e0 < E; e0 += kSelRows) {
    float acc[kSelRows];
#pragma unroll
    for (int r = 0; r < kSelRows; ++r) acc[r] = 0.f;
    for (int h = lane * 8; h < H; h += 256) {
      const uint4 wr = *reinterpret_cast<const uint4*>(W + size_t(j) * H + h);
      const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wr);
      float w[8];
#pragma unroll
      for (int k = 0; k < 4; ++k) w[2 * k] = __low2float(w2[k]), w[2 * k + 1] = __high2float(w2[k]);
#pragma unroll
      for (int r = 0; r < kSelRows; ++r)
        if (e0 + r < E) {
          const float4 a = *reinterpret_cast<const float4*>(x + size_t(e0 + r) * H + h);
          const float4 b = *reinterpret_cast<const float4*>(x + size_t(e0 + r) * H + h + 4);
          acc[r] = fmaf(a.x, w[0], fmaf(a.y, w[1], fmaf(a.z, w[2], fmaf(a.w, w[3], acc[r]))));
          acc[r] = fmaf(b.x, w[4], fmaf(b.y, w[5], fmaf(b.z, w[6], fmaf(b.w, w[7], acc[r]))));
        }
    }
#pragma unroll
    for (int r = 0; r < kSelRows; ++r) {
      const float s = warp_sum(acc[r]);
      if (lane == 0 && e0 + r < E) hp[size_t(e0 + r) * kSelRank + j] = s;
    }
  }
}

// score[e][p][c] = unary[e][c] + sum_r P[pred(e, p)][r] hp[e][r] S[cand[e][c]][r], pred(0, p) = the anchor, pred(e, p) =
// cand[e - 1][p].  One block per position e: the sixteen predecessor rows times hp and the sixteen successor rows go to
// shared memory (fp32), then thread (p, c) takes its dot product as four interleaved partial sums.
__global__ void __launch_bounds__(kSelTop * kSelTop)
    selector_lattice_kernel(const float* __restrict__ hp, const int* __restrict__ cand, const float* __restrict__ unary,
                            const __nv_bfloat16* __restrict__ P, const __nv_bfloat16* __restrict__ S, int vocab, int anchor,
                            const int* __restrict__ anchor_dev, float* __restrict__ scores, int* __restrict__ err) {
  pdl_sync();  // first statement: see common.cuh
  __shared__ float ph[kSelTop][kSelRank + 4], ss[kSelTop][kSelRank + 4];
  const int e = blockIdx.x, t = threadIdx.x;
  const int root = anchor_dev ? *anchor_dev : anchor;
  const float h = hp[size_t(e) * kSelRank + t];
  for (int i = 0; i < kSelTop; ++i) {
    int pid = e == 0 ? root : cand[(e - 1) * kSelTop + i], cid = cand[e * kSelTop + i];
    if (pid < 0 || pid >= vocab || cid < 0 || cid >= vocab) {  // a list shorter than 16 (ids 0x7fffffff) or a bad anchor
      if (t == 0) dev_fail(err, 7);
      pid = min(max(pid, 0), vocab - 1), cid = min(max(cid, 0), vocab - 1);
    }
    ph[i][t] = __bfloat162float(P[size_t(pid) * kSelRank + t]) * h;
    ss[i][t] = __bfloat162float(S[size_t(cid) * kSelRank + t]);
  }
  __syncthreads();
  const int p = t / kSelTop, c = t % kSelTop;
  float part[4] = {0.f, 0.f, 0.f, 0.f};
  for (int r = 0; r < kSelRank; r += 4) {
    const float4 a = *reinterpret_cast<const float4*>(&ph[p][r]);
    const float4 b = *reinterpret_cast<const float4*>(&ss[c][r]);
    part[0] = fmaf(a.x, b.x, part[0]), part[1] = fmaf(a.y, b.y, part[1]);
    part[2] = fmaf(a.z, b.z, part[2]), part[3] = fmaf(a.w, b.w, part[3]);
  }
  scores[(size_t(e) * kSelTop + p) * kSelTop + c] = unary[e * kSelTop + c] + ((part[0] + part[1]) + (part[2] + part[3]));
}

}  // namespace

// Segments per row: about a block's registers each, and few enough for their lists to be merged by one block in one chunk.
int topk_segments(int V, int K) { return std::max(1, std::min(ceil_div(V, kTopChunk), kTopChunk / K)); }
size_t topk_scratch_floats(int rows, int V, int K) { return size_t(rows) * topk_segments(V, K) * K * 2; }

int topk_rows_launch(const float* x, int rows, int V, int K, float* scratch, float* vals, int* ids, cudaStream_t s) {
  if (rows < 1 || V < 1 || K < 1 || K > kTopMaxK) return LING_B200_ERR_ARG;
  const int segs = topk_segments(V, K);
  float* pv = scratch;
  int* pi = reinterpret_cast<int*>(scratch + size_t(rows) * segs * K);
  LB_CUDA(launch_kernel(topk_segments_kernel, dim3(segs, rows), dim3(kTopThreads), size_t(0), s, x, V, K, ceil_div(V, segs), pv, pi));
  LB_LAUNCH("topk_segments_kernel");
  LB_CUDA(launch_kernel(topk_merge_kernel, dim3(rows), dim3(kTopThreads), size_t(0), s, (const float*)pv, (const int*)pi, segs * K, K, vals, ids));
  LB_LAUNCH("topk_merge_kernel");
  return LING_B200_OK;
}

int selector_project_launch(const float* x, const __nv_bfloat16* W, int E, int H, float* hp, cudaStream_t s) {
  if (E < 1 || H % 256 != 0) return LING_B200_ERR_ARG;
  LB_CUDA(launch_kernel(selector_project_kernel, dim3(kSelRank / 8), dim3(256), size_t(0), s, x, W, E, H, hp));
  LB_LAUNCH("selector_project_kernel");
  return LING_B200_OK;
}

int selector_lattice_launch(const float* hp, const int* cand, const float* unary, const __nv_bfloat16* P, const __nv_bfloat16* S,
                            int vocab, int anchor, const int* anchor_dev, int E, float* scores, int* err, cudaStream_t s) {
  if (E < 1 || vocab < 1) return LING_B200_ERR_ARG;
  LB_CUDA(launch_kernel(selector_lattice_kernel, dim3(E), dim3(kSelTop * kSelTop), size_t(0), s, hp, cand, unary, P, S, vocab, anchor,
                        anchor_dev, scores, err));
  LB_LAUNCH("selector_lattice_kernel");
  return LING_B200_OK;
}

}  // namespace lb
