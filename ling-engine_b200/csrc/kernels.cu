// kernels.cu -- the verify step's non-GEMM kernels for sm_100a: ragged packing and tree description on the device,
// fused residual + RMSNorm + FP8 quantization, the gated-DeltaNet conv/recurrence over trees and its commit,
// tree-masked attention over the paged FP8 KV cache, argmax, greedy acceptance and KV compaction.
// Every kernel reads its real extents (rows, sequences) from device memory, so one captured graph serves any step
// of the same capacity class.  Citations name the reference project's files (dreamference/ling-engine).
#include "kernels.h"

#include <cooperative_groups.h>

#include <cfloat>

namespace lb {
namespace {

constexpr int kLeaf = LING_B200_TREE_LEAF, kWrite = LING_B200_TREE_WRITE;

// A GEMM output is up to kMaxPlanes partial sums (its K splits).  The loads are issued together and added in plane order,
// so a consumer pays one memory latency, not one per plane, and the sum is the same whoever computes it.
__device__ __forceinline__ float plane_sum(const Planes& a, int m, int c) {
  float t[kMaxPlanes];
  const float* base = a.p + size_t(m) * a.ld + c;
#pragma unroll
  for (int p = 0; p < kMaxPlanes; ++p) t[p] = p < a.n ? base[size_t(p) * a.stride] : 0.f;
  float v = 0.f;
#pragma unroll
  for (int p = 0; p < kMaxPlanes; ++p) v += t[p];
  return v;
}
__device__ __forceinline__ float4 plane_sum4(const Planes& a, int m, int c) {
  float4 t[kMaxPlanes];
  const float* base = a.p + size_t(m) * a.ld + c;
#pragma unroll
  for (int p = 0; p < kMaxPlanes; ++p)
    t[p] = p < a.n ? *reinterpret_cast<const float4*>(base + size_t(p) * a.stride) : make_float4(0.f, 0.f, 0.f, 0.f);
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int p = 0; p < kMaxPlanes; ++p) v.x += t[p].x, v.y += t[p].y, v.z += t[p].z, v.w += t[p].w;
  return v;
}

// One warp owns one 128-column block of row m: lane l holds columns c .. c+3 (c = block * 128 + l * 4).
// scale = amax / 448 (1 for an all-zero block), codes = E4M3(x / scale); columns at or past K are zero codes.
__device__ __forceinline__ void quant_store4(float4 x, int c, int m, const QuantOut& q) {
  const int lane = threadIdx.x & 31;
  if (c >= q.K) x = make_float4(0.f, 0.f, 0.f, 0.f);
  float amax = fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w)));
  amax = warp_max(amax);
  const float sc = amax > 0.f ? amax / 448.f : 1.f;
  if (c < q.K_pad) {
    uchar4 o;
    o.x = to_e4m3(__fdiv_rn(x.x, sc)), o.y = to_e4m3(__fdiv_rn(x.y, sc));
    o.z = to_e4m3(__fdiv_rn(x.z, sc)), o.w = to_e4m3(__fdiv_rn(x.w, sc));
    *reinterpret_cast<uchar4*>(q.codes + size_t(m) * q.K_pad + c) = o;
    if (lane == 0) q.scales[size_t(c >> 7) * q.rows_alloc + m] = sc;
  }
}

// ---------------------------------------------------------------------------------------------- packing
// One warp per sequence.  Packing as src/core/speculate.cpp:1190-1201 and src/core/kernels.cuh:58-78 define it
// (rows concatenated, row0 prefix sums; a tree row's RoPE position is pos + depth, its cache slot pos + row index,
// src/core/kernels.cuh:109-118), and describe_tree (src/core/tree.cpp:81-146) by lane 0 with children as bit masks.
__global__ void __launch_bounds__(32) pack_kernel(StepBuffers sb, ModelDims d) {
  pdl_sync();  // first statement: see common.cuh
  __shared__ int par[kTreeRows], dep[kTreeRows];
  __shared__ uint32_t kids[kTreeRows];
  const int s = blockIdx.x, lane = threadIdx.x;
  const int nseq = *sb.n_seqs;
  int r0 = 0, total = 0;
  for (int t = 0; t < nseq; ++t) {
    if (t == s) r0 = total;
    total += sb.seqs[t].n_rows;
  }
  if (s == 0 && lane == 0) {
    sb.row0[nseq] = total;
    *sb.n_rows_total = total;
  }
  if (s >= nseq) return;
  const SeqDev q = sb.seqs[s];
  const int n = q.n_rows;
  if (lane == 0) sb.row0[s] = r0;
  if (lane < n) {
    int p = lane == 0 ? -1 : sb.in_parent[s * kTreeRows + lane];
    if (lane > 0 && (p < 0 || p >= lane)) {
      dev_fail(sb.err, kDevBadTree);
      p = 0;
    }
    par[lane] = p;
  }
  __syncwarp();
  if (lane < n) {
    uint32_t mask = 0;
    int dd = -1;
    for (int a = lane; a >= 0; a = par[a]) mask |= 1u << a, ++dd;
    dep[lane] = dd;
    uint32_t km = 0;
    for (int r = lane + 1; r < n; ++r)
      if (par[r] == lane) km |= 1u << r;
    kids[lane] = km;
    int tok = sb.in_token[s * kTreeRows + lane];
    if (tok < 0 || tok >= d.V) {
      dev_fail(sb.err, kDevBadToken);
      tok = 0;
    }
    const int row = r0 + lane;
    sb.token[row] = tok;
    sb.seq_of[row] = s;
    sb.local[row] = lane;
    sb.depth[row] = dd;
    sb.rope_pos[row] = q.pos + dd + q.rope_delta;
    sb.cache_slot[row] = q.pos + lane;
    sb.anc[row] = mask;
  }
  ling_b200_tree_desc& T = sb.trees[s];
  int* raw = reinterpret_cast<int*>(&T);
  for (int i = lane; i < int(sizeof(ling_b200_tree_desc) / 4); i += 32) raw[i] = 0;
  __syncwarp();
  if (lane != 0) return;
  T.n = n;
  int leaf_var[kTreeRows];
  int nvar = 0;
  bool bad = false;
  for (int r = 0; r < n; ++r) {
    T.depth[r] = dep[r];
    leaf_var[r] = -1;
    if (kids[r]) continue;
    if (nvar >= LING_B200_MAX_TREE_VARIANTS) {
      bad = true;
      break;
    }
    leaf_var[r] = nvar;
    for (int a = r; a >= 0; a = par[a]) T.path[nvar][dep[a]] = a;
    ++nvar;
  }
  T.nvar = nvar;
  if (!bad)
    for (int r = 0; r < n; ++r) {
      int a = r;
      while (kids[a]) a = __ffs(kids[a]) - 1;
      T.var[r] = leaf_var[a];
    }
  uint32_t written = 0, covered = 0;
  int ngdn = 0;
  int nodes[kTreeRows];
  auto emit = [&](int cnt) {
    int* steps = T.gdn_step[ngdn];
    int len = 0;
    for (int i = 0; i < cnt; ++i) {
      const int w = nodes[i];
      steps[len++] = w | ((written >> w) & 1u ? 0 : kWrite);
      written |= 1u << w, covered |= 1u << w;
      for (uint32_t km = kids[w]; km; km &= km - 1) {
        const int c = __ffs(km) - 1;
        if (kids[c] == 0 && !((written >> c) & 1u)) {
          steps[len++] = c | kLeaf | kWrite;
          written |= 1u << c, covered |= 1u << c;
        }
      }
    }
    T.gdn_len[ngdn++] = len;
  };
  int cnt = 0;
  for (int r = 0; r <= q.chain && r < n; ++r) nodes[cnt++] = r;
  emit(cnt);
  for (int r = 0; r < n && !bad; ++r) {
    if (((covered >> r) & 1u) || kids[r] == 0) continue;
    cnt = dep[r] + 1;
    for (int a = r, i = cnt - 1; a >= 0; a = par[a], --i) nodes[i] = a;
    for (int a = r;;) {
      int nxt = -1;
      for (uint32_t km = kids[a]; km; km &= km - 1) {
        const int c = __ffs(km) - 1;
        if (kids[c]) {
          nxt = c;
          break;
        }
      }
      if (nxt < 0) break;
      nodes[cnt++] = nxt;
      a = nxt;
    }
    if (ngdn >= LING_B200_MAX_TREE_VARIANTS) {
      bad = true;
      break;
    }
    emit(cnt);
  }
  T.ngdn = ngdn;
  if (bad || written != (n == 32 ? 0xffffffffu : ((1u << n) - 1u))) dev_fail(sb.err, kDevBadTree);
  // what the fused DeltaNet kernel needs per path and per row (GdnAux)
  GdnAux& A = sb.gdn_aux[s];
  for (int p = 0; p < ngdn; ++p) {
    uint32_t seen = 0, wr = 0;
    int np = 0;
    for (int i = 0; i < T.gdn_len[p]; ++i) {
      const int st = T.gdn_step[p][i], t = st & 0xff;
      if (!((seen >> t) & 1u)) seen |= 1u << t, A.prow[p][np++] = uint8_t(t);
      if (st & kWrite) wr |= 1u << t;
    }
    A.np[p] = np, A.wmask[p] = wr;
  }
  for (int t = 0; t < n && !bad; ++t)
    for (int j = 0; j < 3; ++j) {
      const int dj = dep[t] - 3 + j;
      A.tap[t][j] = static_cast<signed char>(dj >= 0 ? T.path[T.var[t]][dj] : dj);
    }
}

// ---------------------------------------------------------------------------------------------- norms
// h[m] (+= the previous GEMM's partial sums, or = the embedding row) -> Gemma RMSNorm x * rsqrt(mean x^2 + eps) *
// (1 + w) (src/core/kernels.cu:280-301) -> fp32 copy (for the BF16 a/b projections) and the FP8 copy for the GEMMs
// (the reference's rmsnorm_half, src/core/stream_gemm.cu:383-418, at block-scaled FP8 instead of scaled FP16).
// One thread-block cluster per row: CTA j of the cluster owns columns [1024 j, 1024 j + 1024) (four per thread), the
// partial sums of squares meet through distributed shared memory, and every CTA normalizes and quantizes its own 1024
// columns (eight 128-column blocks, one per warp).  H <= 8192 keeps the cluster within the portable size of 8.
// (Measured against one block per row: a single SM's L2 bandwidth makes that form ~3 us slower per launch at 5120 columns
// and seven partial-sum planes.)
__device__ __forceinline__ unsigned long long gtime_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Debugging aid: where set (kernels_norm_stamps), block (0, 0) of every norm_quant launch leaves five %globaltimer
// stamps there -- entry, dependency wait passed, row loaded, cluster reduction done, end -- so the last launch's remain.
__device__ unsigned long long* g_norm_stamps = nullptr;
__global__ void __launch_bounds__(256)
    norm_quant_kernel(float* __restrict__ h, Planes add, const int* __restrict__ ids, const __nv_bfloat16* __restrict__ embed,
                      const __nv_bfloat16* __restrict__ w, float* __restrict__ xn, QuantOut q, const int* __restrict__ n_rows,
                      int H, float eps) {
  unsigned long long* st = nullptr;
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) st = g_norm_stamps;
  if (st) st[0] = gtime_ns();
  // the norm weight is constant over the step: fetched before the dependency wait, so its latency hides behind the wait
  const int m = blockIdx.y;
  const int c = blockIdx.x * 1024 + threadIdx.x * 4;
  uint2 wraw = make_uint2(0u, 0u);
  if (c < H) wraw = *reinterpret_cast<const uint2*>(w + c);
  // first half of a cluster barrier whose second half stands before the first store into a peer's shared memory: by then
  // every CTA of the cluster has started (the condition for touching its shared memory), and nobody has waited for it
  if (gridDim.x > 1) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  pdl_sync();
  if (st) st[1] = gtime_ns();
  namespace cg = cooperative_groups;
  __shared__ __align__(16) float parts[64];  // [CTA of the cluster][warp]
  // The row count is requested together with the row (every row of the grid is allocated): one memory round trip, not
  // two -- behind a GEMM that is already prefetching its weights a round trip costs microseconds.
  const int nr = *n_rows;
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (ids) {
    if (m >= nr) return;
    if (c < H) {
      const __nv_bfloat16* e = embed + size_t(ids[m]) * H + c;
      v = make_float4(__bfloat162float(e[0]), __bfloat162float(e[1]), __bfloat162float(e[2]), __bfloat162float(e[3]));
    }
  } else if (c < H) {
    v = *reinterpret_cast<const float4*>(h + size_t(m) * H + c);
    if (add.p) {
      const float4 t = plane_sum4(add, m, c);
      v.x += t.x, v.y += t.y, v.z += t.z, v.w += t.w;
    }
  }
  if (m >= nr) return;  // the whole cluster shares the row, so it leaves together
  if (c < H) *reinterpret_cast<float4*>(h + size_t(m) * H + c) = v;
  const float sq = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  if (st && sq >= 0.f) st[2] = gtime_ns();
  // Sum of squares over the row: every warp pushes its partial sum into every CTA of the cluster (its own included)
  // through distributed shared memory, one cluster barrier, and each CTA adds the partials from its own shared memory
  // in (CTA, warp) order -- the same sum everywhere, nobody reads a peer that may have left, one barrier in all.
  const float wsum = warp_sum(sq);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float total = 0.f;
  if (gridDim.x > 1) {
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned me = cluster.block_rank(), nb = cluster.num_blocks();
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (lane < nb) *cluster.map_shared_rank(&parts[me * 8 + warp], lane) = wsum;
    cluster.sync();
    for (unsigned r = 0; r < nb; ++r) {
      const float4 a = *reinterpret_cast<const float4*>(&parts[r * 8]), b4 = *reinterpret_cast<const float4*>(&parts[r * 8 + 4]);
      total += ((a.x + a.y) + (a.z + a.w)) + ((b4.x + b4.y) + (b4.z + b4.w));
    }
  } else {
    if (lane == 0) parts[warp] = wsum;
    __syncthreads();
    const float4 a = *reinterpret_cast<const float4*>(&parts[0]), b4 = *reinterpret_cast<const float4*>(&parts[4]);
    total = ((a.x + a.y) + (a.z + a.w)) + ((b4.x + b4.y) + (b4.z + b4.w));
  }
  if (st) st[3] = gtime_ns();
  const float rstd = rsqrtf(total / H + eps);
  float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
  if (c < H) {
    const __nv_bfloat162 w01 = *reinterpret_cast<const __nv_bfloat162*>(&wraw.x), w23 = *reinterpret_cast<const __nv_bfloat162*>(&wraw.y);
    x.x = v.x * rstd * (1.f + __low2float(w01));
    x.y = v.y * rstd * (1.f + __high2float(w01));
    x.z = v.z * rstd * (1.f + __low2float(w23));
    x.w = v.w * rstd * (1.f + __high2float(w23));
    if (xn) *reinterpret_cast<float4*>(xn + size_t(m) * H + c) = x;
  }
  if (c - (threadIdx.x & 31) * 4 < q.K_pad) quant_store4(x, c, m, q);
  if (st) st[4] = gtime_ns();
}

__global__ void __launch_bounds__(256)
    tap_kernel(const float* __restrict__ h, Planes add, float* __restrict__ out, const int* __restrict__ n_rows, int H) {
  pdl_sync();  // first statement: see common.cuh
  const int m = blockIdx.x;
  if (m >= *n_rows) return;
  for (int c = threadIdx.x; c < H; c += blockDim.x)
    out[size_t(m) * H + c] = h[size_t(m) * H + c] + (add.p ? plane_sum(add, m, c) : 0.f);
}

// h[m][:] += planes, in place (a GEMM's partial sums into residual rows that no norm follows in the same pass)
__global__ void __launch_bounds__(256) add_planes_kernel(float* h, Planes add, const int* __restrict__ n_rows, int H) {
  pdl_sync();  // first statement: see common.cuh
  const int m = blockIdx.x;
  if (m >= *n_rows) return;
  for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4) {
    float4 v = *reinterpret_cast<const float4*>(h + size_t(m) * H + c);
    const float4 t = plane_sum4(add, m, c);
    v.x += t.x, v.y += t.y, v.z += t.z, v.w += t.w;
    *reinterpret_cast<float4*>(h + size_t(m) * H + c) = v;
  }
}

// a = xn . W_a^T, b = xn . W_b^T against BF16 weights with fp32 accumulation (src/core/kernels.cu:200-253), then the
// gating g = -exp(A_log) * softplus(a + dt_bias), beta = sigmoid(b) (src/core/kernels.cu:385-395).  One block per
// (value head, row): 128 threads split the hidden dimension four columns at a time.
__global__ void __launch_bounds__(128)
    ab_gating_kernel(const float* __restrict__ xn, const __nv_bfloat16* __restrict__ wa, const __nv_bfloat16* __restrict__ wb,
                     const __nv_bfloat16* __restrict__ A_log, const __nv_bfloat16* __restrict__ dt_bias, float* __restrict__ g,
                     float* __restrict__ beta, const int* __restrict__ n_rows, int H, int HV) {
  // The head's two weight rows are constant over the step and come from HBM: the first row's block asks for them to be
  // brought into L2 before the dependency wait, so that behind it every block of the head finds them there.
  if (blockIdx.y == 0) {
    const char* pa = reinterpret_cast<const char*>(wa + size_t(blockIdx.x) * H);
    const char* pb = reinterpret_cast<const char*>(wb + size_t(blockIdx.x) * H);
    for (int o = threadIdx.x * 128; o < H * 2; o += blockDim.x * 128) {
      asm volatile("prefetch.global.L2 [%0];" ::"l"(pa + o));
      asm volatile("prefetch.global.L2 [%0];" ::"l"(pb + o));
    }
  }
  pdl_sync();
  __shared__ float red[32];
  const int hv = blockIdx.x, m = blockIdx.y;
  const int nr = *n_rows;  // requested together with the row (every row of the grid is allocated): one round trip
  const float* x = xn + size_t(m) * H;
  const __nv_bfloat16* a = wa + size_t(hv) * H;
  const __nv_bfloat16* b = wb + size_t(hv) * H;
  float sa = 0.f, sb2 = 0.f;
#pragma unroll 5
  for (int c = threadIdx.x * 4; c < H; c += 512) {
    const float4 xv = *reinterpret_cast<const float4*>(x + c);
    const uint2 ar = *reinterpret_cast<const uint2*>(a + c), br = *reinterpret_cast<const uint2*>(b + c);
    const __nv_bfloat162 a01 = *reinterpret_cast<const __nv_bfloat162*>(&ar.x), a23 = *reinterpret_cast<const __nv_bfloat162*>(&ar.y);
    const __nv_bfloat162 b01 = *reinterpret_cast<const __nv_bfloat162*>(&br.x), b23 = *reinterpret_cast<const __nv_bfloat162*>(&br.y);
    sa += xv.x * __low2float(a01) + xv.y * __high2float(a01) + xv.z * __low2float(a23) + xv.w * __high2float(a23);
    sb2 += xv.x * __low2float(b01) + xv.y * __high2float(b01) + xv.z * __low2float(b23) + xv.w * __high2float(b23);
  }
  if (m >= nr) return;
  sa = block_sum(sa, red);
  sb2 = block_sum(sb2, red);
  if (threadIdx.x == 0) {
    const float xx = sa + __bfloat162float(dt_bias[hv]);
    const float sp = xx <= 20.f ? log1pf(__expf(xx)) : xx;
    g[size_t(m) * HV + hv] = -__expf(__bfloat162float(A_log[hv])) * sp;
    beta[size_t(m) * HV + hv] = 1.f / (1.f + __expf(-sb2));
  }
}

// The same for the many rows of a prefill chunk: a block takes four rows and four value heads, so a row of xn is read once per
// four heads and a weight row once per four rows (the per-(row, head) blocks above move 40 KB for 10 K multiply-adds, which at
// 4096 rows is 8 GB of L2 traffic).  The products and sums are the same fp32 ones; only their order differs.
__global__ void __launch_bounds__(128)
    ab_gating_rows_kernel(const float* __restrict__ xn, const __nv_bfloat16* __restrict__ wa, const __nv_bfloat16* __restrict__ wb,
                          const __nv_bfloat16* __restrict__ A_log, const __nv_bfloat16* __restrict__ dt_bias, float* __restrict__ g,
                          float* __restrict__ beta, int M, int H, int HV) {
  pdl_sync();  // first statement: see common.cuh
  __shared__ float red[4][32];
  const int hv0 = blockIdx.x * 4, m0 = blockIdx.y * 4, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float sa[4][4] = {}, sb[4][4] = {};  // [row][head]
  for (int c = threadIdx.x * 4; c < H; c += 512) {
    float4 xv[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) xv[r] = m0 + r < M ? *reinterpret_cast<const float4*>(xn + size_t(m0 + r) * H + c) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int hh = 0; hh < 4; ++hh) {
      if (hv0 + hh >= HV) break;
      const uint2 ar = *reinterpret_cast<const uint2*>(wa + size_t(hv0 + hh) * H + c), br = *reinterpret_cast<const uint2*>(wb + size_t(hv0 + hh) * H + c);
      const __nv_bfloat162 a01 = *reinterpret_cast<const __nv_bfloat162*>(&ar.x), a23 = *reinterpret_cast<const __nv_bfloat162*>(&ar.y);
      const __nv_bfloat162 b01 = *reinterpret_cast<const __nv_bfloat162*>(&br.x), b23 = *reinterpret_cast<const __nv_bfloat162*>(&br.y);
      const float a0 = __low2float(a01), a1 = __high2float(a01), a2 = __low2float(a23), a3 = __high2float(a23);
      const float b0 = __low2float(b01), b1 = __high2float(b01), b2 = __low2float(b23), b3 = __high2float(b23);
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        sa[r][hh] += xv[r].x * a0 + xv[r].y * a1 + xv[r].z * a2 + xv[r].w * a3;
        sb[r][hh] += xv[r].x * b0 + xv[r].y * b1 + xv[r].z * b2 + xv[r].w * b3;
      }
    }
  }
  // 32 sums over the block's 128 threads: warps first, then lane v of warp 0 adds the four warps' value v
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int hh = 0; hh < 4; ++hh) {
      const float va = warp_sum(sa[r][hh]), vb = warp_sum(sb[r][hh]);
      if (lane == 0) red[warp][(r * 4 + hh) * 2] = va, red[warp][(r * 4 + hh) * 2 + 1] = vb;
    }
  __syncthreads();
  if (warp == 0) {
    const float tot = red[0][lane] + red[1][lane] + red[2][lane] + red[3][lane];
    const int r = lane / 8, hh = (lane / 2) % 4, isb = lane & 1, m = m0 + r, hv = hv0 + hh;
    if (m < M && hv < HV) {
      if (isb) {
        beta[size_t(m) * HV + hv] = 1.f / (1.f + __expf(-tot));
      } else {
        const float xx = tot + __bfloat162float(dt_bias[hv]);
        const float sp = xx <= 20.f ? log1pf(__expf(xx)) : xx;
        g[size_t(m) * HV + hv] = -__expf(__bfloat162float(A_log[hv])) * sp;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------- DeltaNet
// The verify's conv over each sequence's tree (src/core/kernels.cu:365-383): a row's taps are the raw inputs of its
// ancestors at depths d-3 .. d-1 (the variant's path) or the session's window before depth 0; the window is left
// unwritten.  A tree row carries no state from the row before it, so every (row, channel) is independent: one thread
// each, the taps summed from the GEMM's partial planes.  Also materializes the raw inputs (`pre`, which the commit's
// window update replays) and L2-normalizes the q and k channels per head (eps 1e-6, q also times 1/sqrt(Dk), the
// normalization src/core/kernels.cu:420-431 applies inside the recurrence), so `post` holds q^, k^ and v.
__global__ void __launch_bounds__(256)
    conv_tree_kernel(Planes in, StepBuffers sb, int C, int Hk, int Dk, const __nv_bfloat16* __restrict__ convw,
                     const float* __restrict__ conv_state, size_t slot_stride, float* __restrict__ pre, float* __restrict__ post) {
  pdl_sync();  // first statement: see common.cuh
  __shared__ float wsum[8];
  const int m = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  if (m >= *sb.n_rows_total) return;
  const int s = sb.seq_of[m], t = sb.local[m], r0 = sb.row0[s];
  float o = 0.f;
  if (c < C) {
    const ling_b200_tree_desc* td = sb.trees + s;
    const int dd = td->depth[t];
    const int* path = td->path[td->var[t]];
    const float* win = conv_state + size_t(sb.seqs[s].slot) * slot_stride;
    const float xv = plane_sum(in, m, c);
    pre[size_t(m) * C + c] = xv;
    float tap[3];
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      const int dj = dd - 3 + j;
      tap[j] = dj >= 0 ? plane_sum(in, r0 + path[dj], c) : win[c * 3 + 3 + dj];
    }
    o = silu(__bfloat162float(convw[c * 4]) * tap[0] + __bfloat162float(convw[c * 4 + 1]) * tap[1] +
             __bfloat162float(convw[c * 4 + 2]) * tap[2] + __bfloat162float(convw[c * 4 + 3]) * xv);
  }
  const int qk = 2 * Hk * Dk;
  const float sq = warp_sum(c < qk ? o * o : 0.f);
  if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = sq;
  __syncthreads();
  if (c < qk) {
    const int wph = Dk / 32, first = ((threadIdx.x >> 5) / wph) * wph;  // warps per head; heads are aligned to the block
    float tot = 0.f;
    for (int w = 0; w < wph; ++w) tot += wsum[first + w];
    o *= rsqrtf(tot + 1e-6f) * (c < Hk * Dk ? rsqrtf(float(Dk)) : 1.f);
  }
  if (c < C) post[size_t(m) * C + c] = o;
}

// One token of the gated delta rule (src/core/kernels.cu:402-453) for 8 value columns of a head.  A warp is 8 columns x 4
// quarters of the key dimension: lane = quarter * 8 + column holds S[quarter * DK/4 .. +DK/4][column], so the two
// dependent dot products are DK/4 long (four interleaved partial sums each) plus two shuffles.  q^ and k^ arrive
// normalized, staged in shared memory with each quarter's segment padded by 16 bytes so that the four quarters of a warp
// read four different bank groups.  S *= decay; kv = S^T k; d = (v - kv) beta; S += k d^T; o = S^T q.  advance = false is
// the leaf rule (src/core/attention_body.cuh:575-603): the output from the parent's state, which stays as it was.
template <int DK>
struct GdnStage {
  static constexpr int KL = DK / 4, SEG = KL + 4, ROW = 8 * SEG;  // floats per step: q quarters 0-3, then k quarters 0-3
  // Stages `len` steps' q^, k^, v, g, beta of (key head h, value head hv) into shared memory, all threads of the block.
  __device__ static void load(const float* __restrict__ post, const float* __restrict__ g, const float* __restrict__ beta, int C,
                              int Hk, int HV, int Dv, int h, int hv, size_t r0, const int* rows, int len, float* qk, float* vv,
                              float* gb) {
    constexpr int V4 = 2 * DK / 4;  // float4 pieces of one step's q and k
    for (int idx = threadIdx.x; idx < len * V4; idx += blockDim.x) {
      const int i = idx / V4, part = idx % V4, isk = part >= DK / 4, e = (isk ? part - DK / 4 : part) * 4;
      const float* src = post + (r0 + rows[i]) * C + (isk ? Hk * DK : 0) + h * DK + e;
      *reinterpret_cast<float4*>(qk + size_t(i) * ROW + (isk ? 4 * SEG : 0) + (e / KL) * SEG + e % KL) =
          *reinterpret_cast<const float4*>(src);
    }
    for (int idx = threadIdx.x; idx < len * (Dv / 4); idx += blockDim.x) {
      const int i = idx / (Dv / 4), e = (idx % (Dv / 4)) * 4;
      *reinterpret_cast<float4*>(vv + size_t(i) * Dv + e) =
          *reinterpret_cast<const float4*>(post + (r0 + rows[i]) * C + 2 * Hk * DK + hv * Dv + e);
    }
    for (int i = threadIdx.x; i < len; i += blockDim.x) {
      gb[2 * i] = g[(r0 + rows[i]) * HV + hv];
      gb[2 * i + 1] = beta[(r0 + rows[i]) * HV + hv];
    }
  }
  __device__ __forceinline__ static float token(float (&S)[KL], const float* qk_i, float v, float gval, float bval, int quarter,
                                                bool advance) {
    const float4* kp = reinterpret_cast<const float4*>(qk_i + 4 * SEG + quarter * SEG);
    const float4* qp = reinterpret_cast<const float4*>(qk_i + quarter * SEG);
    const float decay = __expf(gval);
    float k[KL], Sd[KL], part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < KL / 4; ++i) {
      const float4 a = kp[i];
      k[4 * i] = a.x, k[4 * i + 1] = a.y, k[4 * i + 2] = a.z, k[4 * i + 3] = a.w;
    }
#pragma unroll
    for (int i = 0; i < KL; ++i) {
      Sd[i] = S[i] * decay;
      part[i & 3] = fmaf(Sd[i], k[i], part[i & 3]);
    }
    float kv = (part[0] + part[1]) + (part[2] + part[3]);
    kv += __shfl_xor_sync(0xffffffffu, kv, 8);
    kv += __shfl_xor_sync(0xffffffffu, kv, 16);
    const float dlt = (v - kv) * bval;
    part[0] = part[1] = part[2] = part[3] = 0.f;
#pragma unroll
    for (int i = 0; i < KL / 4; ++i) {
      const float4 qv = qp[i];
      const float qq[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float sn = fmaf(dlt, k[4 * i + j], Sd[4 * i + j]);
        part[j] = fmaf(sn, qq[j], part[j]);
        if (advance) S[4 * i + j] = sn;
      }
    }
    float o = (part[0] + part[1]) + (part[2] + part[3]);
    o += __shfl_xor_sync(0xffffffffu, o, 8);
    o += __shfl_xor_sync(0xffffffffu, o, 16);
    return o;
  }
  // The state update of token() alone, bit for bit (the commit needs no output): S *= decay; S += k ((v - S^T k) beta)^T.
  __device__ __forceinline__ static void advance(float (&S)[KL], const float* qk_i, float v, float gval, float bval, int quarter) {
    const float4* kp = reinterpret_cast<const float4*>(qk_i + 4 * SEG + quarter * SEG);
    const float decay = __expf(gval);
    float k[KL], part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < KL / 4; ++i) {
      const float4 a = kp[i];
      k[4 * i] = a.x, k[4 * i + 1] = a.y, k[4 * i + 2] = a.z, k[4 * i + 3] = a.w;
    }
#pragma unroll
    for (int i = 0; i < KL; ++i) {
      S[i] *= decay;
      part[i & 3] = fmaf(S[i], k[i], part[i & 3]);
    }
    float kv = (part[0] + part[1]) + (part[2] + part[3]);
    kv += __shfl_xor_sync(0xffffffffu, kv, 8);
    kv += __shfl_xor_sync(0xffffffffu, kv, 16);
    const float dlt = (v - kv) * bval;
#pragma unroll
    for (int i = 0; i < KL; ++i) S[i] = fmaf(dlt, k[i], S[i]);
  }
  // The same step with one reduction round instead of two: o = S'^T q = (S d)^T q + delta (k . q), so the two dot products
  // over the decayed state run side by side and k . q (`kq`, the same for every value column) comes precomputed.  The
  // state update is the arithmetic of token() bit for bit; only o is rounded differently.
  __device__ __forceinline__ static float token2(float (&S)[KL], const float* qk_i, float v, float gval, float bval, float kq,
                                                 int quarter, bool advance) {
    const float4* kp = reinterpret_cast<const float4*>(qk_i + 4 * SEG + quarter * SEG);
    const float4* qp = reinterpret_cast<const float4*>(qk_i + quarter * SEG);
    const float decay = __expf(gval);
    // packed fp32x2 arithmetic (two IEEE operations per instruction on sm_100): element pairs (4i, 4i+1) and (4i+2, 4i+3),
    // so the four partial sums per dot product are the ones token() keeps
    const float2 decay2 = make_float2(decay, decay);
    float2 k2[KL / 2], Sd2[KL / 2];
    float2 pk2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)}, pq2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
    for (int i = 0; i < KL / 4; ++i) {
      const float4 a = kp[i], b = qp[i];
      k2[2 * i] = make_float2(a.x, a.y), k2[2 * i + 1] = make_float2(a.z, a.w);
      Sd2[2 * i] = __fmul2_rn(make_float2(S[4 * i], S[4 * i + 1]), decay2);
      Sd2[2 * i + 1] = __fmul2_rn(make_float2(S[4 * i + 2], S[4 * i + 3]), decay2);
      pk2[0] = __ffma2_rn(Sd2[2 * i], k2[2 * i], pk2[0]);
      pk2[1] = __ffma2_rn(Sd2[2 * i + 1], k2[2 * i + 1], pk2[1]);
      pq2[0] = __ffma2_rn(Sd2[2 * i], make_float2(b.x, b.y), pq2[0]);
      pq2[1] = __ffma2_rn(Sd2[2 * i + 1], make_float2(b.z, b.w), pq2[1]);
    }
    float kv = (pk2[0].x + pk2[0].y) + (pk2[1].x + pk2[1].y), sq = (pq2[0].x + pq2[0].y) + (pq2[1].x + pq2[1].y);
    kv += __shfl_xor_sync(0xffffffffu, kv, 8), sq += __shfl_xor_sync(0xffffffffu, sq, 8);
    kv += __shfl_xor_sync(0xffffffffu, kv, 16), sq += __shfl_xor_sync(0xffffffffu, sq, 16);
    const float dlt = (v - kv) * bval;
    if (advance) {
      const float2 dlt2 = make_float2(dlt, dlt);
#pragma unroll
      for (int m = 0; m < KL / 2; ++m) {
        const float2 sn = __ffma2_rn(dlt2, k2[m], Sd2[m]);
        S[2 * m] = sn.x, S[2 * m + 1] = sn.y;
      }
    }
    return fmaf(dlt, kq, sq);
  }
  static size_t smem_bytes(int Dv, int steps = 2 * kTreeRows) { return size_t(steps) * (ROW + Dv + 2) * 4; }
};

// The verify's recurrence over every sequence's tree (src/core/kernels.cu:455-477): a work item is (sequence, DeltaNet
// path, value head); its block (one warp per 8 value columns) first stages the whole path's inputs in shared memory with
// one round of coalesced loads, then walks the steps from the session's state (never written here) and writes the rows
// flagged kWrite.  A fixed grid of blocks strides over the items.
constexpr int kGdnCols = 32;  // value columns per block of the DeltaNet kernels (4 warps x 8 columns)
template <int DK>
__global__ void __launch_bounds__(128)
    gdn_tree_kernel(const float* __restrict__ post, const float* __restrict__ g, const float* __restrict__ beta, StepBuffers sb,
                    int Hk, int HV, int Dv, const float* __restrict__ state, size_t slot_stride, float* __restrict__ core) {
  pdl_sync();  // first statement: see common.cuh
  using St = GdnStage<DK>;
  constexpr int KL = St::KL;
  extern __shared__ __align__(16) float gsm[];
  float* qk = gsm;                                         // [64][ROW]
  float* vv = qk + size_t(2 * kTreeRows) * St::ROW;        // [64][Dv]
  float* gb = vv + size_t(2 * kTreeRows) * Dv;             // [64][2]
  __shared__ int pbase[LING_B200_MAX_SEQS + 1];
  __shared__ int steps[2 * kTreeRows], rows[2 * kTreeRows];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, quarter = lane >> 3;
  const int nseq = *sb.n_seqs;
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int s = 0; s < nseq; ++s) {
      pbase[s] = acc;
      acc += sb.trees[s].ngdn;
    }
    pbase[nseq] = acc;
  }
  __syncthreads();
  const int C = 2 * Hk * DK + HV * Dv, groups = Dv / kGdnCols;
  const int total = pbase[nseq] * HV * groups;
  for (int item = blockIdx.x; item < total; item += gridDim.x) {
    const int pg = item / (HV * groups), hv = (item / groups) % HV, col = (item % groups) * kGdnCols + warp * 8 + (lane & 7);
    int s = 0;
    while (pbase[s + 1] <= pg) ++s;
    const int pth = pg - pbase[s], h = hv / (HV / Hk);
    const ling_b200_tree_desc* td = sb.trees + s;
    const size_t r0 = size_t(sb.row0[s]);
    const int len = td->gdn_len[pth];
    __syncthreads();  // the previous item's readers of the staged inputs are done
    for (int i = threadIdx.x; i < len; i += blockDim.x) {
      steps[i] = td->gdn_step[pth][i];
      rows[i] = steps[i] & 0xff;
    }
    const float* st = state + size_t(sb.seqs[s].slot) * slot_stride + size_t(hv) * DK * Dv;
    float S[KL];
#pragma unroll
    for (int i = 0; i < KL; ++i) S[i] = st[size_t(quarter * KL + i) * Dv + col];
    __syncthreads();
    St::load(post, g, beta, C, Hk, HV, Dv, h, hv, r0, rows, len, qk, vv, gb);
    __syncthreads();
    for (int i = 0; i < len; ++i) {
      const int st_i = steps[i];
      const float o = St::token(S, qk + size_t(i) * St::ROW, vv[size_t(i) * Dv + col], gb[2 * i], gb[2 * i + 1], quarter,
                                (st_i & kLeaf) == 0);
      if ((st_i & kWrite) && quarter == 0) core[(r0 + (st_i & 0xff)) * HV * Dv + size_t(hv) * Dv + col] = o;
    }
  }
}

// The DeltaNet mixer between the in and the out projection as one kernel: causal conv over the tree + SiLU, L2 norm of
// q and k, the gated delta rule over every DeltaNet path, the gated RMSNorm and the FP8 copy for the out projection
// (conv_tree_kernel, gdn_tree_kernel and gated_norm_quant_kernel above in one launch: the step is latency-bound here,
// and each kernel boundary costs more than the arithmetic).  A work item is (sequence, DeltaNet path, 128 value
// columns) = one quantization block of the out projection's input: one head of 128, or two heads of 64.  The block
// (16 warps, 8 value columns each) stages the raw inputs of all the sequence's rows for its channels, runs the conv and
// the normalization in shared memory, walks the path with the state in registers, and normalizes and quantizes the rows
// this path writes, for which it also stores `pre` and `post`, which the commit kernels replay.
template <int DK>
struct GdnFused {
  using St = GdnStage<DK>;
  static constexpr int NH = 128 / DK;        // heads per block
  static constexpr int CH = NH * 3 * DK;     // staged channels: per head q, k, v  (= 384)
  static constexpr int RAWS = CH + 4;        // floats per staged row
  static constexpr size_t smem_floats() {
    return size_t(kTreeRows) * RAWS + size_t(NH) * kTreeRows * St::ROW + size_t(kTreeRows) * 128 + size_t(NH) * kTreeRows * 2 +
           size_t(kTreeRows) * 128 + size_t(CH) * 8;
  }
};
template <int DK>
__global__ void __launch_bounds__(512)
    gdn_fused_kernel(Planes in, StepBuffers sb, ModelDims d, const __nv_bfloat16* __restrict__ convw,
                     const float* __restrict__ conv_state, size_t conv_slot_stride, const float* __restrict__ g,
                     const float* __restrict__ beta, const float* __restrict__ state, size_t state_slot_stride,
                     const __nv_bfloat16* __restrict__ norm_w, QuantOut q, float* __restrict__ pre, float* __restrict__ post,
                     float* __restrict__ core_out, int n_slots, PrefetchPlan plan, unsigned long long* stamps) {
  const bool stamp = stamps != nullptr && blockIdx.x == 0 && threadIdx.x == 0;
  if (stamp) stamps[0] = gtime_ns();
  using F = GdnFused<DK>;
  using St = GdnStage<DK>;
  constexpr int KL = St::KL, NH = F::NH, CH = F::CH, RAWS = F::RAWS;
  // ---- Before the dependency wait: the state of the block's first item, 64 KB that come from HBM.  No kernel of the step
  // writes the state before the commit at its end, so a value loaded here is the value after the wait; what may be stale
  // this early is the step's description that says WHICH state the item needs, so the choice is checked again behind the
  // wait and the state is reloaded if it was wrong (indices are clamped, so a stale description cannot lead outside).
  extern __shared__ __align__(16) float gsm[];
  float* raw = gsm;                                   // [32][RAWS] raw conv inputs of the sequence's rows
  float* qk = raw + size_t(kTreeRows) * RAWS;         // [NH][32][ROW] q^ and k^ per row (GdnStage layout)
  float* vv = qk + size_t(NH) * kTreeRows * St::ROW;  // [32][128] conv output of the value channels
  float* gb = vv + size_t(kTreeRows) * 128;           // [NH][32][2] g, beta
  float* osm = gb + NH * kTreeRows * 2;               // [32][128] the recurrence's outputs
  float* cwin = osm + size_t(kTreeRows) * 128;        // [CH][8] per channel: the four conv taps' weights, the session's window
  // channel c of the block -> (head in block, part 0 q / 1 k / 2 v, element) and its conv channel
  auto conv_channel = [&](int c, int qb, int& hb, int& part, int& e) {
    hb = c / (3 * DK), part = (c % (3 * DK)) / DK, e = c % DK;
    const int hv = qb * NH + hb, h = hv / (d.HV / d.Hk);
    return part == 0 ? h * DK + e : part == 1 ? d.Hk * DK + h * DK + e : 2 * d.Hk * DK + hv * DK + e;
  };
  // weights and window (taps before depth 0) of the block's channels into shared memory
  auto load_conv_consts = [&](int qb, int slot) {
    for (int c = threadIdx.x; c < CH; c += blockDim.x) {
      int hb, part, e;
      const int gc = conv_channel(c, qb, hb, part, e);
      const uint2 wr = *reinterpret_cast<const uint2*>(convw + size_t(gc) * 4);
      const float* wsrc = conv_state + size_t(slot) * conv_slot_stride + size_t(gc) * 3;
      const float w0 = wsrc[0], w1 = wsrc[1], w2 = wsrc[2];
      const __nv_bfloat162 c01 = *reinterpret_cast<const __nv_bfloat162*>(&wr.x), c23 = *reinterpret_cast<const __nv_bfloat162*>(&wr.y);
      *reinterpret_cast<float4*>(cwin + c * 8) = make_float4(__low2float(c01), __high2float(c01), __low2float(c23), __high2float(c23));
      *reinterpret_cast<float4*>(cwin + c * 8 + 4) = make_float4(w0, w1, w2, 0.f);
    }
  };
  const int colb_ = (threadIdx.x >> 5) * 8 + (threadIdx.x & 7), quarter_ = (threadIdx.x & 31) >> 3;
  int spec_slot = -1, spec_hv = -1;
  float S[KL];
  {
    const int QB_ = d.HV / NH, pg0 = int(blockIdx.x) / QB_, qb0 = int(blockIdx.x) % QB_;
    const int ns = min(max(*sb.n_seqs, 0), d.max_seqs);
    int s0 = -1, acc = 0;
    for (int s = 0; s < ns; ++s) {
      const int k = min(max(sb.trees[s].ngdn, 0), LING_B200_MAX_TREE_VARIANTS);
      if (s0 < 0 && pg0 < acc + k) s0 = s;
      acc += k;
    }
    const int sl = s0 >= 0 ? sb.seqs[s0].slot : -1;
    if (sl >= 0 && sl < n_slots) {
      spec_slot = sl, spec_hv = qb0 * NH + colb_ / DK;
      const float* st = state + size_t(sl) * state_slot_stride + size_t(spec_hv) * DK * DK;
#pragma unroll
      for (int i = 0; i < KL; ++i) S[i] = st[size_t(quarter_ * KL + i) * DK + colb_ % DK];
      load_conv_consts(qb0, sl);  // the conv's constants of the same item, with the same check behind the wait
    }
  }
  pdl_sync();
  if (stamp) stamps[1] = gtime_ns();
  __shared__ int pbase[LING_B200_MAX_SEQS + 1];
  __shared__ int steps[2 * kTreeRows], taprow[3 * kTreeRows], prow[kTreeRows];
  __shared__ float kqs[2 * kTreeRows];  // k^ . q^ per (head in block, row)
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, quarter = lane >> 3;
  const int nseq = *sb.n_seqs;
  if (tid == 0) {
    int acc = 0;
    for (int s = 0; s < nseq; ++s) {
      pbase[s] = acc;
      acc += sb.trees[s].ngdn;
    }
    pbase[nseq] = acc;
  }
  __syncthreads();
  const int C = d.C, Hk = d.Hk, HV = d.HV, ratio = HV / Hk, QB = HV / NH;  // QB: 128-column blocks of the value width
  const int total = pbase[nseq] * QB;
  if (int(blockIdx.x) >= total) {
    // A CTA without an item (a step of few sequences leaves a third of the SMs idle here) asks the weights of the GEMMs
    // behind this kernel into L2: HBM has nothing else to do while the recurrence runs.  Bulk prefetches of 4 KB, this
    // CTA's share of each range, after the working CTAs' first loads have gone out.
    prefetch_plan_share(plan, int(blockIdx.x) - total, int(gridDim.x) - total);
    return;
  }
  for (int item = blockIdx.x; item < total; item += gridDim.x) {
    const int pg = item / QB, qb = item % QB;
    int s = 0;
    while (pbase[s + 1] <= pg) ++s;
    const int pth = pg - pbase[s];
    const ling_b200_tree_desc* td = sb.trees + s;
    const int r0 = sb.row0[s], n = sb.seqs[s].n_rows, len = td->gdn_len[pth], slot = sb.seqs[s].slot;
    __syncthreads();  // the previous item's readers of shared memory are done
    // ---- Everything the item needs from memory is requested here in one go -- the tree, the state (this thread's KL rows
    // of its value column), the raw inputs of every row of the sequence for the block's channels (no dependence on the
    // path: one round trip less than staging the path's rows only) and the gates -- and only then stored to shared
    // memory: a load behind a dependent store would cost a further round trip each time.
    static_assert(3 * kTreeRows <= 512 && NH * kTreeRows <= 512, "one element per thread");
    const GdnAux* aux = sb.gdn_aux + s;
    const int np = aux->np[pth];
    const uint32_t wmask = aux->wmask[pth];
    const int v_step = tid < len ? td->gdn_step[pth][tid] : 0;
    const int v_prow = tid < kTreeRows ? aux->prow[pth][tid] : 0;
    const int v_tap = tid < 3 * n ? aux->tap[tid / 3][tid % 3] : 0;
    const int colb = warp * 8 + (lane & 7);  // column inside the block's 128
    const int hb_t = colb / DK, hv_t = qb * NH + hb_t, col = colb % DK;
    if (item != int(blockIdx.x) || slot != spec_slot) load_conv_consts(qb, slot);
    if (item != int(blockIdx.x) || slot != spec_slot || hv_t != spec_hv) {  // not what was loaded before the wait
      const float* st = state + size_t(slot) * state_slot_stride + size_t(hv_t) * DK * DK;
#pragma unroll
      for (int i = 0; i < KL; ++i) S[i] = st[size_t(quarter * KL + i) * DK + col];
    }
    float v_g = 0.f, v_beta = 0.f;
    if (tid < NH * n) {
      const int hv = qb * NH + tid / n, t = tid % n;
      v_g = g[size_t(r0 + t) * HV + hv], v_beta = beta[size_t(r0 + t) * HV + hv];
    }
    {
      constexpr int RAWL = (kTreeRows * (CH / 4) + 511) / 512;
      float4 rawv[RAWL];
#pragma unroll
      for (int k = 0; k < RAWL; ++k) {
        const int idx = tid + k * 512;
        if (idx < n * (CH / 4)) {
          int hb, part, e;
          rawv[k] = plane_sum4(in, r0 + idx / (CH / 4), conv_channel((idx % (CH / 4)) * 4, qb, hb, part, e));
        }
      }
      if (tid < len) steps[tid] = v_step;
      if (tid < kTreeRows) prow[tid] = v_prow;
      if (tid < 3 * n) taprow[tid] = v_tap;
      if (tid < NH * n) {
        const int hb = tid / n, t = tid % n;
        gb[(hb * kTreeRows + t) * 2] = v_g, gb[(hb * kTreeRows + t) * 2 + 1] = v_beta;
      }
#pragma unroll
      for (int k = 0; k < RAWL; ++k) {
        const int idx = tid + k * 512;
        if (idx < n * (CH / 4)) *reinterpret_cast<float4*>(raw + size_t(idx / (CH / 4)) * RAWS + (idx % (CH / 4)) * 4) = rawv[k];
      }
    }
    __syncthreads();
    // (only the path's distinct rows -- prow, np of them -- are convolved and normalized here; a row's `pre` / `post` are
    // stored by the path that writes the row: wmask)
    if (stamp && item == blockIdx.x) stamps[2] = gtime_ns();
    // ---- conv + SiLU: a thread owns a channel (its taps, window and destinations stay in registers) and walks a quarter
    // of the path's rows: 4 x 384 slots = three per thread
    for (int w0 = tid; w0 < 4 * CH; w0 += blockDim.x) {
      const int c = w0 % CH, qr = w0 / CH;
      int hb, part, e;
      const int gc = conv_channel(c, qb, hb, part, e);
      const float4 cw = *reinterpret_cast<const float4*>(cwin + c * 8);
      const float4 win = *reinterpret_cast<const float4*>(cwin + c * 8 + 4);
      const float cw0 = cw.x, cw1 = cw.y, cw2 = cw.z, cw3 = cw.w;
      const bool own = part == 2 || (qb * NH + hb) % ratio == 0;  // q, k channels belong to the first head of their group
      float* dst = part == 2 ? vv + hb * DK + e
                             : qk + size_t(hb) * kTreeRows * St::ROW + (part == 1 ? 4 * St::SEG : 0) + (e / KL) * St::SEG + e % KL;
      const int dstride = part == 2 ? 128 : St::ROW;
      for (int li = (np * qr) / 4; li < (np * (qr + 1)) / 4; ++li) {
        const int t = prow[li];
        float tap[3];
#pragma unroll
        for (int j = 0; j < 3; ++j) {
          const int tr = taprow[t * 3 + j];
          tap[j] = tr >= 0 ? raw[size_t(tr) * RAWS + c] : (tr == -1 ? win.z : tr == -2 ? win.y : win.x);
        }
        const float xv = raw[size_t(t) * RAWS + c];
        const float o = silu(cw0 * tap[0] + cw1 * tap[1] + cw2 * tap[2] + cw3 * xv);
        dst[size_t(t) * dstride] = o;
        if (own && ((wmask >> t) & 1u)) {
          pre[size_t(r0 + t) * C + gc] = xv;
          if (part == 2) post[size_t(r0 + t) * C + gc] = o;
        }
      }
    }
    __syncthreads();
    if (stamp && item == blockIdx.x) stamps[3] = gtime_ns();
    // ---- L2 norm of q and k per (head, row) (eps 1e-6; q also times 1/sqrt(DK)) and their dot product: one warp per
    // (head, row), lane l holds the elements l, l + 32, ..
    for (int v = warp; v < NH * np; v += blockDim.x / 32) {
      const int hb = v / np, t = prow[v % np];
      float* qb_ = qk + (size_t(hb) * kTreeRows + t) * St::ROW;
      float* kb_ = qb_ + 4 * St::SEG;
      float xq[DK / 32], xk[DK / 32];
      float sq = 0.f, sk = 0.f;
#pragma unroll
      for (int j = 0; j < DK / 32; ++j) {
        const int off = ((j * 32 + lane) / KL) * St::SEG + (j * 32 + lane) % KL;
        xq[j] = qb_[off], xk[j] = kb_[off];
        sq = fmaf(xq[j], xq[j], sq), sk = fmaf(xk[j], xk[j], sk);
      }
      sq = warp_sum(sq), sk = warp_sum(sk);
      const float cq = rsqrtf(sq + 1e-6f) * rsqrtf(float(DK)), ck = rsqrtf(sk + 1e-6f);
      const int hv = qb * NH + hb;
      const bool own = hv % ratio == 0 && ((wmask >> t) & 1u);
      float* gq = post + size_t(r0 + t) * C + (hv / ratio) * DK;
      float* gk = gq + Hk * DK;
      float dot = 0.f;
#pragma unroll
      for (int j = 0; j < DK / 32; ++j) {
        const int off = ((j * 32 + lane) / KL) * St::SEG + (j * 32 + lane) % KL;
        const float yq = xq[j] * cq, yk = xk[j] * ck;
        qb_[off] = yq, kb_[off] = yk;
        dot = fmaf(yq, yk, dot);
        if (own) gq[j * 32 + lane] = yq, gk[j * 32 + lane] = yk;
      }
      dot = warp_sum(dot);
      if (lane == 0) kqs[hb * kTreeRows + t] = dot;
    }
    __syncthreads();
    if (stamp && item == blockIdx.x) stamps[4] = gtime_ns();
    // ---- the gated delta rule along the path (src/core/kernels.cu:402-477)
    for (int i = 0; i < len; ++i) {
      const int st_i = steps[i], t = st_i & 0xff;
      const float* gbt = gb + (hb_t * kTreeRows + t) * 2;
      const float* qkt = qk + (size_t(hb_t) * kTreeRows + t) * St::ROW;
      const float kq = kqs[hb_t * kTreeRows + t];
      const float o = (st_i & kLeaf) ? St::token2(S, qkt, vv[t * 128 + colb], gbt[0], gbt[1], kq, quarter, false)   // block-uniform
                                     : St::token2(S, qkt, vv[t * 128 + colb], gbt[0], gbt[1], kq, quarter, true);
      if ((st_i & kWrite) && quarter == 0) {
        osm[t * 128 + colb] = o;
        if (core_out) core_out[size_t(r0 + t) * d.Vs + qb * 128 + colb] = o;  // the recurrence's output before the gated norm (parity checks)
      }
    }
    __syncthreads();
    if (stamp && item == blockIdx.x) stamps[5] = gtime_ns();
    // ---- gated RMSNorm per head with the plain weight, times silu(z) (src/core/kernels.cu:543-554), and the FP8 copy:
    // a warp takes a written row, lane l its columns 4 l .. 4 l + 3
    for (int i = warp; i < len; i += blockDim.x / 32) {
      if (!(steps[i] & kWrite)) continue;  // warp-uniform
      const int t = steps[i] & 0xff, c = qb * 128 + lane * 4;
      float4 x = *reinterpret_cast<const float4*>(osm + t * 128 + lane * 4);
      const float4 zz = plane_sum4(in, r0 + t, C + c);
      float ss = x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
#pragma unroll
      for (int o = DK / 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float rstd = rsqrtf(ss / DK + d.eps);
      const int dd = (lane * 4) % DK;
      x.x = x.x * rstd * __bfloat162float(norm_w[dd]) * silu(zz.x);
      x.y = x.y * rstd * __bfloat162float(norm_w[dd + 1]) * silu(zz.y);
      x.z = x.z * rstd * __bfloat162float(norm_w[dd + 2]) * silu(zz.z);
      x.w = x.w * rstd * __bfloat162float(norm_w[dd + 3]) * silu(zz.w);
      quant_store4(x, c, r0 + t, q);
    }
    if (stamp && item == blockIdx.x) stamps[6] = gtime_ns();
  }
}

// Engine::commit (src/core/speculate.cpp:516-529), the recurrence half: the accepted rows path[0..n) replayed from the
// session's state over their saved conv outputs, the state written back.  Item = (sequence, layer, value head, 32 value
// columns).  The commit reads and writes every session state once (151 MB each way per sequence of the 27B model), so it
// is a bandwidth problem: the path's inputs are staged kCommitRows rows at a time, which keeps the block's shared memory
// small enough for five blocks per SM (the registers' limit), and the grid has a block per item (two blocks per SM with the
// whole path staged and a strided grid: 200 us per step; this form 130).  What bounds an item is its chain of dependent
// loads (the path, then the path's rows) and its steps, not the tile's bytes: a form that moved the 64 KB tiles of whole
// heads by bulk copies through two shared-memory buffers, one persistent block per SM, measured the same.
constexpr int kCommitRows = 16;
template <int DK>
__global__ void __launch_bounds__(128, 5)
    gdn_commit_kernel(const float* __restrict__ post, const float* __restrict__ g, const float* __restrict__ beta,
                      size_t post_layer_stride, size_t g_layer_stride, StepBuffers sb, int Hk, int HV, int Dv, int n_gdn,
                      float* __restrict__ state, size_t slot_stride, size_t layer_stride) {
  pdl_sync();  // first statement: see common.cuh
  using St = GdnStage<DK>;
  constexpr int KL = St::KL;
  extern __shared__ __align__(16) float gsm[];
  float* qk = gsm;
  float* vv = qk + size_t(kCommitRows) * St::ROW;
  float* gb = vv + size_t(kCommitRows) * Dv;
  __shared__ int rows[kTreeRows];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, quarter = lane >> 3;
  const int nseq = *sb.n_seqs;
  const int C = 2 * Hk * DK + HV * Dv, groups = Dv / kGdnCols;
  const int per_seq = n_gdn * HV * groups;
  const int total = nseq * per_seq;
  for (int item = blockIdx.x; item < total; item += gridDim.x) {
    const int s = item / per_seq, gl = (item % per_seq) / (HV * groups), hv = (item / groups) % HV, h = hv / (HV / Hk);
    const int col = (item % groups) * kGdnCols + warp * 8 + (lane & 7);
    const ling_b200_seq_result* R = sb.results + s;
    if (R->status != 0) continue;  // block-uniform
    const size_t r0 = size_t(sb.row0[s]);
    const int n = min(R->n_path, kTreeRows);
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) rows[i] = R->path[i];
    float* st = state + size_t(sb.seqs[s].slot) * slot_stride + size_t(gl) * layer_stride + size_t(hv) * DK * Dv;
    float S[KL];
#pragma unroll
    for (int i = 0; i < KL; ++i) S[i] = st[size_t(quarter * KL + i) * Dv + col];
    for (int c0 = 0; c0 < n; c0 += kCommitRows) {
      const int cn = min(kCommitRows, n - c0);
      __syncthreads();  // the path is staged / the previous rows have been consumed
      St::load(post + size_t(gl) * post_layer_stride, g + size_t(gl) * g_layer_stride, beta + size_t(gl) * g_layer_stride, C, Hk,
               HV, Dv, h, hv, r0, rows + c0, cn, qk, vv, gb);
      __syncthreads();
      for (int i = 0; i < cn; ++i)
        St::advance(S, qk + size_t(i) * St::ROW, vv[size_t(i) * Dv + col], gb[2 * i], gb[2 * i + 1], quarter);
    }
#pragma unroll
    for (int i = 0; i < KL; ++i) st[size_t(quarter * KL + i) * Dv + col] = S[i];
  }
}

// The conv half of the commit: the window advanced over the accepted rows' raw inputs (src/core/kernels.cu:320-338).
__global__ void __launch_bounds__(256)
    conv_commit_kernel(StepBuffers sb, int C, const float* __restrict__ pre, size_t layer_stride, float* __restrict__ conv_state,
                       size_t slot_stride, size_t conv_layer_stride) {
  pdl_sync();  // first statement: see common.cuh
  const int s = blockIdx.y, gl = blockIdx.z, c = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= *sb.n_seqs || c >= C) return;
  const ling_b200_seq_result* R = sb.results + s;
  if (R->status != 0) return;
  const int r0 = sb.row0[s];
  float* win = conv_state + size_t(sb.seqs[s].slot) * slot_stride + size_t(gl) * conv_layer_stride + size_t(c) * 3;
  float s0 = win[0], s1 = win[1], s2 = win[2];
  const float* P = pre + size_t(gl) * layer_stride;
  for (int j = 0; j < R->n_path; ++j) {
    s0 = s1, s1 = s2;
    s2 = P[size_t(r0 + R->path[j]) * C + c];
  }
  win[0] = s0, win[1] = s1, win[2] = s2;
}

// rmsnorm(core) * w * silu(z) per (row, value head) over Dv with the plain weight (src/core/kernels.cu:543-554), then
// the FP8 copy for the out projection.  A warp covers 128 columns: one head (Dv = 128) or several.
__global__ void __launch_bounds__(256)
    gated_norm_quant_kernel(const float* __restrict__ core, Planes z, int z_col, const __nv_bfloat16* __restrict__ w, QuantOut q,
                            const int* __restrict__ n_rows, int Vs, int Dv, float eps) {
  pdl_sync();  // first statement: see common.cuh
  const int m = blockIdx.x;
  if (m >= *n_rows) return;
  const int seg = Dv / 4;  // lanes per head
  {
    const int c = blockIdx.y * 1024 + threadIdx.x * 4;
    if (c - (threadIdx.x & 31) * 4 >= q.K_pad) return;  // warp-uniform
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 zz = x;
    if (c < Vs) {
      x = *reinterpret_cast<const float4*>(core + size_t(m) * Vs + c);
      zz = plane_sum4(z, m, z_col + c);
    }
    float ss = x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
    for (int o = seg >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rstd = rsqrtf(ss / Dv + eps);
    if (c < Vs) {
      const int dd = c % Dv;
      x.x = x.x * rstd * __bfloat162float(w[dd]) * silu(zz.x);
      x.y = x.y * rstd * __bfloat162float(w[dd + 1]) * silu(zz.y);
      x.z = x.z * rstd * __bfloat162float(w[dd + 2]) * silu(zz.z);
      x.w = x.w * rstd * __bfloat162float(w[dd + 3]) * silu(zz.w);
    }
    quant_store4(x, c, m, q);
  }
}

// silu(gate) * up (src/core/kernels.cu:308-312) from the gate|up GEMM's partial sums, and its FP8 copy.
__global__ void __launch_bounds__(256)
    silu_mul_quant_kernel(Planes gu, int I, int up_col0, QuantOut q, const int* __restrict__ n_rows) {
  pdl_sync();  // first statement: see common.cuh
  const int m = blockIdx.x;
  const int nr = *n_rows;  // requested together with the row (every row of the grid is allocated): one round trip
  {
    const int c = blockIdx.y * 1024 + threadIdx.x * 4;
    if (c - (threadIdx.x & 31) * 4 >= q.K_pad) return;  // warp-uniform
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < I) {
      const float4 a = plane_sum4(gu, m, c), b = plane_sum4(gu, m, up_col0 + c);
      x = make_float4(silu(a.x) * b.x, silu(a.y) * b.y, silu(a.z) * b.z, silu(a.w) * b.w);
    }
    if (m >= nr) return;
    quant_store4(x, c, m, q);
  }
}

// ---------------------------------------------------------------------------------------------- attention
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < warps ? red[lane] : 0.f;
  return warp_max(t);
}

// attn_prepare (src/core/kernels.cu:558-596, src/core/attention_body.cuh:54-99): per head RMSNorm with (1 + w) and the
// rotation of the first `rot` dims for q and k; K (rotated) and V (raw) go to cache slot pos + row index through the
// page table as E4M3 with one fp32 scale per (position, head); q is kept as FP16 for the tensor-core score product.
// Block = one (row, head): heads [0, Hq) are q, then Hkv k heads, then Hkv v heads.
__global__ void attn_prepare_kernel(Planes qkv, StepBuffers sb, ModelDims d, int al, const __nv_bfloat16* __restrict__ q_norm,
                                    const __nv_bfloat16* __restrict__ k_norm, __half* __restrict__ q, KvPoolDev kv) {
  pdl_sync();  // first statement: see common.cuh
  extern __shared__ float xs[];
  __shared__ float red[32];
  const int m = blockIdx.x, slot = blockIdx.y, dd = threadIdx.x;
  if (m >= *sb.n_rows_total) return;
  const int D = d.D, Hq = d.Hq, Hkv = d.Hkv;
  const bool is_q = slot < Hq, is_v = slot >= Hq + Hkv;
  const int head = is_q ? slot : (is_v ? slot - Hq - Hkv : slot - Hq);
  const int col = is_q ? head * 2 * D + dd : (is_v ? Hq * 2 * D + Hkv * D + head * D + dd : Hq * 2 * D + head * D + dd);
  float x = plane_sum(qkv, m, col);
  if (!is_v) {
    const float rstd = rsqrtf(block_sum(x * x, red) / D + d.eps);
    xs[dd] = x * rstd * (1.f + __bfloat162float((is_q ? q_norm : k_norm)[dd]));
    __syncthreads();
    x = xs[dd];
    if (dd < d.rot) {
      const int half = d.rot / 2, i = dd % half;
      const float inv_freq = powf(d.theta, -2.f * i / d.rot);
      float sn, cs;
      sincosf(float(sb.rope_pos[m]) * inv_freq, &sn, &cs);
      x = dd < half ? xs[dd] * cs - xs[dd + half] * sn : xs[dd] * cs + xs[dd - half] * sn;
    }
    if (is_q) {
      q[(size_t(m) * Hq + head) * D + dd] = __float2half_rn(x);
      return;
    }
  }
  const float amax = block_max(fabsf(x), red);
  const float sc = amax > 0.f ? amax / 448.f : 1.f;
  const int s = sb.seq_of[m], pos = sb.cache_slot[m];
  const int page = kv.tables[size_t(sb.seqs[s].slot) * d.max_pages + pos / d.page_tokens];
  if (page <= 0 || page > d.pool_pages) {
    if (dd == 0) dev_fail(sb.err, kDevBadPage);
    return;
  }
  kv.codes[kv_code_index(d, al, is_v ? 1 : 0, head, page, pos % d.page_tokens, dd)] = to_e4m3(__fdiv_rn(x, sc));
  if (dd == 0) kv.scales[kv_slot_index(d, al, is_v ? 1 : 0, head, page, pos % d.page_tokens)] = sc;
}

__device__ __forceinline__ void cp_async16(void* dst, const void* src, int src_bytes) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(a), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async4(void* dst, const void* src, int src_bytes) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(a), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}


__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
// Position of reduction index c (0..15) inside its group of 16 after the permutation that makes a thread's four
// B-fragment values of one m16n8k16 MMA (logical k 2t, 2t+1, 2t+8, 2t+9) four consecutive bytes 4t .. 4t+3 of the FP8
// operand: physical c = 4t + j sits at logical 2t + j (j < 2) or 8 + 2t + j - 2 (j >= 2).
__host__ __device__ constexpr int perm16(int c) { return (c & 3) < 2 ? 2 * (c >> 2) + (c & 3) : 8 + 2 * (c >> 2) + (c & 3) - 2; }

// Tree-masked attention over the paged FP8 cache, flash-decoding style (the reference's attention_rows,
// src/core/kernels.cu:919-961 with body src/core/attention_body.cuh:262-501, rebuilt for an FP8 cache and any number
// of sequences).  Work item = (sequence, kv head, key chunk, kAttnRowTile query rows); the query rows of a kv head are
// (token row, q head of the group) pairs, so one pass over a K/V tile serves every row of the tree and every q head
// of the group.  Context chunks hold kAttnChunk keys (kAttnChunkShort in a step of few sequences, attn_chunk_keys); the last chunk of a sequence is its in-flight rows (cache slots
// pos .. pos + n_rows), read from the 16-aligned position below pos so that every copy stays 16-byte aligned; a row sees
// an in-flight key only where its ancestor mask has the bit.  K tiles ([key][D]) and V tiles ([D][key], the pool's V
// layout) arrive by 16-byte cp.async into double-buffered shared memory and stay E4M3 there; fragments are converted on
// load (cvt.f16x2.e4m3x2) and the per-position scales are applied to scores and probabilities in fp32.
// Every converted fragment is used for all query rows of the CTA: for Q.K^T the warps split the tile's 64 keys and each
// multiplies its keys with all the rows; the probabilities go through shared memory as FP16; for P.V the warps split
// the head dimension and each again covers all rows.  (Measured: four warps of ~240 registers beat eight of 128 --
// the eight-warp form re-reads the Q and P fragments twice as often and executed 1.5x the instructions.)  The reduction index of both
// products is permuted within groups of 16 (perm16) so that a thread's B fragment is one 32-bit load of four
// consecutive FP8 bytes: Q is stored permuted along d, P along keys.
// Output: per (chunk slot, query row) the unnormalized sum and (max, denominator); attn_combine_kernel merges chunks.
constexpr int kAttnThreads = 128;
template <int D, int G>
__global__ void __launch_bounds__(kAttnThreads, 2)
    attention_kernel(const __half* __restrict__ q, StepBuffers sb, ModelDims d, int al, KvPoolDev kv, float* __restrict__ part_o,
                     float* __restrict__ part_ml, int chunk_slots) {
  pdl_sync();  // first statement: see common.cuh
  constexpr int QS = D + 8;              // halves per Q row in shared memory
  constexpr int KS = D + 16;             // bytes per K row (one key) in shared memory
  constexpr int VS = kAttnKeyTile + 16;  // bytes per V row (one dim, 64 keys) in shared memory
  constexpr int PS = kAttnKeyTile + 8;   // halves per P row in shared memory
  constexpr int MT = kAttnRowTile / 16;  // m16 row tiles per CTA
  constexpr int NW = kAttnThreads / 32;  // warps
  constexpr int DW = D / NW;             // output dims per warp
  constexpr int NTO = DW / 8;            // n8 output tiles per warp
  constexpr int RMAX = kTreeRows * G;
  constexpr int NKT = kAttnKeyTile / (8 * NW);  // n8 key tiles per warp in Q.K^T
  static_assert(kAttnKeyTile % (8 * NW) == 0 && DW % 8 == 0 && (NKT == 1 || NKT == 2), "warps split 64 keys and D dims");
  extern __shared__ __align__(16) uint8_t smem[];
  __half* Qs = reinterpret_cast<__half*>(smem);                          // [RowTile][QS], d permuted within 16s
  __half* Ps = Qs + kAttnRowTile * QS;                                   // [RowTile][PS], keys permuted within 16s
  uint8_t* Ks8 = reinterpret_cast<uint8_t*>(Ps + kAttnRowTile * PS);     // [2][64][KS]
  uint8_t* Vs8 = Ks8 + 2 * kAttnKeyTile * KS;                            // [2][D][VS]
  float* ksc = reinterpret_cast<float*>(Vs8 + 2 * D * VS);               // [2][64]
  float* vsc = ksc + 2 * kAttnKeyTile;                                   // [2][64]
  float* redm = vsc + 2 * kAttnKeyTile;                                  // [NW][RowTile]
  __shared__ int cbase[LING_B200_MAX_SEQS + 1], ibase[LING_B200_MAX_SEQS + 1];
  __shared__ int chunk_sh;  // keys per chunk of this step (attn_chunk_keys)

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g8 = lane >> 2, t4 = lane & 3;
  const int nseq = *sb.n_seqs;
  if (tid == 0) {
    const int chunk = attn_chunk_keys(sb, nseq, d.Hkv, G, kAttnRowTile, int(gridDim.x));
    chunk_sh = chunk;
    int cb = 0, ib = 0;
    for (int s = 0; s < nseq; ++s) {
      cbase[s] = cb, ibase[s] = ib;
      const int nch = (sb.seqs[s].pos + chunk - 1) / chunk + 1;
      const int nrg = (sb.seqs[s].n_rows * G + kAttnRowTile - 1) / kAttnRowTile;
      cb += nch, ib += d.Hkv * nch * nrg;
    }
    cbase[nseq] = cb, ibase[nseq] = ib;
  }
  __syncthreads();
  const int chunk = chunk_sh;
  const float inv_sqrt_d = rsqrtf(float(D));
  const int pt = d.page_tokens, lp = 31 - __clz(pt), pmask = pt - 1;  // pages hold 16, 32 or 64 positions
  // ldmatrix row addresses of this lane inside a 16x16 A tile: matrices 0..3 = (rows 0-7, k 0-7), (rows 8-15, k 0-7),
  // (rows 0-7, k 8-15), (rows 8-15, k 8-15)
  const int lm_row = (lane & 7) + ((lane >> 3) & 1) * 8, lm_col = (lane >> 4) * 8;
  // this thread's part in the tile copies: K = (key, 16-byte part of its D bytes), V = (dim, 16 positions)
  constexpr int PK = D / 16, KPI = kAttnThreads / PK;
  const int k_part = tid % PK, k_key0 = tid / PK;
  const int v_kc = (tid & 3) * 16, v_dd0 = tid >> 2;

  for (int item = blockIdx.x; item < ibase[nseq]; item += gridDim.x) {
    int s = 0;
    while (ibase[s + 1] <= item) ++s;
    const SeqDev sq = sb.seqs[s];
    const int nch = (sq.pos + chunk - 1) / chunk + 1;
    const int nrg = (sq.n_rows * G + kAttnRowTile - 1) / kAttnRowTile;
    const int loc = item - ibase[s];
    const int hk = loc / (nch * nrg), ch = (loc % (nch * nrg)) / nrg, rg = loc % nrg;
    const int slot_idx = cbase[s] * d.Hkv + hk * nch + ch;
    if (slot_idx >= chunk_slots) {
      if (tid == 0) dev_fail(sb.err, kDevBadPage);
      continue;
    }
    const bool tail = ch == nch - 1;
    // keys [key_base + key_lo, key_base + key_hi) count; a tail chunk starts at the 16-aligned position below pos
    const int key_base = tail ? (sq.pos & ~15) : ch * chunk;
    const int key_lo = tail ? sq.pos - key_base : 0;
    const int key_hi = tail ? key_lo + sq.n_rows : min(chunk, sq.pos - key_base);
    const int R = sq.n_rows * G, r_begin = rg * kAttnRowTile, r0 = sb.row0[s];
    const int mt_n = min(MT, (R - r_begin + 15) / 16);  // row tiles that hold a real row
    const int* table = kv.tables + size_t(sq.slot) * d.max_pages;
    const uint8_t* kcodes = kv.codes + kv_slot_index(d, al, 0, hk, 0, 0) * D;
    const uint8_t* vcodes = kv.codes + kv_slot_index(d, al, 1, hk, 0, 0) * D;
    const float* kscales = kv.scales + kv_slot_index(d, al, 0, hk, 0, 0);
    const float* vscales = kv.scales + kv_slot_index(d, al, 1, hk, 0, 0);

    __syncthreads();  // the previous item's readers of Qs and the tiles are done
    for (int idx = tid; idx < kAttnRowTile * (D / 8); idx += kAttnThreads) {
      const int r = idx / (D / 8), part = idx % (D / 8);
      uint4 val = make_uint4(0, 0, 0, 0);
      const int rr = r_begin + r;
      if (rr < R) val = *reinterpret_cast<const uint4*>(q + (size_t(r0 + rr / G) * d.Hq + hk * G + rr % G) * D + part * 8);
      // physical dims 8 * (part & 1) + {0,1 | 2,3 | 4,5 | 6,7} of the 16-group go to their permuted places
      uint32_t* dst = reinterpret_cast<uint32_t*>(Qs + size_t(r) * QS + (part >> 1) * 16);
      const int c0 = (part & 1) * 8;
      dst[perm16(c0) >> 1] = val.x, dst[perm16(c0 + 2) >> 1] = val.y, dst[perm16(c0 + 4) >> 1] = val.z, dst[perm16(c0 + 6) >> 1] = val.w;
    }
    auto page_of = [&](int pos) {
      const int page = table[pos >> lp];
      return (page < 0 || page > d.pool_pages) ? 0 : page;  // an unmapped position lands in the reserved page
    };
    auto load_tile = [&](int tile, int buf) {
      const int k0 = tile * kAttnKeyTile;
      // K: one key's D bytes are contiguous in its page
#pragma unroll
      for (int it = 0; it < kAttnKeyTile / KPI; ++it) {
        const int key = it * KPI + k_key0;
        const bool valid = k0 + key < key_hi;
        const int pos = key_base + k0 + key;
        const size_t at = valid ? (size_t(page_of(pos)) << lp) + (pos & pmask) : 0;
        cp_async16(Ks8 + (size_t(buf) * kAttnKeyTile + key) * KS + k_part * 16, kcodes + at * D + k_part * 16, valid ? 16 : 0);
        if (k_part == 0) {
          cp_async4(ksc + buf * kAttnKeyTile + key, kscales + at, valid ? 4 : 0);
          cp_async4(vsc + buf * kAttnKeyTile + key, vscales + at, valid ? 4 : 0);
        }
      }
      // V: one dim's 16 consecutive positions are contiguous in their page (pages hold a multiple of 16 positions); this
      // thread's 16 positions are the same for all its dims
      {
        const bool valid = k0 + v_kc < key_hi;
        const int pos = key_base + k0 + v_kc;
        const uint8_t* src = vcodes + (valid ? (size_t(page_of(pos)) << lp) * D + (pos & pmask) : 0);
#pragma unroll
        for (int it = 0; it < D / (kAttnThreads / 4); ++it) {
          const int dd = it * (kAttnThreads / 4) + v_dd0;
          cp_async16(Vs8 + (size_t(buf) * D + dd) * VS + v_kc, src + (valid ? size_t(dd) << lp : 0), valid ? 16 : 0);
        }
      }
      cp_async_commit();
    };
    // Positions past key_hi inside the last 16-position piece hold whatever the page held; their probability is zero,
    // but 0 x NaN is NaN, so their V codes are cleared before use.
    auto clear_v_tail = [&](int tile, int buf) {
      const int k0 = tile * kAttnKeyTile, first = key_hi - k0;  // first invalid key of this tile
      if (first >= kAttnKeyTile || (first & 15) == 0) return;
      const int last = (first | 15) + 1;
      for (int idx = tid; idx < D * (last - first); idx += kAttnThreads)
        Vs8[(size_t(buf) * D + idx / (last - first)) * VS + first + idx % (last - first)] = 0;
    };

    // This thread's rows: row tile mt holds rows mt * 16 + g8 (index 2 * mt) and + 8 (index 2 * mt + 1), the same in
    // every warp; O[mt][nt] covers output dims warp * DW + nt * 8 + 2 * t4 .. + 1.
    float O[MT][NTO][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int i = 0; i < NTO; ++i) O[mt][i][0] = O[mt][i][1] = O[mt][i][2] = O[mt][i][3] = 0.f;
    float m_run[2 * MT], l_run[2 * MT];
    uint32_t anc[2 * MT];
#pragma unroll
    for (int r = 0; r < 2 * MT; ++r) {
      m_run[r] = -INFINITY, l_run[r] = 0.f;
      const int row = r_begin + (r >> 1) * 16 + g8 + (r & 1) * 8;
      anc[r] = !tail ? 0xffffffffu : (row < R ? sb.anc[r0 + row / G] : 0u);
    }

    const int ntiles = (key_hi + kAttnKeyTile - 1) / kAttnKeyTile;
    load_tile(0, 0);
    for (int tile = 0; tile < ntiles; ++tile) {
      const int buf = tile & 1;
      if (tile + 1 < ntiles) {
        load_tile(tile + 1, buf ^ 1);
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      __syncthreads();
      if (tile == ntiles - 1) {
        clear_v_tail(tile, buf);
        __syncthreads();
      }
      const uint8_t* Kt = Ks8 + size_t(buf) * kAttnKeyTile * KS;
      const uint8_t* Vt = Vs8 + size_t(buf) * D * VS;
      // ---- S = Q . K^T for this warp's 8 * NKT keys and every row tile
      float S[MT][NKT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < NKT; ++nt) S[mt][nt][0] = S[mt][nt][1] = S[mt][nt][2] = S[mt][nt][3] = 0.f;
      const uint8_t* ka = Kt + size_t(warp * 8 * NKT + g8) * KS + 4 * t4;
      const __half* qa = Qs + size_t(lm_row) * QS + lm_col;
#pragma unroll 4
      for (int kt = 0; kt < D / 16; ++kt) {
        uint32_t bk[NKT][2];
#pragma unroll
        for (int nt = 0; nt < NKT; ++nt) {
          const uint32_t kw = *reinterpret_cast<const uint32_t*>(ka + size_t(nt * 8) * KS + kt * 16);
          bk[nt][0] = e4m3x2_to_h2(uint16_t(kw)), bk[nt][1] = e4m3x2_to_h2(uint16_t(kw >> 16));
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          if (mt < mt_n) {
            uint32_t a[4];
            ldmatrix_x4(a, qa + size_t(mt * 16) * QS + kt * 16);
#pragma unroll
            for (int nt = 0; nt < NKT; ++nt) mma_f16(S[mt][nt], a[0], a[1], a[2], a[3], bk[nt][0], bk[nt][1]);
          }
        }
      }
      // ---- scale and mask; the tile's row maxima go through shared memory (each warp saw a part of the keys)
      const int k0 = tile * kAttnKeyTile;
      float kscl[NKT][2], vscl[NKT][2];
      bool inrange[NKT][2];
#pragma unroll
      for (int nt = 0; nt < NKT; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int key = warp * 8 * NKT + nt * 8 + 2 * t4 + e;
          kscl[nt][e] = ksc[buf * kAttnKeyTile + key] * inv_sqrt_d;
          vscl[nt][e] = vsc[buf * kAttnKeyTile + key] * kPScale;
          inrange[nt][e] = k0 + key >= key_lo && k0 + key < key_hi;
        }
      const int kbit = k0 + warp * 8 * NKT + 2 * t4 - key_lo;  // + nt * 8 + e: the key's bit in the ancestor mask (tail chunk)
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float tm = -INFINITY;
#pragma unroll
          for (int nt = 0; nt < NKT; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const bool vis = inrange[nt][e] && (!tail || ((anc[2 * mt + h] >> ((kbit + nt * 8 + e) & 31)) & 1u));
              const float sv = vis ? S[mt][nt][2 * h + e] * kscl[nt][e] : -INFINITY;
              S[mt][nt][2 * h + e] = sv;
              tm = fmaxf(tm, sv);
            }
          tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 1));
          tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 2));
          if (t4 == 0) redm[warp * kAttnRowTile + mt * 16 + h * 8 + g8] = tm;
        }
      __syncthreads();
      // ---- probabilities (FP16, times the key's V scale) to shared memory at their permuted key positions
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int r = 2 * mt + h, row = mt * 16 + h * 8 + g8;
          float tmax = redm[row];
#pragma unroll
          for (int w = 1; w < NW; ++w) tmax = fmaxf(tmax, redm[w * kAttnRowTile + row]);
          const float mnew = fmaxf(m_run[r], tmax);
          const float muse = mnew == -INFINITY ? 0.f : mnew;
          const float corr = __expf(m_run[r] - muse);  // exp(-inf) = 0 on the first tile
          m_run[r] = mnew;
          float lsum = 0.f;
#pragma unroll
          for (int nt = 0; nt < NKT; ++nt) {
            const float p0 = __expf(S[mt][nt][2 * h] - muse), p1 = __expf(S[mt][nt][2 * h + 1] - muse);
            lsum += p0 + p1;
            const int key = warp * 8 * NKT + nt * 8 + 2 * t4;  // even: the pair stays adjacent under perm16
            *reinterpret_cast<uint32_t*>(Ps + size_t(row) * PS + (key & ~15) + perm16(key & 15)) = pack_h2(p0 * vscl[nt][0], p1 * vscl[nt][1]);
          }
          l_run[r] = l_run[r] * corr + lsum;  // this thread's keys only; summed over the quad and the warps at the end
#pragma unroll
          for (int i = 0; i < NTO; ++i) O[mt][i][2 * h] *= corr, O[mt][i][2 * h + 1] *= corr;
        }
      __syncthreads();
      // ---- O += P . V for this warp's D / NW output dims and every row tile
      const uint8_t* va = Vt + size_t(warp * DW + g8) * VS + 4 * t4;
      const __half* pa = Ps + size_t(lm_row) * PS + lm_col;
#pragma unroll
      for (int kk = 0; kk < kAttnKeyTile / 16; ++kk) {
        uint32_t a[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
          if (mt < mt_n) ldmatrix_x4(a[mt], pa + size_t(mt * 16) * PS + kk * 16);
#pragma unroll
        for (int nt = 0; nt < NTO; ++nt) {
          const uint32_t vw = *reinterpret_cast<const uint32_t*>(va + size_t(nt * 8) * VS + kk * 16);
          const uint32_t b0 = e4m3x2_to_h2(uint16_t(vw)), b1 = e4m3x2_to_h2(uint16_t(vw >> 16));
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
            if (mt < mt_n) mma_f16(O[mt][nt], a[mt][0], a[mt][1], a[mt][2], a[mt][3], b0, b1);
        }
      }
      __syncthreads();
    }
    // ---- denominators: over the quad, then over the warps (through redm, free after the last tile's barrier)
#pragma unroll
    for (int r = 0; r < 2 * MT; ++r) {
      l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
      l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
      if (t4 == 0) redm[warp * kAttnRowTile + (r >> 1) * 16 + (r & 1) * 8 + g8] = l_run[r];
    }
    __syncthreads();
    float* po = part_o + size_t(slot_idx) * RMAX * D;
    float* pm = part_ml + size_t(slot_idx) * RMAX * 2;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int lrow = mt * 16 + h * 8 + g8, row = r_begin + lrow;
        if (row >= R) continue;
#pragma unroll
        for (int nt = 0; nt < NTO; ++nt)
          *reinterpret_cast<float2*>(po + size_t(row) * D + warp * DW + nt * 8 + 2 * t4) = make_float2(O[mt][nt][2 * h], O[mt][nt][2 * h + 1]);
        if (warp == 0 && t4 == 0) {
          float l = redm[lrow];
#pragma unroll
          for (int w = 1; w < NW; ++w) l += redm[w * kAttnRowTile + lrow];
          pm[row * 2] = m_run[2 * mt + h];
          pm[row * 2 + 1] = l;
        }
      }
  }
}

// Merges a row's chunks (the reference's attention_combine, src/core/attention_body.cuh:506-525), applies the output gate
// out * sigmoid(gate) (src/core/kernels.cu:314-318; the gate is the second D values of each q head's projection) and
// writes the FP8 copy for the o projection.  One block per (packed row, 128 or D output columns, whichever is larger):
// a long context has hundreds of chunks, so the chunks are spread over the block -- a thread owns four columns and one of
// NG chunk groups (chunk c belongs to group c mod NG); the chunk weights exp(m_c - max) are computed once per block in
// shared memory; the groups' sums meet in shared memory and are added in group order, so the result does not depend on
// how the block is scheduled.  The first group's threads (whole warps of 128 columns) finish and quantize.
template <int G>
__global__ void __launch_bounds__(256)
    attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, Planes qkv, StepBuffers sb,
                        ModelDims d, QuantOut q, float* __restrict__ raw, int max_chunks, int tile_rows, int budget, int chunk_slots) {
  pdl_sync();  // first statement: see common.cuh
  constexpr int RMAX = kTreeRows * G;
  extern __shared__ __align__(16) float csm[];  // [HB][max_chunks] chunk weights, [4] denominators, [NG][CB] partial sums (max_chunks a multiple of 4)
  __shared__ float red[32];
  const int m = blockIdx.x;
  if (m >= *sb.n_rows_total) return;
  const int D = d.D, CB = D > 128 ? D : 128, HB = CB / D;  // columns and heads of this block
  const int CT = CB / 4, NG = blockDim.x / CT;              // column threads, chunk groups
  const int ct = threadIdx.x % CT, grp = threadIdx.x / CT;
  const int c0 = blockIdx.y * CB;
  if (c0 >= q.K_pad) return;
  const int s = sb.seq_of[m], local = sb.local[m];
  const int chunk = attn_chunk_keys(sb, *sb.n_seqs, d.Hkv, G, tile_rows, budget);
  // chunk slots of the sequences ahead of this one: every warp adds them up for itself, a lane per sequence (a serial loop
  // over up to 64 sequences in every block of a thousand-row step was a sixth of the kernel's time there)
  int cb = 0;
  for (int t = threadIdx.x & 31; t < s; t += 32) cb += (sb.seqs[t].pos + chunk - 1) / chunk + 1;
  cb = __reduce_add_sync(0xffffffffu, cb);
  const int nch = min(max_chunks, (sb.seqs[s].pos + chunk - 1) / chunk + 1);
  float* wgt = csm;                       // [HB][max_chunks]
  float* den = csm + HB * max_chunks;     // [HB]
  float* acc = den + 4;                   // [NG][CB], 16-byte aligned: max_chunks is a multiple of 4
  // ---- chunk weights and denominators per head of the block
  for (int hb = 0; hb < HB; ++hb) {
    const int hq = c0 / D + hb;
    if (hq * D >= q.K) {  // a head past the real columns (padding): weights zero
      for (int ch = threadIdx.x; ch < nch; ch += blockDim.x) wgt[hb * max_chunks + ch] = 0.f;
      if (threadIdx.x == 0) den[hb] = 1.f;
      __syncthreads();
      continue;
    }
    const int hk = hq / G, r = local * G + hq % G;
    const float* ml = part_ml + ((size_t(cb) * d.Hkv + size_t(hk) * nch) * RMAX + r) * 2;
    // chunk slots past the buffers' end were never written (the attention kernel skipped their items and set the error
    // word): they are not read either
    const int nlim = max(0, min(nch, chunk_slots - (cb * d.Hkv + hk * nch)));
    for (int ch = nlim + threadIdx.x; ch < nch; ch += blockDim.x) wgt[hb * max_chunks + ch] = 0.f;
    float mx = -INFINITY;
    for (int ch = threadIdx.x; ch < nlim; ch += blockDim.x) mx = fmaxf(mx, ml[size_t(ch) * RMAX * 2]);
    mx = block_max(mx, red);
    float dsum = 0.f;
    for (int ch = threadIdx.x; ch < nlim; ch += blockDim.x) {
      const float mc = ml[size_t(ch) * RMAX * 2];
      const float w = mc == -INFINITY ? 0.f : __expf(mc - mx);  // an empty chunk weighs nothing
      wgt[hb * max_chunks + ch] = w;
      dsum = fmaf(ml[size_t(ch) * RMAX * 2 + 1], w, dsum);
    }
    dsum = block_sum(dsum, red);
    if (threadIdx.x == 0) den[hb] = dsum;
    __syncthreads();
  }
  // ---- numerators: this thread's four columns over its group's chunks
  const int c = c0 + ct * 4;
  float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
  const int hb = (ct * 4) / D;
  if (c < q.K) {
    const int hq = c / D, dd = c % D, hk = hq / G, r = local * G + hq % G;
    const float* po = part_o + ((size_t(cb) * d.Hkv + size_t(hk) * nch) * RMAX + r) * D + dd;
    const float* w = wgt + hb * max_chunks;
    const int nlim = max(0, min(nch, chunk_slots - (cb * d.Hkv + hk * nch)));
#pragma unroll 4
    for (int ch = grp; ch < nlim; ch += NG) {
      const float4 o = *reinterpret_cast<const float4*>(po + size_t(ch) * RMAX * D);
      const float wc = w[ch];
      num.x = fmaf(o.x, wc, num.x), num.y = fmaf(o.y, wc, num.y), num.z = fmaf(o.z, wc, num.z), num.w = fmaf(o.w, wc, num.w);
    }
  }
  *reinterpret_cast<float4*>(acc + grp * CB + ct * 4) = num;
  __syncthreads();
  if (grp != 0) return;  // whole warps: CT is a multiple of 32
  float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
  if (c < q.K) {
    for (int g2 = 0; g2 < NG; ++g2) {
      const float4 a = *reinterpret_cast<const float4*>(acc + g2 * CB + ct * 4);
      x.x += a.x, x.y += a.y, x.z += a.z, x.w += a.w;
    }
    const float inv = 1.f / (den[hb] * kPScale);
    x = make_float4(x.x * inv, x.y * inv, x.z * inv, x.w * inv);
    if (qkv.p) {  // the output gate, where the q|gate projection is given (a parity entry may ask for the ungated rows)
      const int hq = c / D, dd = c % D;
      const float4 gate = plane_sum4(qkv, m, hq * 2 * D + D + dd);
      x = make_float4(x.x * sigmoidf(gate.x), x.y * sigmoidf(gate.y), x.z * sigmoidf(gate.z), x.w * sigmoidf(gate.w));
    }
    if (raw) *reinterpret_cast<float4*>(raw + size_t(m) * q.K + c) = x;
  }
  quant_store4(x, c, m, q);
}

// ---------------------------------------------------------------------------------------------- argmax / accept
__device__ __forceinline__ bool better(float v, int i, float v2, int i2) { return v > v2 || (v == v2 && i < i2); }

// Second stage of the argmax: merges the head GEMM's per-tile winners with the first stage's comparison, so the result
// does not depend on the tiling (src/core/topk.cu:1-9,19).
__global__ void __launch_bounds__(256)
    argmax_reduce_kernel(const float* __restrict__ tile_val, const int* __restrict__ tile_idx, int tiles, int rows_alloc,
                         int* __restrict__ ids, float* __restrict__ vals, const int* __restrict__ n_rows) {
  pdl_sync();  // first statement: see common.cuh
  __shared__ float sv[256];
  __shared__ int si[256];
  const int m = blockIdx.x;
  if (m >= *n_rows) return;
  float bv = -FLT_MAX;
  int bi = 0x7fffffff;
  for (int t = threadIdx.x; t < tiles; t += blockDim.x) {
    const float v = tile_val[size_t(t) * rows_alloc + m];
    const int i = tile_idx[size_t(t) * rows_alloc + m];
    if (v == v && better(v, i, bv, bi)) bv = v, bi = i;
  }
  sv[threadIdx.x] = bv, si[threadIdx.x] = bi;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o && better(sv[threadIdx.x + o], si[threadIdx.x + o], sv[threadIdx.x], si[threadIdx.x]))
      sv[threadIdx.x] = sv[threadIdx.x + o], si[threadIdx.x] = si[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) ids[m] = si[0], vals[m] = sv[0];
}

// topk_rows with K = 1 over materialized logits (src/core/topk.cu:83-129): one block per row.
__global__ void __launch_bounds__(256)
    argmax_rows_kernel(const float* __restrict__ logits, int vocab, int* __restrict__ ids, float* __restrict__ vals) {
  pdl_sync();  // first statement: see common.cuh
  __shared__ float sv[256];
  __shared__ int si[256];
  const int m = blockIdx.x;
  float bv = -FLT_MAX;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = logits[size_t(m) * vocab + i];
    if (v == v && better(v, i, bv, bi)) bv = v, bi = i;
  }
  sv[threadIdx.x] = bv, si[threadIdx.x] = bi;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o && better(sv[threadIdx.x + o], si[threadIdx.x + o], sv[threadIdx.x], si[threadIdx.x]))
      sv[threadIdx.x] = sv[threadIdx.x + o], si[threadIdx.x] = si[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) ids[m] = si[0], vals[m] = sv[0];
}

// One thread per sequence: the finiteness guard over its rows (require_finite_topk, src/core/sampling.cpp:20-23), then
// accept_tree_greedy (src/core/tree.cpp:148-166): from the root, the first child in row order whose token is the current
// row's argmax; `next` is the argmax that no child matched.  out = the accepted drafts, then next
// (src/core/speculate.cpp:1066-1067).
__global__ void accept_kernel(StepBuffers sb, int vocab) {
  pdl_sync();  // first statement: see common.cuh
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= *sb.n_seqs) return;
  const SeqDev q = sb.seqs[s];
  const int r0 = sb.row0[s], n = q.n_rows;
  ling_b200_seq_result R;
  R.status = LING_B200_SEQ_OK, R.n_path = 0, R.next_token = 0, R.n_out = 0;
  for (int i = 0; i < kTreeRows; ++i) R.path[i] = 0;
  for (int i = 0; i < kTreeRows + 1; ++i) R.out[i] = 0;
  for (int r = 0; r < n; ++r) {
    const float v = sb.argmax_val[r0 + r];
    const int id = sb.argmax_id[r0 + r];
    if (!isfinite(v) || v == -FLT_MAX || id < 0 || id >= vocab) R.status = LING_B200_SEQ_NONFINITE;
  }
  if (R.status == LING_B200_SEQ_OK) {
    const int* par = sb.in_parent + s * kTreeRows;
    const int* tok = sb.in_token + s * kTreeRows;
    const int* forced = sb.in_force + s * kTreeRows;
    int u = 0;
    R.path[R.n_path++] = 0;
    for (;;) {
      const int x = (q.has_force && forced[u] >= 0) ? forced[u] : sb.argmax_id[r0 + u];  // a negative entry imposes nothing
      int child = -1;
      for (int c = u + 1; c < n; ++c)
        if (par[c] == u && tok[c] == x) {
          child = c;
          break;
        }
      if (child < 0) {
        R.next_token = x;
        break;
      }
      R.path[R.n_path++] = child;
      u = child;
    }
    for (int j = 1; j < R.n_path; ++j) R.out[R.n_out++] = tok[R.path[j]];
    R.out[R.n_out++] = R.next_token;
  }
  sb.results[s] = R;
}

// tree_gather for the KV cache (src/core/kernels.cu:481-498): cache slot pos + path[j] moves to pos + j, j ascending,
// through the page table (source and destination may sit in different pages); codes and the per-position scale.
// Block = one (sequence, layer, K|V, kv head).
__global__ void __launch_bounds__(64) kv_compact_kernel(StepBuffers sb, ModelDims d, KvPoolDev kv) {
  pdl_sync();  // first statement: see common.cuh
  const int s = blockIdx.y;
  if (s >= *sb.n_seqs) return;
  const ling_b200_seq_result* R = sb.results + s;
  if (R->status != 0) return;
  const int hk = blockIdx.x % d.Hkv, kvi = (blockIdx.x / d.Hkv) % 2, al = blockIdx.x / (2 * d.Hkv);
  const SeqDev q = sb.seqs[s];
  const int* table = kv.tables + size_t(q.slot) * d.max_pages;
  for (int j = 1; j < R->n_path; ++j) {
    const int src = q.pos + R->path[j], dst = q.pos + j;
    if (src != dst) {
      const int pa = table[src / d.page_tokens], pb = table[dst / d.page_tokens];
      const int ta = src % d.page_tokens, tb = dst % d.page_tokens;
      for (int i = threadIdx.x; i < d.D; i += blockDim.x)
        kv.codes[kv_code_index(d, al, kvi, hk, pb, tb, i)] = kv.codes[kv_code_index(d, al, kvi, hk, pa, ta, i)];
      if (threadIdx.x == 0) kv.scales[kv_slot_index(d, al, kvi, hk, pb, tb)] = kv.scales[kv_slot_index(d, al, kvi, hk, pa, ta)];
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------------------------- weights, synthetic data
// One warp per (row, 128-column block): BF16 rounding, scale = amax / 448, E4M3 codes; padding columns get zero codes.
// The source is a host-supplied fp32 matrix [rows][K] or the generator.  Row r lands at row row_off + r of the
// destination, whose scales are stored block-major with stride N_pad (several tensors share one fused matrix).
__global__ void __launch_bounds__(256)
    quant_weight_kernel(const float* __restrict__ src, uint64_t key, float std_, int from_generator, uint8_t* __restrict__ codes,
                        float* __restrict__ scales, int row_off, int K, int N_pad, int K_pad) {
  pdl_sync();  // first statement: see common.cuh
  const int r = blockIdx.x, n = row_off + r, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, KB = K_pad / 128;
  for (int kb = blockIdx.y * 8 + warp; kb < KB; kb += gridDim.y * 8) {
    const int c = kb * 128 + lane * 4;
    float x[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      x[i] = 0.f;
      if (c + i < K) {
        const size_t e = size_t(r) * K + c + i;
        x[i] = bf16_round(from_generator ? synth_z(key, e) * std_ : src[e]);
      }
    }
    const float amax = warp_max(fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3]))));
    const float sc = amax > 0.f ? amax / 448.f : 1.f;
    uchar4 o;
    o.x = to_e4m3(__fdiv_rn(x[0], sc)), o.y = to_e4m3(__fdiv_rn(x[1], sc));
    o.z = to_e4m3(__fdiv_rn(x[2], sc)), o.w = to_e4m3(__fdiv_rn(x[3], sc));
    *reinterpret_cast<uchar4*>(codes + size_t(n) * K_pad + c) = o;
    if (lane == 0) scales[size_t(kb) * N_pad + n] = sc;
  }
}

// Plain fp32 rows to the activation encoding (codes [rows][K_pad], scales [KB][rows_alloc]).
__global__ void __launch_bounds__(256) quant_acts_kernel(const float* __restrict__ x, QuantOut q) {
  pdl_sync();  // first statement: see common.cuh
  const int m = blockIdx.x;
  for (int c0 = 0; c0 < q.K_pad; c0 += 1024) {
    const int c = c0 + threadIdx.x * 4;
    if (c - (threadIdx.x & 31) * 4 >= q.K_pad) break;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < q.K) {
      const float* r = x + size_t(m) * q.K + c;
      v = make_float4(r[0], c + 1 < q.K ? r[1] : 0.f, c + 2 < q.K ? r[2] : 0.f, c + 3 < q.K ? r[3] : 0.f);
    }
    quant_store4(v, c, m, q);
  }
}

__global__ void fill_bf16_kernel(const float* __restrict__ src, uint64_t key, float std_, float bias, int from_generator,
                                 __nv_bfloat16* __restrict__ dst, size_t n) {
  pdl_sync();  // first statement: see common.cuh
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x)
    dst[i] = __float2bfloat16(from_generator ? synth_z(key, i) * std_ + bias : src[i]);
}
__global__ void fill_f32_kernel(uint64_t key, float std_, float* __restrict__ dst, size_t n) {
  pdl_sync();  // first statement: see common.cuh
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x)
    dst[i] = synth_z(key, i) * std_;
}

// K and V of positions [from, from + n) of one attention layer into the slot's pages, quantized as the step quantizes
// them.  Block = (position, kv head, K|V), one thread per dim.
__global__ void kv_write_kernel(const float* __restrict__ k, const float* __restrict__ v, uint64_t key_k, uint64_t key_v,
                                int from_generator, ModelDims d, int al, int slot, int from, KvPoolDev kv, int* err) {
  pdl_sync();  // first statement: see common.cuh
  __shared__ float red[32];
  const int i = blockIdx.x, h = blockIdx.y, kvi = blockIdx.z, dd = threadIdx.x, pos = from + i;
  const size_t e = (size_t(from_generator ? pos : i) * d.Hkv + h) * d.D + dd;
  const float x = from_generator ? synth_z(kvi ? key_v : key_k, e) : (kvi ? v : k)[e];
  const float amax = block_max(fabsf(x), red);
  const float sc = amax > 0.f ? amax / 448.f : 1.f;
  const int page = kv.tables[size_t(slot) * d.max_pages + pos / d.page_tokens];
  if (page <= 0 || page > d.pool_pages) {
    if (dd == 0) dev_fail(err, kDevBadPage);
    return;
  }
  kv.codes[kv_code_index(d, al, kvi, h, page, pos % d.page_tokens, dd)] = to_e4m3(__fdiv_rn(x, sc));
  if (dd == 0) kv.scales[kv_slot_index(d, al, kvi, h, page, pos % d.page_tokens)] = sc;
}

// A whole page copied for copy-on-write (the reference's kv_pages_copy role, src/core/kernels.cu:513-527).
__global__ void kv_page_copy_kernel(ModelDims d, KvPoolDev kv, int src, int dst) {
  pdl_sync();  // first statement: see common.cuh
  const int lane_kv = blockIdx.x;  // (layer, K|V, head)
  const size_t a = (size_t(lane_kv) * (d.pool_pages + 1) + src) * d.page_tokens;
  const size_t b = (size_t(lane_kv) * (d.pool_pages + 1) + dst) * d.page_tokens;
  const int words = d.page_tokens * d.D / 4;
  for (int i = threadIdx.x; i < words; i += blockDim.x)
    reinterpret_cast<uint32_t*>(kv.codes + b * d.D)[i] = reinterpret_cast<const uint32_t*>(kv.codes + a * d.D)[i];
  for (int i = threadIdx.x; i < d.page_tokens; i += blockDim.x) kv.scales[b + i] = kv.scales[a + i];
}

__global__ void f32_to_half_kernel(const float* __restrict__ src, __half* __restrict__ dst, size_t n) {
  pdl_sync();  // first statement: see common.cuh
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) dst[i] = __float2half_rn(src[i]);
}

__global__ void flush_kernel(float* __restrict__ buf, size_t n) {
  pdl_sync();  // first statement: see common.cuh
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) buf[i] = float(i);
}

template <int D, int G>
constexpr size_t attn_smem() {
  return size_t(kAttnRowTile) * (D + 8) * 2 + size_t(kAttnRowTile) * (kAttnKeyTile + 8) * 2 + size_t(2) * kAttnKeyTile * (D + 16) +
         size_t(2) * D * (kAttnKeyTile + 16) + size_t(4) * kAttnKeyTile * 4 + size_t(kAttnThreads / 32) * kAttnRowTile * 4;
}

}  // namespace

// ---------------------------------------------------------------------------------------------- launchers
int pack_launch(const StepBuffers& sb, const ModelDims& d, cudaStream_t s) {
  LB_CUDA(launch_kernel(pack_kernel, dim3(d.max_seqs), dim3(32), size_t(0), s, sb, d));
  LB_LAUNCH("pack_kernel");
  return LING_B200_OK;
}

int kernels_norm_stamps(unsigned long long* stamps) {
  LB_CUDA(cudaMemcpyToSymbol(g_norm_stamps, &stamps, sizeof(stamps)));
  return LING_B200_OK;
}

int norm_quant_launch(float* h, const Planes& add, const int* ids, const __nv_bfloat16* embed, const __nv_bfloat16* w,
                      float* xn, const QuantOut& q, const int* n_rows, int rows_grid, int H, float eps, cudaStream_t s) {
  const int chunks = ceil_div(q.K_pad, 1024);
  if (chunks > 8) {
    set_error("norm: hidden size above 8192");
    return LING_B200_ERR_UNSUPPORTED;
  }
  LB_CUDA(launch_kernel_cluster(norm_quant_kernel, dim3(chunks, rows_grid), dim3(256), size_t(0), chunks, s, h, add, ids, embed, w, xn,
                                q, n_rows, H, eps));
  LB_LAUNCH("norm_quant_kernel");
  return LING_B200_OK;
}

int add_planes_launch(float* h, const Planes& add, const int* n_rows, int rows_grid, int H, cudaStream_t s) {
  if (H % 4 != 0 || !add.p) return LING_B200_ERR_ARG;
  LB_CUDA(launch_kernel(add_planes_kernel, dim3(rows_grid), dim3(256), size_t(0), s, h, add, n_rows, H));
  LB_LAUNCH("add_planes_kernel");
  return LING_B200_OK;
}

int tap_launch(const float* h, const Planes& add, float* out, const int* n_rows, int rows_grid, int H, cudaStream_t s) {
  LB_CUDA(launch_kernel(tap_kernel, dim3(rows_grid), dim3(256), size_t(0), s, h, add, out, n_rows, H));
  LB_LAUNCH("tap_kernel");
  return LING_B200_OK;
}

int copy_rows_launch(const float* src, float* out, const int* n_rows, int rows_grid, int H, cudaStream_t s) {
  Planes none;
  LB_CUDA(launch_kernel(tap_kernel, dim3(rows_grid), dim3(256), size_t(0), s, src, none, out, n_rows, H));
  LB_LAUNCH("tap_kernel");
  return LING_B200_OK;
}

int ab_gating_rows_launch(const float* xn, const __nv_bfloat16* wa, const __nv_bfloat16* wb, const __nv_bfloat16* A_log,
                          const __nv_bfloat16* dt_bias, float* g, float* beta, int M, int H, int HV, cudaStream_t s) {
  if (M < 1 || H % 4 != 0) return LING_B200_ERR_ARG;
  LB_CUDA(launch_kernel(ab_gating_rows_kernel, dim3(ceil_div(HV, 4), ceil_div(M, 4)), dim3(128), size_t(0), s, xn, wa, wb, A_log, dt_bias, g, beta, M, H, HV));
  LB_LAUNCH("ab_gating_rows_kernel");
  return LING_B200_OK;
}

int ab_gating_launch(const float* xn, const __nv_bfloat16* wa, const __nv_bfloat16* wb, const __nv_bfloat16* A_log,
                     const __nv_bfloat16* dt_bias, float* g, float* beta, const int* n_rows, int rows_grid, int H, int HV,
                     cudaStream_t s) {
  LB_CUDA(launch_kernel(ab_gating_kernel, dim3(HV, rows_grid), dim3(128), size_t(0), s, xn, wa, wb, A_log, dt_bias, g, beta, n_rows, H, HV));
  LB_LAUNCH("ab_gating_kernel");
  return LING_B200_OK;
}

int conv_tree_launch(const Planes& in, const StepBuffers& sb, const ModelDims& d, const __nv_bfloat16* convw,
                     const float* conv_state, size_t conv_slot_stride, float* pre, float* post, int rows_grid, cudaStream_t s) {
  LB_CUDA(launch_kernel(conv_tree_kernel, dim3(dim3(ceil_div(d.C, 256), rows_grid)), dim3(256), size_t(0), s, in, sb, d.C, d.Hk, d.Dk, convw, conv_state, conv_slot_stride, pre, post));
  LB_LAUNCH("conv_tree_kernel");
  return LING_B200_OK;
}

int gdn_tree_launch(const float* post, const float* g, const float* beta, const StepBuffers& sb, const ModelDims& d,
                    const float* state, size_t state_slot_stride, float* core, int grid, cudaStream_t s) {
  if (d.Dk == 128)
    LB_CUDA(launch_kernel(gdn_tree_kernel<128>, dim3(grid), dim3(128), GdnStage<128>::smem_bytes(d.Dv), s, post, g, beta, sb, d.Hk, d.HV, d.Dv, state, state_slot_stride, core));
  else if (d.Dk == 64)
    LB_CUDA(launch_kernel(gdn_tree_kernel<64>, dim3(grid), dim3(128), GdnStage<64>::smem_bytes(d.Dv), s, post, g, beta, sb, d.Hk, d.HV, d.Dv, state, state_slot_stride, core));
  else {
    set_error("DeltaNet key dim must be 64 or 128");
    return LING_B200_ERR_UNSUPPORTED;
  }
  LB_LAUNCH("gdn_tree_kernel");
  return LING_B200_OK;
}

bool gdn_fused_supported(const ModelDims& d) {
  return d.Dk == d.Dv && (d.Dk == 64 || d.Dk == 128) && d.HV % d.Hk == 0 && (d.HV * d.Dv) % 128 == 0;
}

int gdn_fused_launch(const Planes& in, const StepBuffers& sb, const ModelDims& d, const __nv_bfloat16* convw, const float* conv_state,
                     size_t conv_slot_stride, const float* g, const float* beta, const float* state, size_t state_slot_stride,
                     const __nv_bfloat16* norm_w, const QuantOut& q, float* pre, float* post, float* core_out, int n_slots, int grid,
                     const PrefetchPlan& plan, unsigned long long* stamps, cudaStream_t s) {
  if (!gdn_fused_supported(d)) {
    set_error("fused DeltaNet kernel: key dim = value dim = 64 or 128 expected");
    return LING_B200_ERR_UNSUPPORTED;
  }
  if (d.Dk == 128)
    LB_CUDA(launch_kernel(gdn_fused_kernel<128>, dim3(grid), dim3(512), GdnFused<128>::smem_floats() * 4, s, in, sb, d, convw, conv_state,
                          conv_slot_stride, g, beta, state, state_slot_stride, norm_w, q, pre, post, core_out, n_slots, plan, stamps));
  else
    LB_CUDA(launch_kernel(gdn_fused_kernel<64>, dim3(grid), dim3(512), GdnFused<64>::smem_floats() * 4, s, in, sb, d, convw, conv_state,
                          conv_slot_stride, g, beta, state, state_slot_stride, norm_w, q, pre, post, core_out, n_slots, plan, stamps));
  LB_LAUNCH("gdn_fused_kernel");
  return LING_B200_OK;
}

int gated_norm_quant_launch(const float* core, const Planes& z, int z_col, const __nv_bfloat16* w, const QuantOut& q,
                            const int* n_rows, int rows_grid, int HV, int Dv, float eps, cudaStream_t s) {
  LB_CUDA(launch_kernel(gated_norm_quant_kernel, dim3(rows_grid, ceil_div(q.K_pad, 1024)), dim3(256), size_t(0), s, core, z, z_col, w, q, n_rows, HV * Dv, Dv, eps));
  LB_LAUNCH("gated_norm_quant_kernel");
  return LING_B200_OK;
}

int attn_prepare_launch(const Planes& qkv, const StepBuffers& sb, const ModelDims& d, int al, const __nv_bfloat16* q_norm,
                        const __nv_bfloat16* k_norm, __half* q, const KvPoolDev& kv, int rows_grid, cudaStream_t s) {
  LB_CUDA(launch_kernel(attn_prepare_kernel, dim3(dim3(rows_grid, d.Hq + 2 * d.Hkv)), dim3(d.D), size_t(d.D * sizeof(float)), s, qkv, sb, d, al, q_norm, k_norm, q, kv));
  LB_LAUNCH("attn_prepare_kernel");
  return LING_B200_OK;
}

template <int D, int G>
static int attention_launch_t(const __half* q, const StepBuffers& sb, const ModelDims& d, int al, const KvPoolDev& kv,
                              float* part_o, float* part_ml, int chunk_slots, int grid, cudaStream_t s) {
  constexpr size_t smem = attn_smem<D, G>();
  LB_CUDA(launch_kernel(attention_kernel<D, G>, dim3(grid), dim3(kAttnThreads), size_t(smem), s, q, sb, d, al, kv, part_o, part_ml, chunk_slots));
  LB_LAUNCH("attention_kernel");
  return LING_B200_OK;
}

// Opts the attention kernels into their dynamic shared memory (once per device, never inside a stream capture).
int kernels_init() {
  if (const int r = attention_tc_init()) return r;
  LB_CUDA(cudaFuncSetAttribute(gdn_tree_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(GdnStage<128>::smem_bytes(128))));
  LB_CUDA(cudaFuncSetAttribute(gdn_tree_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(GdnStage<64>::smem_bytes(128))));
  LB_CUDA(cudaFuncSetAttribute(gdn_commit_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(GdnStage<128>::smem_bytes(128, kCommitRows))));
  LB_CUDA(cudaFuncSetAttribute(gdn_commit_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(GdnStage<64>::smem_bytes(128, kCommitRows))));
  LB_CUDA(cudaFuncSetAttribute(gdn_fused_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(GdnFused<128>::smem_floats() * 4)));
  LB_CUDA(cudaFuncSetAttribute(gdn_fused_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(GdnFused<64>::smem_floats() * 4)));
  LB_CUDA(cudaFuncSetAttribute(attention_kernel<256, 6>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(attn_smem<256, 6>())));
  LB_CUDA(cudaFuncSetAttribute(attention_kernel<64, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(attn_smem<64, 4>())));
  LB_CUDA(cudaFuncSetAttribute(attention_kernel<128, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(attn_smem<128, 4>())));
  LB_CUDA(cudaFuncSetAttribute(attention_kernel<128, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(attn_smem<128, 8>())));
  return LING_B200_OK;
}

int attention_launch(const __half* q, const StepBuffers& sb, const ModelDims& d, int al, const KvPoolDev& kv, float* part_o,
                     float* part_ml, int chunk_slots, int grid, cudaStream_t s) {
  const int G = d.Hq / d.Hkv;
  if (d.D == 256 && G == 6) return attention_launch_t<256, 6>(q, sb, d, al, kv, part_o, part_ml, chunk_slots, grid, s);
  if (d.D == 64 && G == 4) return attention_launch_t<64, 4>(q, sb, d, al, kv, part_o, part_ml, chunk_slots, grid, s);
  if (d.D == 128 && G == 4) return attention_launch_t<128, 4>(q, sb, d, al, kv, part_o, part_ml, chunk_slots, grid, s);
  if (d.D == 128 && G == 8) return attention_launch_t<128, 8>(q, sb, d, al, kv, part_o, part_ml, chunk_slots, grid, s);
  set_error("attention: unsupported (head_dim, q heads per kv head); built: (256,6), (64,4), (128,4), (128,8)");
  return LING_B200_ERR_UNSUPPORTED;
}

int attn_combine_launch(const float* part_o, const float* part_ml, const Planes& qkv, const StepBuffers& sb,
                        const ModelDims& d, const QuantOut& q, float* raw, int rows_grid, int max_chunks, int tile_rows, int budget,
                        int chunk_slots, cudaStream_t s) {
  const int G = d.Hq / d.Hkv;
  const int CB = d.D > 128 ? d.D : 128, HB = CB / d.D, NG = 256 / (CB / 4);
  if (CB % 128 != 0 || 256 % (CB / 4) != 0 || CB % d.D != 0) {
    set_error("attention combine: head dim must be 64, 128 or 256");
    return LING_B200_ERR_UNSUPPORTED;
  }
  const dim3 grid(rows_grid, ceil_div(q.K_pad, CB));
  max_chunks = round_up(max_chunks, 4);  // keeps the float4 partial sums behind the weights 16-byte aligned
  const size_t smem = (size_t(HB) * max_chunks + 4 + size_t(NG) * CB) * sizeof(float);
  if (smem > 48 * 1024) {
    set_error("attention combine: too many chunks for one sequence");
    return LING_B200_ERR_UNSUPPORTED;
  }
  if (G == 6) LB_CUDA(launch_kernel(attn_combine_kernel<6>, grid, dim3(256), smem, s, part_o, part_ml, qkv, sb, d, q, raw, max_chunks, tile_rows, budget, chunk_slots));
  else if (G == 4) LB_CUDA(launch_kernel(attn_combine_kernel<4>, grid, dim3(256), smem, s, part_o, part_ml, qkv, sb, d, q, raw, max_chunks, tile_rows, budget, chunk_slots));
  else if (G == 8) LB_CUDA(launch_kernel(attn_combine_kernel<8>, grid, dim3(256), smem, s, part_o, part_ml, qkv, sb, d, q, raw, max_chunks, tile_rows, budget, chunk_slots));
  else {
    set_error("attention combine: unsupported group size");
    return LING_B200_ERR_UNSUPPORTED;
  }
  LB_LAUNCH("attn_combine_kernel");
  return LING_B200_OK;
}

int silu_mul_quant_launch(const Planes& gu, int I, int up_col0, const QuantOut& q, const int* n_rows, int rows_grid, cudaStream_t s) {
  LB_CUDA(launch_kernel(silu_mul_quant_kernel, dim3(rows_grid, ceil_div(q.K_pad, 1024)), dim3(256), size_t(0), s, gu, I, up_col0, q, n_rows));
  LB_LAUNCH("silu_mul_quant_kernel");
  return LING_B200_OK;
}

int argmax_reduce_launch(const float* tile_val, const int* tile_idx, int tiles, int rows_alloc, int* ids, float* vals,
                         const int* n_rows, int rows_grid, cudaStream_t s) {
  LB_CUDA(launch_kernel(argmax_reduce_kernel, dim3(rows_grid), dim3(256), size_t(0), s, tile_val, tile_idx, tiles, rows_alloc, ids, vals, n_rows));
  LB_LAUNCH("argmax_reduce_kernel");
  return LING_B200_OK;
}

int argmax_rows_launch(const float* logits, int rows, int vocab, int* ids, float* vals, cudaStream_t s) {
  LB_CUDA(launch_kernel(argmax_rows_kernel, dim3(rows), dim3(256), size_t(0), s, logits, vocab, ids, vals));
  LB_LAUNCH("argmax_rows_kernel");
  return LING_B200_OK;
}

int accept_launch(const StepBuffers& sb, const ModelDims& d, int, cudaStream_t s) {
  LB_CUDA(launch_kernel(accept_kernel, dim3(1), dim3(64), size_t(0), s, sb, d.V));
  LB_LAUNCH("accept_kernel");
  return LING_B200_OK;
}

int kv_compact_launch(const StepBuffers& sb, const ModelDims& d, const KvPoolDev& kv, cudaStream_t s) {
  if (d.n_attn == 0) return LING_B200_OK;
  LB_CUDA(launch_kernel(kv_compact_kernel, dim3(dim3(d.n_attn * 2 * d.Hkv, d.max_seqs)), dim3(64), size_t(0), s, sb, d, kv));
  LB_LAUNCH("kv_compact_kernel");
  return LING_B200_OK;
}

int conv_commit_launch(const StepBuffers& sb, const ModelDims& d, const float* pre, size_t layer_stride, float* conv_state,
                       size_t conv_slot_stride, size_t conv_layer_stride, cudaStream_t s) {
  if (d.n_gdn == 0) return LING_B200_OK;
  LB_CUDA(launch_kernel(conv_commit_kernel, dim3(dim3(ceil_div(d.C, 256), d.max_seqs, d.n_gdn)), dim3(256), size_t(0), s, sb, d.C, pre, layer_stride, conv_state, conv_slot_stride, conv_layer_stride));
  LB_LAUNCH("conv_commit_kernel");
  return LING_B200_OK;
}

int gdn_commit_launch(const StepBuffers& sb, const ModelDims& d, const float* post, const float* g, const float* beta,
                      size_t post_layer_stride, size_t g_layer_stride, float* state, size_t state_slot_stride,
                      size_t state_layer_stride, int grid, cudaStream_t s) {
  if (d.n_gdn == 0) return LING_B200_OK;
  if (d.Dk == 128)
    LB_CUDA(launch_kernel(gdn_commit_kernel<128>, dim3(grid), dim3(128), GdnStage<128>::smem_bytes(d.Dv, kCommitRows), s, post, g, beta, post_layer_stride, g_layer_stride, sb, d.Hk, d.HV, d.Dv, d.n_gdn, state, state_slot_stride, state_layer_stride));
  else if (d.Dk == 64)
    LB_CUDA(launch_kernel(gdn_commit_kernel<64>, dim3(grid), dim3(128), GdnStage<64>::smem_bytes(d.Dv, kCommitRows), s, post, g, beta, post_layer_stride, g_layer_stride, sb, d.Hk, d.HV, d.Dv, d.n_gdn, state, state_slot_stride, state_layer_stride));
  else {
    set_error("DeltaNet key dim must be 64 or 128");
    return LING_B200_ERR_UNSUPPORTED;
  }
  LB_LAUNCH("gdn_commit_kernel");
  return LING_B200_OK;
}

int quant_weight_launch(const float* src_f32, uint64_t key, float std_, int from_generator, uint8_t* codes, float* scales,
                        int row_off, int rows, int K, int N_pad, int K_pad, cudaStream_t s) {
  const int KB = K_pad / 128;
  LB_CUDA(launch_kernel(quant_weight_kernel, dim3(dim3(rows, std::min(ceil_div(KB, 8), 8))), dim3(256), size_t(0), s, src_f32, key, std_, from_generator, codes, scales, row_off, K, N_pad, K_pad));
  LB_LAUNCH("quant_weight_kernel");
  return LING_B200_OK;
}

int quant_acts_launch(const float* x, int rows, const QuantOut& q, cudaStream_t s) {
  LB_CUDA(launch_kernel(quant_acts_kernel, dim3(rows), dim3(256), size_t(0), s, x, q));
  LB_LAUNCH("quant_acts_kernel");
  return LING_B200_OK;
}

int fill_bf16_launch(const float* src_f32, uint64_t key, float std_, float bias, int from_generator, __nv_bfloat16* dst,
                     size_t n, cudaStream_t s) {
  const int grid = int(std::min<size_t>((n + 255) / 256, 148 * 16));
  LB_CUDA(launch_kernel(fill_bf16_kernel, dim3(std::max(grid, 1)), dim3(256), size_t(0), s, src_f32, key, std_, bias, from_generator, dst, n));
  LB_LAUNCH("fill_bf16_kernel");
  return LING_B200_OK;
}

int fill_f32_launch(uint64_t key, float std_, float* dst, size_t n, cudaStream_t s) {
  const int grid = int(std::min<size_t>((n + 255) / 256, 148 * 16));
  LB_CUDA(launch_kernel(fill_f32_kernel, dim3(std::max(grid, 1)), dim3(256), size_t(0), s, key, std_, dst, n));
  LB_LAUNCH("fill_f32_kernel");
  return LING_B200_OK;
}

int kv_write_launch(const float* k, const float* v, uint64_t key_k, uint64_t key_v, int from_generator, const ModelDims& d,
                    int al, int slot, int from, int n, const KvPoolDev& kv, int* err, cudaStream_t s) {
  if (n <= 0) return LING_B200_OK;
  LB_CUDA(launch_kernel(kv_write_kernel, dim3(dim3(n, d.Hkv, 2)), dim3(d.D), size_t(0), s, k, v, key_k, key_v, from_generator, d, al, slot, from, kv, err));
  LB_LAUNCH("kv_write_kernel");
  return LING_B200_OK;
}

int kv_page_copy_launch(const ModelDims& d, const KvPoolDev& kv, int src, int dst, cudaStream_t s) {
  if (d.n_attn == 0) return LING_B200_OK;
  LB_CUDA(launch_kernel(kv_page_copy_kernel, dim3(d.n_attn * 2 * d.Hkv), dim3(256), size_t(0), s, d, kv, src, dst));
  LB_LAUNCH("kv_page_copy_kernel");
  return LING_B200_OK;
}

int f32_to_half_launch(const float* src, __half* dst, size_t n, cudaStream_t s) {
  LB_CUDA(launch_kernel(f32_to_half_kernel, dim3(int(std::min<size_t>((n + 255) / 256, 148 * 8))), dim3(256), size_t(0), s, src, dst, n));
  return LING_B200_OK;
}

int flush_launch(float* buf, size_t n, cudaStream_t s) {
  LB_CUDA(launch_kernel(flush_kernel, dim3(148 * 8), dim3(256), size_t(0), s, buf, n));
  LB_LAUNCH("flush_kernel");
  return LING_B200_OK;
}

}  // namespace lb
