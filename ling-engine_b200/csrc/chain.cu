// chain.cu -- a layer segment as ONE persistent kernel: up to three block-scaled FP8 weight GEMMs (gemm.h) with the
// row-wise kernels that stand between them (residual add + RMSNorm + FP8 quantization, the DeltaNet gating projections,
// SiLU(gate) * up + quantization), for steps of at most 32 packed rows.
//
// The reference ships the same idea for its own GEMM (persistent per-layer kernels with counter dependencies,
// src/core/stream_gemm.cu:841-851,1074-1086,1459-1477 in the reference project); this is that idea rebuilt around the
// tcgen05 / TMEM / TMA GEMM of gemm.cu.  What it buys: between two GEMMs of a layer the step otherwise pays a kernel
// boundary (the dependent-launch hand-off, ~2.3 us each) and HBM idles while the small kernel between them runs.  Here the
// TMA producer warp of every CTA rolls straight from one matrix's weight tiles into the next one's -- weight tiles do not
// depend on anything the step computes -- and runs an L2 prefetch a fixed number of K blocks ahead of its loads, across
// matrix boundaries, so HBM keeps streaming weights while the epilogue warps do the row-wise work.
//
// Shape of the kernel: a grid of at most 2 CTAs per SM, all co-resident (the kernel waits on its own CTAs, never on
// another launch).  Per CTA, as in gemm.cu: warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner, warps 2-5 =
// epilogue (promotion of every 128-wide K block with the two block scales in fp32).  GEMM g's unit u = (weight tile, K
// split) belongs to CTA u.  The epilogue warps also carry out the row-wise units between the GEMMs:
//   norm unit (row m, 1024-column chunk j)  -> CTA m * chunks + j     waits: the GEMM before it, per chunk
//   gating unit (value head, row)           -> strided over the CTAs  waits: every norm unit
//   activation unit (128-column block j)    -> the CTA of up tile j   waits: gate tile j
// Dependencies travel through counters in global memory (zeroed by the host before the step): writers store, fence
// (gpu scope and the async proxy, since the readers are TMA loads) and add; readers poll with acquire loads.  Every poll
// is bounded by the wall clock; a role that gives up records a code in the device error word, raises the chain's abort
// word so that every other poller leaves too, drains its copies, frees TMEM, and the kernel returns.  Nothing traps.
//
// Arithmetic: every unit computes exactly what the stand-alone kernels compute (same K split per shape, same order of the
// partial sums, same reductions), so a step through this kernel is bit-identical to the step through the separate
// launches; the tests compare the two.
#include "chain.h"

#include <algorithm>

#include "../../include/ling_b200.h"
#include "tc.cuh"

namespace lb {
namespace {
using namespace tc;

constexpr int NT = kChainRows;            // token rows per MMA (the instruction's N)
constexpr int STAGES = 5;                 // as the 32-row tile of gemm.cu
constexpr int BUFS = 4, ACCW = NT, kTmemCols = 128;
constexpr int kScaleRing = 16, kScaleAhead = 12;
constexpr int kABytes = kTileN * kBlockK, kBBytes = NT * kBlockK, kStageBytes = kABytes + kBBytes;
constexpr int kThreads = 192, kEpi = 128;
constexpr size_t kSmemBytes = size_t(STAGES) * kStageBytes + 1024 + 512 + 2048 /* glue scratch */ + size_t(4) * kScaleRing * NT * 4;

// counters of one chain (unsigned words, zeroed by the host before the step)
// (the hot counters sit 32 words = one 128-byte line apart: adds to different counters do not queue behind each other)
constexpr int kLine = 32;
constexpr int kCtAbort = 0;                  // raised by a role that gave up
constexpr int kCtDone = 1 * kLine;           // [8 lines]: units of the GEMM before the norm that are complete, per 1024-column chunk
constexpr int kCtReady = 9 * kLine;          // [8 lines]: norm units complete, per chunk (= the next GEMM's K blocks 8j .. 8j+7 are quantized)
constexpr int kCtRow = 17 * kLine;           // [32 lines]: chunks of row m whose partial sums of squares are published
constexpr int kCtTile = 49 * kLine;          // [tiles]: gate tile t of the gate|up GEMM is stored
constexpr int kCtSplit = 49 * kLine + 512;   // [8 lines]: activation blocks quantized, per K split of the GEMM that reads them

__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Everything this thread wrote is visible to the GPU and to the async proxy (TMA reads) before the count that follows.
__device__ __forceinline__ void publish_fence() {
  __threadfence();
  asm volatile("fence.proxy.async;" ::: "memory");
}
__device__ __forceinline__ void signal_add(unsigned* p) { atomicAdd(p, 1u); }

__device__ __forceinline__ unsigned ld_relaxed(const unsigned* p) {
  unsigned v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Polls *p until it reaches `want` (one thread per CTA and dependency polls, with a pause between loads: hundreds of
// pollers on one line would otherwise queue in front of the adds they wait for).  false: the limit ran out or the chain was
// aborted.
__device__ __forceinline__ bool wait_count(const unsigned* p, unsigned want, const unsigned* abort_word) {
  if (ld_acquire(p) >= want) return true;
  const uint64_t t0 = global_ns();
  for (uint32_t spin = 1;; ++spin) {
    asm volatile("nanosleep.u32 100;" ::: "memory");
    if (ld_relaxed(p) >= want) {
      __threadfence();
      return true;
    }
    if ((spin & 63u) == 0) {
      if (ld_relaxed(abort_word) != 0) return false;
      if (global_ns() - t0 > kWaitLimitNs) return false;
    }
  }
}

struct Unit {
  int tile, split, kb0, kb1;
  bool have;
};
__device__ __forceinline__ Unit unit_of(const ChainGemm& g, int cta) {
  Unit u;
  u.have = cta < (g.N_pad / kTileN) * g.splits;
  u.tile = cta / g.splits, u.split = cta % g.splits;
  u.kb0 = int(int64_t(g.KB) * u.split / g.splits), u.kb1 = int(int64_t(g.KB) * (u.split + 1) / g.splits);
  if (!u.have) u.kb0 = u.kb1 = 0;
  return u;
}

__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kEpi) : "memory"); }
// block_sum of kernels.cu over the 128 epilogue threads: warp sums, then the four partials added by a shuffle tree.
__device__ __forceinline__ float epi_sum(float v, float* red, int et) {
  const int lane = et & 31, warp = et >> 5;
  v = warp_sum(v);
  epi_sync();
  if (lane == 0) red[warp] = v;
  epi_sync();
  const float t = lane < 4 ? red[lane] : 0.f;
  return warp_sum(t);
}

// acc[j] += v[j] * (wsc * s[j]) for four accumulator columns (gemm.cu promote4: packed fp32x2, scalar rounding).
__device__ __forceinline__ void promote4(float* acc, const uint32_t* v, float wsc, const float4& s4) {
  const float2 w2 = make_float2(wsc, wsc);
  const float2 c01 = __fmul2_rn(w2, make_float2(s4.x, s4.y)), c23 = __fmul2_rn(w2, make_float2(s4.z, s4.w));
  const float2 a01 = __ffma2_rn(make_float2(__uint_as_float(v[0]), __uint_as_float(v[1])), c01, make_float2(acc[0], acc[1]));
  const float2 a23 = __ffma2_rn(make_float2(__uint_as_float(v[2]), __uint_as_float(v[3])), c23, make_float2(acc[2], acc[3]));
  acc[0] = a01.x, acc[1] = a01.y, acc[2] = a23.x, acc[3] = a23.y;
}

// A GEMM output's partial planes added in plane order, read past L1 (the planes may have been written by other CTAs of
// this launch).  The sum is the one kernels.cu plane_sum4 forms.
__device__ __forceinline__ float4 plane_sum4_cg(const Planes& a, int m, int c) {
  float4 t[kMaxPlanes];
  const float* base = a.p + size_t(m) * a.ld + c;
#pragma unroll
  for (int p = 0; p < kMaxPlanes; ++p)
    t[p] = p < a.n ? __ldcg(reinterpret_cast<const float4*>(base + size_t(p) * a.stride)) : make_float4(0.f, 0.f, 0.f, 0.f);
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int p = 0; p < kMaxPlanes; ++p) v.x += t[p].x, v.y += t[p].y, v.z += t[p].z, v.w += t[p].w;
  return v;
}

// One warp owns one 128-column block of row m (kernels.cu quant_store4): scale = amax / 448 (1 for an all-zero block).
__device__ __forceinline__ void quant_store4(float4 x, int c, int m, const QuantOut& q, int lane) {
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

// ---- residual add + Gemma RMSNorm + FP8 copy of one (row, 1024-column chunk): norm_quant_kernel of kernels.cu with the
// cluster's shared-memory exchange replaced by partial sums in global memory and a per-row count.  The 128 threads take
// the chunk as two halves of 512 columns, so half hh, warp w holds what warp 4 hh + w of the stand-alone kernel holds, and
// the row's sum of squares is formed from the same eight partials per chunk in the same order.
__device__ void norm_unit(const ChainNorm& n, int m, int j, int chunks, unsigned* ct, float* ssq, int nr, int et, bool& ok,
                          unsigned long long* st) {
  const int lane = et & 31, warp = et >> 5;
  float4 v[2];
  uint2 wraw[2];
  int c[2];
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    c[hh] = j * 1024 + hh * 512 + et * 4;
    v[hh] = make_float4(0.f, 0.f, 0.f, 0.f);
    wraw[hh] = make_uint2(0u, 0u);
    if (c[hh] < n.H) wraw[hh] = *reinterpret_cast<const uint2*>(n.w + c[hh]);
  }
  if (m >= nr) return;
  if (n.ids) {
#pragma unroll
    for (int hh = 0; hh < 2; ++hh)
      if (c[hh] < n.H) {
        const __nv_bfloat16* e = n.embed + size_t(n.ids[m]) * n.H + c[hh];
        v[hh] = make_float4(__bfloat162float(e[0]), __bfloat162float(e[1]), __bfloat162float(e[2]), __bfloat162float(e[3]));
      }
  } else {
    float4 t[2];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh)
      if (c[hh] < n.H) {
        v[hh] = __ldcg(reinterpret_cast<const float4*>(n.h + size_t(m) * n.H + c[hh]));
        if (n.add.p) t[hh] = plane_sum4_cg(n.add, m, c[hh]);
      }
#pragma unroll
    for (int hh = 0; hh < 2; ++hh)
      if (c[hh] < n.H && n.add.p) v[hh].x += t[hh].x, v[hh].y += t[hh].y, v[hh].z += t[hh].z, v[hh].w += t[hh].w;
  }
  float* part = ssq + (size_t(m) * 8 + j) * 8;  // [row][chunk][8 partials]
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    if (c[hh] < n.H) *reinterpret_cast<float4*>(n.h + size_t(m) * n.H + c[hh]) = v[hh];
    const float sq = v[hh].x * v[hh].x + v[hh].y * v[hh].y + v[hh].z * v[hh].z + v[hh].w * v[hh].w;
    const float wsum = warp_sum(sq);
    if (lane == 0) part[hh * 4 + warp] = wsum;
  }
  __threadfence();
  epi_sync();
  if (et == 0) {
    signal_add(ct + kCtRow + m * kLine);
    ok = wait_count(ct + kCtRow + m * kLine, unsigned(chunks), ct + kCtAbort);
  }
  epi_sync();
  if (st) st[12] = global_ns();
  // every thread re-reads the verdict through shared memory in the caller; here only the partials matter
  float total = 0.f;
  for (int r = 0; r < chunks; ++r) {
    const float4 a = __ldcg(reinterpret_cast<const float4*>(ssq + (size_t(m) * 8 + r) * 8));
    const float4 b4 = __ldcg(reinterpret_cast<const float4*>(ssq + (size_t(m) * 8 + r) * 8 + 4));
    total += ((a.x + a.y) + (a.z + a.w)) + ((b4.x + b4.y) + (b4.z + b4.w));
  }
  const float rstd = rsqrtf(total / n.H + n.eps);
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c[hh] < n.H) {
      const __nv_bfloat162 w01 = *reinterpret_cast<const __nv_bfloat162*>(&wraw[hh].x), w23 = *reinterpret_cast<const __nv_bfloat162*>(&wraw[hh].y);
      x.x = v[hh].x * rstd * (1.f + __low2float(w01));
      x.y = v[hh].y * rstd * (1.f + __high2float(w01));
      x.z = v[hh].z * rstd * (1.f + __low2float(w23));
      x.w = v[hh].w * rstd * (1.f + __high2float(w23));
      if (n.xn) *reinterpret_cast<float4*>(n.xn + size_t(m) * n.H + c[hh]) = x;
    }
    if (c[hh] - lane * 4 < n.q.K_pad) quant_store4(x, c[hh], m, n.q, lane);
  }
}

// ---- the DeltaNet gating projections of one value head for four rows (rows m0 .. m0 + 3): ab_gating_kernel of kernels.cu
// on the 128 epilogue threads, each row's sums formed exactly as that kernel forms them (thread t takes columns 4t + 512k,
// then the block sum), the head's two weight rows read once for the four rows and the rows' loads in flight together.
constexpr int kAbRows = 4;
__device__ void ab_unit(const ChainAb& a, int hv, int m0, int nr, float* red, int et) {
  const __nv_bfloat16* wa = a.wa + size_t(hv) * a.H;
  const __nv_bfloat16* wb = a.wb + size_t(hv) * a.H;
  float sa[kAbRows], sb2[kAbRows];
#pragma unroll
  for (int r = 0; r < kAbRows; ++r) sa[r] = sb2[r] = 0.f;
#pragma unroll 5
  for (int c = et * 4; c < a.H; c += 512) {
    const uint2 ar = *reinterpret_cast<const uint2*>(wa + c), br = *reinterpret_cast<const uint2*>(wb + c);
    float4 xv[kAbRows];
#pragma unroll
    for (int r = 0; r < kAbRows; ++r)
      xv[r] = m0 + r < nr ? __ldcg(reinterpret_cast<const float4*>(a.xn + size_t(m0 + r) * a.H + c)) : make_float4(0.f, 0.f, 0.f, 0.f);
    const __nv_bfloat162 a01 = *reinterpret_cast<const __nv_bfloat162*>(&ar.x), a23 = *reinterpret_cast<const __nv_bfloat162*>(&ar.y);
    const __nv_bfloat162 b01 = *reinterpret_cast<const __nv_bfloat162*>(&br.x), b23 = *reinterpret_cast<const __nv_bfloat162*>(&br.y);
#pragma unroll
    for (int r = 0; r < kAbRows; ++r) {
      sa[r] += xv[r].x * __low2float(a01) + xv[r].y * __high2float(a01) + xv[r].z * __low2float(a23) + xv[r].w * __high2float(a23);
      sb2[r] += xv[r].x * __low2float(b01) + xv[r].y * __high2float(b01) + xv[r].z * __low2float(b23) + xv[r].w * __high2float(b23);
    }
  }
#pragma unroll
  for (int r = 0; r < kAbRows; ++r) {
    const float ta = epi_sum(sa[r], red, et), tb = epi_sum(sb2[r], red, et);
    if (et == 0 && m0 + r < nr) {
      const float xx = ta + __bfloat162float(a.dt_bias[hv]);
      const float sp = xx <= 20.f ? log1pf(__expf(xx)) : xx;
      a.g[size_t(m0 + r) * a.HV + hv] = -__expf(__bfloat162float(a.A_log[hv])) * sp;
      a.beta[size_t(m0 + r) * a.HV + hv] = 1.f / (1.f + __expf(-tb));
    }
  }
}

__global__ void __launch_bounds__(kThreads, 2) gemm_chain_kernel(const __grid_constant__ ChainProgram P) {
  pdl_trigger();
  // Optional stamps (debugging aid, %globaltimer ns; minima in words that start at ~0, maxima in words that start at 0):
  // [0] first CTA's start, [1] CTA 0's epilogue past the dependency wait; over all CTAs, the first K loop to begin (inputs
  // ready) and the last to end, of GEMM 0 [4] / [6], GEMM 1 [5] / [7], GEMM 2 [8] / [14]; [11] last CTA's end; CTA 0's norm
  // unit: [9] begins, [12] row sums exchanged, [13] published.
  if (P.stamps && threadIdx.x == 0) atomicMin(P.stamps, global_ns());
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* tiles = smem;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * kStageBytes);
  uint64_t* empty = full + STAGES;
  uint64_t* tmem_full = empty + STAGES;
  uint64_t* tmem_empty = tmem_full + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* x_ready = reinterpret_cast<volatile int*>(tmem_slot + 4);  // [kChainGemms]: the epilogue found GEMM g's inputs complete
  float* scratch = reinterpret_cast<float*>(smem + STAGES * kStageBytes + 512);                 // [512] floats of glue scratch
  float* xs_ring = reinterpret_cast<float*>(smem + STAGES * kStageBytes + 512 + 2048);          // [4 warps][kScaleRing][NT]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x;
  unsigned* ct = P.counters;

  if (threadIdx.x == 0) {
    for (int g = 0; g < P.n_gemm; ++g) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&P.g[g].mapW)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&P.g[g].mapX)) : "memory");
    }
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < BUFS; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 4);
    }
    *abort_flag = 0;
    for (int g = 0; g < kChainGemms; ++g) x_ready[g] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Whose X is whose: GEMM P.norm_gemm reads the norm's output, GEMM P.norm_gemm + 1 (with P.has_silu) the activation's,
  // every other GEMM an input the kernel before this one left.
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const uint64_t pol_w = policy_evict_first(), pol_x = policy_evict_last();
      bool waited = false, ok = true;
      int base = 0;        // K blocks of earlier GEMMs of this CTA: stage and parity run on across GEMMs
      // This CTA's unit of every GEMM, worked out once (the K split's bounds take 64-bit divisions).
      Unit units[kChainGemms];
#pragma unroll
      for (int g = 0; g < kChainGemms; ++g) units[g] = g < P.n_gemm ? unit_of(P.g[g], cta) : Unit{0, 0, 0, 0, false};
      // The L2 prefetch cursor walks this CTA's K blocks of every GEMM in order and stays P.l2_ahead blocks in front of the
      // loads, across GEMM boundaries: `loaded` and `passed` count blocks from the start of the chain.
      int pf_g = 0, pf_i = 0, loaded = 0, passed = 0;
      auto prefetch_ahead = [&] {
        while (passed < loaded + P.l2_ahead && pf_g < P.n_gemm) {
          const Unit& pu = units[pf_g];
          if (pf_i >= pu.kb1 - pu.kb0) {
            ++pf_g, pf_i = 0;
            continue;
          }
          if (passed >= loaded) tma_prefetch_l2_2d(&P.g[pf_g].mapW, (pu.kb0 + pf_i) * kBlockK, pu.tile * kTileN);
          ++pf_i, ++passed;
        }
      };
      for (int g = 0; g < P.n_gemm && ok; ++g) {
        const ChainGemm& G = P.g[g];
        const Unit u = units[g];
        const int n = u.kb1 - u.kb0;
        const int wy = u.tile * kTileN;
        const bool from_norm = g == P.norm_gemm, from_silu = P.has_silu && g == P.norm_gemm + 1;
        int w_cur = 0, x_cur = 0, ready_upto = (from_norm || from_silu) ? 0 : n;  // X blocks [0, ready_upto) are known to be quantized
        uint64_t t0 = 0;
        uint32_t idle = 0;
        while (x_cur < n) {
          // Activation tiles of stages whose weight tile is already on its way go out as soon as the inputs are known to be
          // ready; weight tiles go out whenever a stage is free (they depend on nothing).  Both tests are non-blocking: a
          // blocking wait for a free stage would hold back an activation tile that the MMA warp is waiting for.
          bool progressed = false;
          if (x_cur < w_cur) {
            if (!waited) {  // inputs of the kernel before this one: its completion, once
              pdl_wait();
              waited = true;
            }
            if (x_cur >= ready_upto && x_ready[g]) {
              // this CTA's epilogue has seen every K block of the unit quantized (its acquire, a fence, then the flag)
              __threadfence();
              asm volatile("fence.proxy.async;" ::: "memory");
              ready_upto = n;
            }
            while (x_cur < w_cur && x_cur < ready_upto) {
              const int s = (base + x_cur) % STAGES;
              tma_load_2d(tiles + s * kStageBytes + kABytes, &G.mapX, &full[s], (u.kb0 + x_cur) * kBlockK, 0, pol_x);
              ++x_cur, progressed = true;
            }
          }
          if (w_cur < n) {
            const int bb = base + w_cur, s = bb % STAGES;
            // With nothing else to send, the wait for a free stage may suspend the thread (try_wait): a producer that spins
            // instead takes issue slots from the epilogue warp on its scheduler, and the promotion is what bounds a K block.
            const uint32_t par = ((bb / STAGES) & 1) ^ 1;
            if (x_cur == w_cur ? mbar_try_wait(&empty[s], par) : mbar_test_wait(&empty[s], par)) {
              mbar_expect_tx(&full[s], kStageBytes);
              tma_load_2d(tiles + s * kStageBytes, &G.mapW, &full[s], (u.kb0 + w_cur) * kBlockK, wy, pol_w);
              ++w_cur, ++loaded, progressed = true;
              if (P.l2_ahead > 0) prefetch_ahead();
            }
          }
          if (progressed) {
            idle = 0;
            continue;
          }
          if (x_cur < w_cur && x_cur >= ready_upto) asm volatile("nanosleep.u32 64;" ::: "memory");  // the row-wise units are at work
          if ((++idle & 1023u) == 0) {
            if (t0 == 0) t0 = global_ns();
            if (*abort_flag || ld_relaxed(ct + kCtAbort) != 0 || global_ns() - t0 > kWaitLimitNs) {
              dev_fail(P.err_flag, kDevWaitEmpty);
              *abort_flag = 1;
              atomicExch(ct + kCtAbort, 1u);
              ok = false;
            }
          }
          if (!ok) break;
        }
        if (!ok) {
          // Giving up: stages that hold only their weight half get their activation half now (the buffers exist whether or
          // not their content is final; nobody will consume these stages), so that every copy in flight completes and can be
          // waited for before the CTA's shared memory goes away.
          if (!waited) pdl_wait(), waited = true;
          for (; x_cur < w_cur; ++x_cur)
            tma_load_2d(tiles + ((base + x_cur) % STAGES) * kStageBytes + kABytes, &G.mapX, &full[(base + x_cur) % STAGES],
                        (u.kb0 + x_cur) * kBlockK, 0, pol_x);
          base += w_cur;
          break;
        }
        base += n;
      }
      if (!waited) pdl_wait();
      // every copy this lane issued has landed before it leaves (bounded like every other wait)
      for (int j = max(base - STAGES, 0); j < base; ++j) mbar_wait(&full[j % STAGES], (j / STAGES) & 1, nullptr);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (shared memory and TMEM only)
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_e4m3(NT);
      int b = 0;
      bool ok = true;
      for (int g = 0; g < P.n_gemm && ok; ++g) {
        const Unit u = unit_of(P.g[g], cta);
        for (int i = u.kb0; i < u.kb1; ++i, ++b) {
          const int s = b % STAGES, buf = b % BUFS;
          if (!mbar_wait(&tmem_empty[buf], ((b / BUFS) & 1) ^ 1, abort_flag)) {
            dev_fail(P.err_flag, kDevWaitTmemEmpty);
            ok = false;
            break;
          }
          if (!mbar_wait(&full[s], (b / STAGES) & 1, abort_flag)) {
            dev_fail(P.err_flag, kDevWaitFull);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t adesc = umma_desc_sw128(smem_u32(tiles + s * kStageBytes));
          const uint64_t bdesc = umma_desc_sw128(smem_u32(tiles + s * kStageBytes + kABytes));
          const uint32_t d = tmem_base + uint32_t(buf * ACCW);
#pragma unroll
          for (int k = 0; k < kBlockK / 32; ++k) umma_f8(d, adesc + uint64_t(k * 2), bdesc + uint64_t(k * 2), idesc, k > 0 ? 1u : 0u);
          umma_commit(&empty[s]);
          umma_commit(&tmem_full[buf]);
        }
      }
      if (!ok) {
        *abort_flag = 1;
        atomicExch(ct + kCtAbort, 1u);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps: K-block promotion and the row-wise units
    const int et = threadIdx.x - 64;      // 0 .. 127
    const int quarter = warp & 3;         // the TMEM lane quarter this warp may read
    const int row = quarter * 32 + lane;  // weight row inside the tile
    float* red = scratch;                 // [32] block sums; [64 ..] amax exchange
    volatile int* verdict = reinterpret_cast<volatile int*>(scratch + 48);
    pdl_wait();
    const bool stamp = P.stamps != nullptr && cta == 0 && et == 0;
    if (stamp) P.stamps[1] = global_ns();
    const int nr = *P.n_rows;
    bool ok = true;
    int b = 0;
    auto all_ok = [&](bool mine) {  // the group's common verdict (a poll is made by one thread)
      epi_sync();
      if (et == 0) *verdict = 1;
      epi_sync();
      if (!mine) *verdict = 0;
      epi_sync();
      return *verdict != 0;
    };
    for (int g = 0; g < P.n_gemm && ok; ++g) {
      const ChainGemm& G = P.g[g];
      if (g == P.norm_gemm) {
        // ---- the norm between GEMM g - 1 (or the kernel before) and GEMM g
        const int chunks = (P.norm.q.K_pad + 1023) / 1024;
        const int units = P.rows_grid * chunks;
        for (int uidx = cta; uidx < units && ok; uidx += gridDim.x) {
          const int m = uidx / chunks, j = uidx % chunks;
          bool mine = true;
          if (g > 0 && et == 0) {
            // the GEMM before: every (tile, split) unit whose columns fall into this chunk
            const ChainGemm& G0 = P.g[g - 1];
            const int tiles_in_chunk = min(8, G0.N_pad / kTileN - j * 8);
            mine = wait_count(ct + kCtDone + j * kLine, unsigned(tiles_in_chunk * G0.splits), ct + kCtAbort);
          }
          if (g > 0) ok = all_ok(mine);
          if (!ok) break;
          bool sums = true;
          if (stamp) P.stamps[9] = global_ns();
          norm_unit(P.norm, m, j, chunks, ct, P.ssq, nr, et, sums, stamp ? P.stamps : nullptr);
          ok = all_ok(sums);
          publish_fence();
          epi_sync();
          if (et == 0) signal_add(ct + kCtReady + j * kLine);
          if (stamp) P.stamps[13] = global_ns();
        }
        if (ok && P.has_ab) {
          // ---- the gating projections read whole normalized rows: every chunk of the norm must be complete
          bool mine = true;
          if (et < chunks) mine = wait_count(ct + kCtReady + et * kLine, unsigned(P.rows_grid), ct + kCtAbort);  // one poller per chunk
          ok = all_ok(mine);
          const int groups = (nr + kAbRows - 1) / kAbRows;  // only row groups that hold a real row
          for (int uidx = cta; uidx < P.ab.HV * groups && ok; uidx += gridDim.x)
            ab_unit(P.ab, uidx % P.ab.HV, (uidx / P.ab.HV) * kAbRows, nr, red, et);
        }
        if (!ok) break;
      }
      const Unit u = unit_of(G, cta);
      const int nslab = u.kb1 - u.kb0;
      if (nslab > 0) {
        const bool from_norm = g == P.norm_gemm, from_silu = P.has_silu && g == P.norm_gemm + 1;
        if (from_norm || from_silu) {
          // the activation scales of this unit's K range must be in place before the scale ring starts fetching them
          bool mine = true;
          if (from_norm) {  // the norm's chunks that cover this unit's K range, one poller each
            const int j0 = u.kb0 / 8, j1 = (u.kb1 - 1) / 8;
            if (et <= j1 - j0) mine = wait_count(ct + kCtReady + (j0 + et) * kLine, unsigned(P.rows_grid), ct + kCtAbort);
          } else if (et == 0) {  // the activation blocks of this unit's K split
            mine = wait_count(ct + kCtSplit + u.split * kLine, unsigned(nslab), ct + kCtAbort);
          }
          ok = all_ok(mine);
          if (!ok) break;
          if (et == 0) {
            __threadfence();
            x_ready[g] = 1;  // tells this CTA's producer: the activation tiles of the unit may be loaded
          }
        }
        const int n = u.tile * kTileN + row;
        float acc[NT];
#pragma unroll
        for (int j = 0; j < NT; ++j) acc[j] = 0.f;
        for (int j = et; j < nslab * 4; j += kEpi)
          asm volatile("prefetch.global.L2 [%0];" ::"l"(G.ws + size_t(u.kb0 + (j >> 2)) * G.N_pad + u.tile * kTileN + (j & 3) * 32));
        float* ring = xs_ring + (warp - 2) * kScaleRing * NT;
        auto fetch_xs = [&](int i) {
          if (i < nslab && lane < NT / 4) ldgsts16(ring + (i % kScaleRing) * NT + lane * 4, G.xs + size_t(u.kb0 + i) * G.xrows + lane * 4);
          ldgsts_commit();
        };
        float wq[kScaleAhead];
        unsigned long long t_loop = 0;
        if (P.stamps && et == 0) {
          t_loop = global_ns();
          atomicMin(P.stamps + (g == 0 ? 4 : g == 1 ? 5 : 8), t_loop);
          if (g == 1) atomicMax(P.stamps + 2, t_loop);
        }
#pragma unroll
        for (int j = 0; j < kScaleAhead; ++j) {
          wq[j] = j < nslab ? __ldg(G.ws + size_t(u.kb0 + j) * G.N_pad + n) : 0.f;
          fetch_xs(j);
        }
        for (int i = 0; i < nslab && ok; ++i, ++b) {
          const int buf = b % BUFS;
          const float wsc = wq[0];
#pragma unroll
          for (int j = 0; j + 1 < kScaleAhead; ++j) wq[j] = wq[j + 1];
          wq[kScaleAhead - 1] = i + kScaleAhead < nslab ? __ldg(G.ws + size_t(u.kb0 + i + kScaleAhead) * G.N_pad + n) : 0.f;
          fetch_xs(i + kScaleAhead);
          ldgsts_wait<kScaleAhead>();
          __syncwarp();
          const float4* xs4 = reinterpret_cast<const float4*>(ring + (i % kScaleRing) * NT);
          ok = mbar_wait(&tmem_full[buf], (b / BUFS) & 1, abort_flag);
          if (!ok) {
            dev_fail(P.err_flag, kDevWaitTmemFull);
            *abort_flag = 1;
            atomicExch(ct + kCtAbort, 1u);
            break;
          }
          tc_fence_after();
          if (P.stamps && et == 0 && g == 1 && i == 0) atomicMax(P.stamps + 10, global_ns() - t_loop);
          const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(buf * ACCW);
          uint32_t v[NT];
          tmem_ld32(taddr, v);
          tmem_ld_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tmem_empty[buf]);
#pragma unroll
          for (int q = 0; q < NT / 4; ++q) promote4(acc + q * 4, v + q * 4, wsc, xs4[q]);
        }
        ldgsts_wait<0>();
        if (P.stamps && et == 0) {
          const unsigned long long t_end = global_ns();
          atomicMax(P.stamps + (g == 0 ? 6 : g == 1 ? 7 : 14), t_end);
          if (g == 1) atomicMax(P.stamps + 3, t_end - t_loop);
        }
        ok = all_ok(ok);
        if (!ok) break;
        if (n < G.N) {
          float* o = G.out + size_t(u.split) * G.split_stride + n;
#pragma unroll
          for (int j = 0; j < NT; ++j)
            if (j < P.rows_grid) o[size_t(j) * G.N_pad] = acc[j];
        }
        __threadfence();
        epi_sync();
        if (g + 1 == P.norm_gemm && et == 0) signal_add(ct + kCtDone + (u.tile / 8) * kLine);  // the norm behind this GEMM counts units per chunk
        if (P.has_silu && g == P.norm_gemm) {
          // ---- SiLU(gate) * up and its FP8 copy (silu_mul_quant_kernel of kernels.cu): the CTA of up tile j pairs its
          // accumulators (thread = intermediate column j * 128 + row) with gate tile j's stored values.
          const ChainSilu& S = P.silu;
          const int gate_tiles = S.up_col0 / kTileN;
          if (u.tile < gate_tiles) {
            if (et == 0) atomicExch(ct + kCtTile + u.tile, 1u);  // the stores above are fenced: gate tile u.tile is in memory
          } else {
            const int j = u.tile - gate_tiles, col = j * kTileN + row;
            bool mine = true;
            if (et == 0) mine = wait_count(ct + kCtTile + j, 1u, ct + kCtAbort);
            ok = all_ok(mine);
            if (!ok) break;
            const float* gp = G.out + col;  // one plane: the gate|up GEMM of a chain never splits K
            float gv[NT];
#pragma unroll
            for (int m = 0; m < NT; ++m) gv[m] = m < P.rows_grid ? __ldcg(gp + size_t(m) * G.N_pad) : 0.f;
            float* amax_sm = scratch + 64;  // [4 warps][NT]
#pragma unroll
            for (int m = 0; m < NT; ++m) {
              acc[m] = col < S.I ? silu(gv[m]) * acc[m] : 0.f;
              const float a = warp_max(fabsf(acc[m]));
              if (lane == 0) amax_sm[quarter * NT + m] = a;
            }
            epi_sync();
#pragma unroll
            for (int m = 0; m < NT; ++m) {
              const float amax = fmaxf(fmaxf(amax_sm[m], amax_sm[NT + m]), fmaxf(amax_sm[2 * NT + m], amax_sm[3 * NT + m]));
              const float sc = amax > 0.f ? amax / 448.f : 1.f;
              if (m < nr && m < P.rows_grid && col < S.q.K_pad) {
                S.q.codes[size_t(m) * S.q.K_pad + col] = to_e4m3(__fdiv_rn(acc[m], sc));
                if (row == 0) S.q.scales[size_t(j) * S.q.rows_alloc + m] = sc;
              }
            }
            publish_fence();
            epi_sync();
            if (et == 0) {  // block j counts for the K split of the next GEMM whose range holds it
              const ChainGemm& Gn = P.g[g + 1];
              int sp = 0;
              while (sp + 1 < Gn.splits && int(int64_t(Gn.KB) * (sp + 1) / Gn.splits) <= j) ++sp;
              signal_add(ct + kCtSplit + sp * kLine);
            }
          }
        }
      }
    }
    if (!ok) {
      *abort_flag = 1;
      atomicExch(ct + kCtAbort, 1u);
      dev_fail(P.err_flag, kDevWaitTmemFull);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (P.stamps && threadIdx.x == 0) atomicMax(P.stamps + 11, global_ns());
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

}  // namespace

int chain_init() {
  LB_CUDA(cudaFuncSetAttribute(gemm_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSmemBytes)));
  return LING_B200_OK;
}

int chain_grid(int sm_count) { return 2 * sm_count; }

// Whether the chain kernel covers a program: one unit per CTA and GEMM, whole 1024-column norm chunks within the counters,
// a gate|up GEMM that does not split K with the up half on a tile boundary.
bool chain_supported(const ChainProgram& P, int sm_count) {
  if (P.n_gemm < 1 || P.n_gemm > kChainGemms || P.rows_grid < 1 || P.rows_grid > kChainRows) return false;
  const int grid = chain_grid(sm_count);
  for (int g = 0; g < P.n_gemm; ++g)
    if ((P.g[g].N_pad / kTileN) * P.g[g].splits > grid || P.g[g].splits > 8) return false;
  if (P.norm_gemm >= P.n_gemm || (P.norm_gemm >= 0 && P.norm.q.K_pad > 8192)) return false;  // norm_gemm < 0: GEMMs only
  if (P.norm_gemm > 0 && P.g[P.norm_gemm - 1].N_pad > 8192) return false;
  if (P.has_silu) {
    if (P.norm_gemm + 1 >= P.n_gemm) return false;
    const ChainGemm& gu = P.g[P.norm_gemm];
    if (gu.splits != 1 || P.silu.up_col0 % kTileN != 0 || P.silu.I % kTileN != 0 || gu.N_pad != 2 * P.silu.up_col0 ||
        P.silu.up_col0 / kTileN > 512)
      return false;
  }
  return true;
}

int chain_launch(const ChainProgram& P, int sm_count, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(chain_grid(sm_count));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  LB_CUDA(cudaLaunchKernelEx(&cfg, gemm_chain_kernel, P));
  LB_LAUNCH("gemm_chain_kernel");
  return LING_B200_OK;
}

}  // namespace lb
