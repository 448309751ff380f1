// gemm.cu -- the block-scaled FP8 weight GEMM (see gemm.h) for sm_100a.
//
// Kernel shape (one CTA = one 128-row weight tile x one K split x one token tile):
//   warp 0   TMA producer: per 128-wide K block, one 128x128B weight tile and one NTx128B activation tile into a
//            128B-swizzled stage, completion counted on the stage's mbarrier (no multicast, no cluster).
//   warp 1   MMA issuer (one elected lane): four tcgen05.mma kind::f8f6f4 (K = 32 each) per stage into one of the TMEM
//            accumulator buffers (four; two for the 96-row token tile), then tcgen05.commit to the stage's "empty" barrier and the buffer's "full" barrier.
//            Also owns the TMEM allocation.
//   warps 2-5 epilogue: tcgen05.ld of the finished buffer, acc += partial * (weight scale * activation scale) in
//            registers (the 1x128 fp32 block scales are not a native tcgen05 scale format, so each K block is
//            promoted in fp32), release of the buffer; at the end the store (and, for the LM head, the per-tile argmax).
// Every wait is bounded by a wall-clock limit; a wait that runs out records a code in the device error word, the
// CTA drains its outstanding copies, frees its TMEM and returns.
#include "gemm.h"

#include <cfloat>
#include <mutex>
#include <utility>

#include "../../include/ling_b200.h"
#include "tc.cuh"

namespace lb {

namespace {
using namespace tc;

constexpr int kABytes = kTileN * kBlockK;  // 16 KiB
// TMEM accumulator buffers per CTA: the MMA of K block i + bufs may start as soon as the epilogue has drained block i,
// so the epilogue's latency per block is spread over `bufs` blocks.  Columns are allocated in powers of two; two CTAs
// share an SM's 512 columns for the narrow token tiles.
__host__ __device__ constexpr int acc_bufs(int nt) { return nt == 96 ? 2 : 4; }
__host__ __device__ constexpr int tmem_cols(int nt) { return nt == 32 ? 128 : nt == 128 ? 512 : 256; }
// K blocks by which the epilogue's scale loads run ahead of its accumulator reads, and the slots of each epilogue warp's
// activation-scale ring (> the lookahead).  With HBM saturated by the weight stream a scale takes microseconds to arrive
// (a K block lasts ~0.7 us): four blocks of lookahead left the epilogue waiting for scales (GEMM chain of the 27B step 5.20
// ms, 4.99 with seven, the most the eight-slot ring allows; the narrow tile has the shared memory for sixteen slots).
__host__ __device__ constexpr int scale_ring(int nt) { return nt == 32 ? 16 : 8; }
__host__ __device__ constexpr int scale_ahead(int nt) { return nt == 32 ? 12 : 7; }
__host__ __device__ constexpr int stages_for(int nt) { return nt == 32 ? 5 : nt == 64 ? 4 : nt == 96 ? 3 : 6; }
__host__ __device__ constexpr int ctas_per_sm(int nt) { return nt == 128 ? 1 : 2; }
// Epilogue warps: a warp reads the TMEM lane quarter warp % 4; the two widest token tiles have two warps per quarter, each
// promoting half of the accumulator's columns -- at 128 rows the per-block promotion (TMEM read + one FMA per element)
// takes as long as the block's MMAs, and the halves run on different schedulers.
__host__ __device__ constexpr int epi_warps(int nt) { return nt >= 96 ? 8 : 4; }
__host__ __device__ constexpr int gemm_threads(int nt) { return 64 + 32 * epi_warps(nt); }

// acc[j] += v[j] * (wsc * s[j]) for four accumulator columns, as two packed fp32x2 multiplies and two packed FMAs (each
// lane rounds like the scalar instructions, so the result is the scalar one; the promotion is instruction-bound)
__device__ __forceinline__ void promote4(float* acc, const uint32_t* v, float wsc, const float4& s4) {
  const float2 w2 = make_float2(wsc, wsc);
  const float2 c01 = __fmul2_rn(w2, make_float2(s4.x, s4.y)), c23 = __fmul2_rn(w2, make_float2(s4.z, s4.w));
  const float2 a01 = __ffma2_rn(make_float2(__uint_as_float(v[0]), __uint_as_float(v[1])), c01, make_float2(acc[0], acc[1]));
  const float2 a23 = __ffma2_rn(make_float2(__uint_as_float(v[2]), __uint_as_float(v[3])), c23, make_float2(acc[2], acc[3]));
  acc[0] = a01.x, acc[1] = a01.y, acc[2] = a23.x, acc[3] = a23.y;
}

struct HeadArgs {
  float* tile_val;
  int* tile_idx;
  int rows_alloc;
  int store_logits;
};
// The gate|up projection's activation fused into the GEMM (GemmCall::swiglu): see the kernel's epilogue.
constexpr int kFusePlanes = 8;  // most K splits (choose_splits): the planes are added in plane order, absent ones as zero, as every consumer does
struct SwigluArgs {
  unsigned* tickets;   // nullptr: off
  int I, up_col0;      // gate columns [0, I), up columns [up_col0, up_col0 + I); up_col0 a multiple of the weight tile
  uint8_t* codes;      // E4M3 [rows_alloc][K_pad]
  float* scales;       // [K_pad / 128][rows_alloc]
  int K_pad, rows_alloc;
};
constexpr size_t gemm_smem_bytes(int nt) {
  return size_t(stages_for(nt)) * (kABytes + nt * kBlockK) + 1024 /* alignment slack */ + 512 /* barriers */ +
         size_t(4) * nt * 8 /* head argmax scratch */ + size_t(4) * scale_ring(nt) * nt * 4 /* activation-scale rings */;
}

template <int NT>
__global__ void __launch_bounds__(gemm_threads(NT), ctas_per_sm(NT))
    gemm_fp8_tcgen05_kernel(const __grid_constant__ CUtensorMap mapW, const __grid_constant__ CUtensorMap mapX,
                            const float* __restrict__ ws, const float* __restrict__ xs, float* __restrict__ out, int ld,
                            size_t split_stride, int M, int N, int N_pad, int KB, int splits, int xrows, HeadArgs head,
                            int* err_flag, int pdl, int l2_slabs, unsigned long long* timeline, SwigluArgs sw) {
  pdl_trigger();  // the next kernel may be scheduled as soon as every CTA of this one has started
  // Optional timeline (debugging aid, like the reference's per-block %globaltimer stamps, src/core/engine.hpp:637-642):
  // [0] first CTA's start, [1] first producer past the dependency wait, [2] last producer past it, [3] last CTA's end.
  if (timeline && threadIdx.x == 0) atomicMin(timeline, global_ns());
  constexpr int STAGES = stages_for(NT);
  constexpr int kScaleRing = scale_ring(NT), kScaleAhead = scale_ahead(NT);
  constexpr int kBBytes = NT * kBlockK;
  constexpr int kWBytes = kABytes;  // weight bytes per stage, then the activation tile
  constexpr int kStageBytes = kWBytes + kBBytes;
  constexpr int kTmemCols = tmem_cols(NT);
  constexpr int ACCW = NT;  // TMEM columns per accumulator buffer

  extern __shared__ uint8_t smem_raw[];
  // 128B-swizzled tiles need 1024-byte alignment; the dynamic segment's base is not guaranteed to have it.
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* tiles = smem;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * kStageBytes);
  uint64_t* empty = full + STAGES;
  uint64_t* tmem_full = empty + STAGES;
  constexpr int BUFS = acc_bufs(NT);
  uint64_t* tmem_empty = tmem_full + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* red_val = reinterpret_cast<float*>(tmem_slot + 4);  // [4][NT]
  int* red_idx = reinterpret_cast<int*>(red_val + 4 * NT);   // [4][NT]
  float* xs_ring = reinterpret_cast<float*>(smem + STAGES * kStageBytes + 512 + 4 * NT * 8);  // [4 warps][kScaleRing][NT]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // token tiles vary fastest: the CTAs that share a weight tile run together, so only the first of them reads it from HBM
  const int tile_n = blockIdx.z, split = blockIdx.y, tile_m = blockIdx.x;
  const int kb0 = int(int64_t(KB) * split / splits), kb1 = int(int64_t(KB) * (split + 1) / splits);
  const int nslab = kb1 - kb0;

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&mapW)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&mapX)) : "memory");
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < BUFS; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], epi_warps(NT));
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {  // TMEM allocation: one warp, the whole warp executes it
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const uint64_t pol_w = policy_evict_first();  // weights are read once per step
      const uint64_t pol_x = policy_evict_last();   // the activation tile is re-read by every CTA
      const int wy = tile_n * kTileN, xy = tile_m * NT;
      int i = 0;
      bool ok = true;
      if (!pdl) {
        pdl_wait();
        if (timeline) {
          const unsigned long long t = global_ns();
          atomicMin(timeline + 1, t), atomicMax(timeline + 2, t);
        }
      }
      if (pdl) {
        // Weights do not depend on the previous kernel: fill the pipeline with weight tiles and ask for the next
        // l2_slabs tiles to be brought into L2, then wait for the previous kernel and fetch the activation tiles of the
        // filled stages.  While the kernels between two GEMMs run, HBM keeps streaming the next GEMM's weights.
        const int pre = min(min(nslab, STAGES), pdl - 1);
        for (int s = 0; s < pre; ++s) {
          mbar_expect_tx(&full[s], kStageBytes);
          tma_load_2d(tiles + s * kStageBytes, &mapW, &full[s], (kb0 + s) * kBlockK, wy, pol_w);
        }
        const int l2_end = nslab < pre + l2_slabs ? nslab : pre + l2_slabs;
        for (int s = pre; s < l2_end; ++s) tma_prefetch_l2_2d(&mapW, (kb0 + s) * kBlockK, wy);
        pdl_wait();
        if (timeline) {
          const unsigned long long t = global_ns();
          atomicMin(timeline + 1, t), atomicMax(timeline + 2, t);
        }
        for (int s = 0; s < pre; ++s)
          tma_load_2d(tiles + s * kStageBytes + kWBytes, &mapX, &full[s], (kb0 + s) * kBlockK, xy, pol_x);
        i = pre;
      }
      for (; i < nslab && ok; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (i / STAGES) & 1;
        ok = mbar_wait(&empty[s], ph ^ 1, abort_flag);
        if (!ok) {
          dev_fail(err_flag, kDevWaitEmpty);
          *abort_flag = 1;
          break;
        }
        mbar_expect_tx(&full[s], kStageBytes);
        tma_load_2d(tiles + s * kStageBytes, &mapW, &full[s], (kb0 + i) * kBlockK, wy, pol_w);
        tma_load_2d(tiles + s * kStageBytes + kWBytes, &mapX, &full[s], (kb0 + i) * kBlockK, xy, pol_x);
      }
      // Every copy this lane issued has landed before it leaves (also when a role gave up): the last STAGES
      // stages' barriers complete exactly once more and are never re-armed.  Bounded like every other wait.
      for (int j = (i > STAGES ? i - STAGES : 0); j < i; ++j) mbar_wait(&full[j % STAGES], (j / STAGES) & 1, nullptr);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (touches shared memory and TMEM only)
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_e4m3(NT);
      for (int i = 0; i < nslab; ++i) {
        const int s = i % STAGES, buf = i % BUFS;
        const uint32_t ph = (i / STAGES) & 1, bph = (i / BUFS) & 1;
        if (!mbar_wait(&tmem_empty[buf], bph ^ 1, abort_flag)) {
          dev_fail(err_flag, kDevWaitTmemEmpty);
          *abort_flag = 1;
          break;
        }
        if (!mbar_wait(&full[s], ph, abort_flag)) {
          dev_fail(err_flag, kDevWaitFull);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint64_t adesc = umma_desc_sw128(smem_u32(tiles + s * kStageBytes));
        const uint64_t bdesc = umma_desc_sw128(smem_u32(tiles + s * kStageBytes + kWBytes));
        const uint32_t d = tmem_base + uint32_t(buf * ACCW);
#pragma unroll
        for (int k = 0; k < kBlockK / 32; ++k)  // K = 32 bytes per instruction: advance the start address by 32 B
          umma_f8(d, adesc + uint64_t(k * 2), bdesc + uint64_t(k * 2), idesc, k > 0 ? 1u : 0u);

        umma_commit(&empty[s]);         // the stage may be refilled once these MMAs have read it
        umma_commit(&tmem_full[buf]);   // the accumulator is complete
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps (TMEM lane quarter = warp % 4)
    // The tile's weight scales (128 floats per K block, constant over the step) are requested into L2 before the wait:
    // the register ring below then reads them at L2 latency however busy HBM is.
    for (int j = threadIdx.x - 64; j < nslab * 4; j += epi_warps(NT) * 32)
      asm volatile("prefetch.global.L2 [%0];" ::"l"(ws + size_t(kb0 + (j >> 2)) * N_pad + tile_n * kTileN + (j & 3) * 32));
    pdl_wait();  // the activation scales and the output planes belong to the kernels before this one
    constexpr int EW = epi_warps(NT), NTH = NT / (EW / 4);  // columns (token rows) of the accumulator this warp promotes
    const int quarter = warp & 3;
    const int col0 = ((warp - 2) >> 2) * NTH;
    const int row = quarter * 32 + lane;
    const int n = tile_n * kTileN + row;
    const int m0 = tile_m * NT + col0;
    float acc[NTH];
#pragma unroll
    for (int j = 0; j < NTH; ++j) acc[j] = 0.f;
    // The block scales run ahead of the accumulators: this row's weight scale of the next kScaleAhead K blocks sits in
    // registers, the token rows' activation scales arrive by cp.async in this warp's ring in shared memory.  Neither
    // load is then on the per-block critical path (wait for the MMA, read TMEM, promote, release the buffer).
    float* ring = xs_ring + (warp - 2) * kScaleRing * NTH;
    auto fetch_xs = [&](int i) {
      if (i < nslab && lane < NTH / 4) ldgsts16(ring + (i % kScaleRing) * NTH + lane * 4, xs + size_t(kb0 + i) * xrows + m0 + lane * 4);
      ldgsts_commit();
    };
    float wq[kScaleAhead];
#pragma unroll
    for (int j = 0; j < kScaleAhead; ++j) {
      wq[j] = j < nslab ? __ldg(ws + size_t(kb0 + j) * N_pad + n) : 0.f;
      fetch_xs(j);
    }
    bool ok = true;
    for (int i = 0; i < nslab && ok; ++i) {
      const int buf = i % BUFS;
      const uint32_t bph = (i / BUFS) & 1;
      const float wsc = wq[0];
#pragma unroll
      for (int j = 0; j + 1 < kScaleAhead; ++j) wq[j] = wq[j + 1];
      wq[kScaleAhead - 1] = i + kScaleAhead < nslab ? __ldg(ws + size_t(kb0 + i + kScaleAhead) * N_pad + n) : 0.f;
      fetch_xs(i + kScaleAhead);
      ldgsts_wait<kScaleAhead>();  // the group of block i has landed (this lane's part)
      __syncwarp();                // ... and every lane's part
      const float4* xs4 = reinterpret_cast<const float4*>(ring + (i % kScaleRing) * NTH);
      ok = mbar_wait(&tmem_full[buf], bph, abort_flag);
      if (!ok) {
        dev_fail(err_flag, kDevWaitTmemFull);
        *abort_flag = 1;
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(buf * ACCW + col0);
      // columns per TMEM read: the whole accumulator for the 32-row token tile, 16 at a time for the wider ones (registers)
      constexpr int CH = NTH == 32 ? 32 : 16;
      static_assert(NTH % CH == 0, "whole TMEM reads");
      // Where the registers allow it (the narrowest and the widest tile) the warp's whole part of the accumulator is read
      // at once and the buffer handed back to the MMA issuer before the promotion; otherwise 16 columns at a time.
      constexpr bool kWhole = NT == 32 || NT == 128;
      if constexpr (kWhole) {
        uint32_t v[NTH / CH][CH];
#pragma unroll
        for (int c = 0; c < NTH / CH; ++c) tmem_ld<CH>(taddr + c * CH, v[c]);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[buf]);
#pragma unroll
        for (int q = 0; q < NTH / 4; ++q) {
          const float4 s4 = xs4[q];
          const uint32_t* vq = &v[(q * 4) / CH][(q * 4) % CH];
          promote4(acc + q * 4, vq, wsc, s4);
        }
      } else {
#pragma unroll
        for (int c = 0; c < NTH / CH; ++c) {
          uint32_t v[CH];
          tmem_ld<CH>(taddr + c * CH, v);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < CH / 4; ++q) {
            const float4 s4 = xs4[c * (CH / 4) + q];
            promote4(acc + c * CH + q * 4, v + q * 4, wsc, s4);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[buf]);
      }
    }
    ldgsts_wait<0>();
    {
      const bool store = ok && (head.tile_val == nullptr || head.store_logits);
      if (store && n < N) {
        float* o = out + size_t(split) * split_stride + n;
#pragma unroll
        for (int j = 0; j < NTH; ++j)
          if (m0 + j < M) o[size_t(m0 + j) * ld] = acc[j];
      }
      if (sw.tickets != nullptr) {
        // silu(gate) * up and its FP8 copy by the CTA that finishes a (gate tile, up tile) pair last: the 2 x splits CTAs
        // of the pair take a ticket once their partial sums are stored; the last one adds the planes in plane order, applies
        // the activation and quantizes the block of 128 features -- the arithmetic of silu_mul_quant_kernel, bit for bit,
        // without that kernel's launch and its round trip.  Every epilogue warp takes part whatever happened before, so the
        // named barriers are complete; the ticket word returns to zero for the next launch.
        const int T = sw.up_col0 / kTileN, pair = tile_n % T;
        unsigned* ticket = sw.tickets + size_t(tile_m) * T + pair;
        __threadfence();
        asm volatile("bar.sync 1, %0;" ::"n"(EW * 32) : "memory");
        if (warp == 2 && lane == 0) {
          const unsigned t = atomicAdd(ticket, 1u);
          const bool last = t == unsigned(2 * splits - 1);
          if (last) *ticket = 0u;
          red_idx[0] = last ? 1 : 0;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(EW * 32) : "memory");
        if (red_idx[0] != 0) {
          __threadfence();
          // A warp takes a token row at a time, lane l its features 4 l .. 4 l + 3 of the pair's 128: the planes' loads of a row
          // are issued together (one round trip to L2, where the other CTAs' partial sums are), and two rows are in flight where the registers allow.
          const int f = pair * kTileN + lane * 4, ew = warp - 2;
          const int m_end = min(M, (tile_m + 1) * NT);
          auto load_row = [&](int m, float4 (&tg)[kFusePlanes], float4 (&tu)[kFusePlanes]) {
            const float* gp = out + size_t(m) * ld + f;
#pragma unroll
            for (int p = 0; p < kFusePlanes; ++p) {
              const bool on = p < splits && m < m_end && f < sw.I;
              tg[p] = on ? __ldcg(reinterpret_cast<const float4*>(gp + size_t(p) * split_stride)) : make_float4(0.f, 0.f, 0.f, 0.f);
              tu[p] = on ? __ldcg(reinterpret_cast<const float4*>(gp + size_t(p) * split_stride + sw.up_col0)) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
          };
          auto finish_row = [&](int m, const float4 (&tg)[kFusePlanes], const float4 (&tu)[kFusePlanes]) {
            if (m >= m_end) return;  // warp-uniform
            float4 g4 = make_float4(0.f, 0.f, 0.f, 0.f), u4 = g4;
#pragma unroll
            for (int p = 0; p < kFusePlanes; ++p) {
              g4.x += tg[p].x, g4.y += tg[p].y, g4.z += tg[p].z, g4.w += tg[p].w;
              u4.x += tu[p].x, u4.y += tu[p].y, u4.z += tu[p].z, u4.w += tu[p].w;
            }
            float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
            if (f < sw.I) x = make_float4(silu(g4.x) * u4.x, silu(g4.y) * u4.y, silu(g4.z) * u4.z, silu(g4.w) * u4.w);
            const float amax = warp_max(fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w))));
            const float sc = amax > 0.f ? amax / 448.f : 1.f;
            if (f < sw.K_pad) {
              uchar4 o;
              o.x = to_e4m3(__fdiv_rn(x.x, sc)), o.y = to_e4m3(__fdiv_rn(x.y, sc));
              o.z = to_e4m3(__fdiv_rn(x.z, sc)), o.w = to_e4m3(__fdiv_rn(x.w, sc));
              *reinterpret_cast<uchar4*>(sw.codes + size_t(m) * sw.K_pad + f) = o;
              if (lane == 0) sw.scales[size_t(pair) * sw.rows_alloc + m] = sc;
            }
          };
          if constexpr (NT == 32) {  // the latency-bound few-row step: two rows in flight (the wider tiles have no registers for that)
            for (int m = tile_m * NT + ew; m < m_end; m += 2 * EW) {
              float4 ag[kFusePlanes], au[kFusePlanes], bg[kFusePlanes], bu[kFusePlanes];
              load_row(m, ag, au);
              load_row(m + EW, bg, bu);
              finish_row(m, ag, au);
              finish_row(m + EW, bg, bu);
            }
          } else {
            for (int m = tile_m * NT + ew; m < m_end; m += EW) {
              float4 ag[kFusePlanes], au[kFusePlanes];
              load_row(m, ag, au);
              finish_row(m, ag, au);
            }
          }
        }
      }
      if (head.tile_val != nullptr) {
        // Per token row: the best (value, id) among this tile's 128 vocabulary rows; larger value first, equal
        // values to the lower id, NaN skipped.  All epilogue warps take part whatever happened before, so the
        // named barrier below is always complete.
#pragma unroll
        for (int j = 0; j < NTH; ++j) {
          float v = acc[j];
          int id = n;
          if (!ok || !(n < N) || v != v) {
            v = -FLT_MAX;
            id = 0x7fffffff;
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            const float v2 = __shfl_xor_sync(0xffffffffu, v, o);
            const int i2 = __shfl_xor_sync(0xffffffffu, id, o);
            if (v2 > v || (v2 == v && i2 < id)) v = v2, id = i2;
          }
          if (lane == 0) red_val[quarter * NT + col0 + j] = v, red_idx[quarter * NT + col0 + j] = id;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(EW * 32) : "memory");
        if (warp == 2) {
          const int m0 = tile_m * NT;  // all columns of the tile
          for (int j = lane; j < NT; j += 32) {
            float v = red_val[j];
            int id = red_idx[j];
#pragma unroll
            for (int q = 1; q < 4; ++q) {
              const float v2 = red_val[q * NT + j];
              const int i2 = red_idx[q * NT + j];
              if (v2 > v || (v2 == v && i2 < id)) v = v2, id = i2;
            }
            if (m0 + j < M) {
              head.tile_val[size_t(tile_n) * head.rows_alloc + m0 + j] = v;
              head.tile_idx[size_t(tile_n) * head.rows_alloc + m0 + j] = id;
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (timeline && threadIdx.x == 0) atomicMax(timeline + 3, global_ns());
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------- tensor peak
// What the FP8 tensor pipe sustains when nothing else is in the way: every CTA (one per SM) issues `iters` groups of four
// tcgen05.mma kind::f8f6f4 (M = 128, N = 256, K = 32 each: one 128-wide K block) on two operand tiles that sit in shared
// memory for the whole kernel, alternating between two TMEM accumulators; no loads, no epilogue.  The denominator for the
// many-row (tensor-bound) configurations, measured rather than quoted.
__global__ void __launch_bounds__(128, 1) tensor_peak_kernel(int iters, int* err_flag) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* a = smem;                    // [128 rows][128 B]
  uint8_t* b = smem + 128 * 128;        // [256 rows][128 B]
  uint64_t* bar = reinterpret_cast<uint64_t*>(b + 256 * 128);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 1);
  for (int i = threadIdx.x; i < (128 + 256) * 128; i += blockDim.x)
    smem[i] = uint8_t(0x30 + ((i * 2654435761u) >> 28));  // E4M3 codes around 1: real switching activity, no NaN
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) {
    constexpr uint32_t idesc = umma_idesc_e4m3(256);
    const uint64_t adesc = umma_desc_sw128(smem_u32(a)), bdesc = umma_desc_sw128(smem_u32(b));
    for (int i = 0; i < iters; ++i) {
      const uint32_t d = tmem_base + uint32_t((i & 1) * 256);
#pragma unroll
      for (int k = 0; k < 4; ++k) umma_f8(d, adesc + uint64_t(k * 2), bdesc + uint64_t(k * 2), idesc, (i > 1 || k > 0) ? 1u : 0u);
    }
    umma_commit(bar);
    if (!mbar_wait(bar, 0, nullptr)) dev_fail(err_flag, kDevWaitTmemFull);
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------- the bounded wait, alone
// One CTA arms an mbarrier that nobody ever arrives at and waits on it with the kernels' bounded wait under a short limit:
// the wait runs out, the thread records the code a GEMM consumer would record (kDevWaitFull) in the error word, notes how
// long it waited, and the kernel returns normally.  What a hung producer looks like to the roles behind it, made on
// purpose and harmlessly: the check that an expired wait leaves the context usable.
__global__ void wait_probe_kernel(unsigned long long limit_ns, int* err_flag, unsigned long long* waited_ns) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned long long t0 = global_ns();
    if (!mbar_wait_for(&bar, 0, nullptr, limit_ns)) dev_fail(err_flag, kDevWaitFull);
    *waited_ns = global_ns() - t0;
  }
}

// ---------------------------------------------------------------------------------------------- CUDA-core GEMM
// The same arithmetic on CUDA cores: one block = one 128-row weight tile x 8 token rows, a warp per weight row,
// lanes split the 128-wide block four codes each.  Exists to cross-check the tensor-core kernel, not to be fast.
__global__ void __launch_bounds__(256)
    gemm_fp8_simt_kernel(const uint8_t* __restrict__ w, const float* __restrict__ ws, const uint8_t* __restrict__ x,
                         const float* __restrict__ xs, float* __restrict__ out, int ld, int M, int N, int N_pad,
                         int K_pad, int KB, int xrows, HeadArgs head) {
  pdl_sync();  // first statement: see common.cuh
  __shared__ float red_val[8][8];
  __shared__ int red_idx[8][8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * 8;
  float bestv[8];
  int besti[8];
#pragma unroll
  for (int r = 0; r < 8; ++r) bestv[r] = -FLT_MAX, besti[r] = 0x7fffffff;
  for (int rr = 0; rr < 16; ++rr) {
    const int n = blockIdx.x * kTileN + warp * 16 + rr;
    float acc[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) acc[r] = 0.f;
    for (int kb = 0; kb < KB; ++kb) {
      const uint32_t wc = *reinterpret_cast<const uint32_t*>(w + size_t(n) * K_pad + kb * kBlockK + lane * 4);
      float wf[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) wf[i] = from_e4m3(uint8_t(wc >> (8 * i)));
      const float wsc = ws[size_t(kb) * N_pad + n];
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const int m = m0 + r;
        if (m >= M) continue;  // uniform across the warp
        const uint32_t xc = *reinterpret_cast<const uint32_t*>(x + size_t(m) * K_pad + kb * kBlockK + lane * 4);
        float p = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) p = fmaf(wf[i], from_e4m3(uint8_t(xc >> (8 * i))), p);
        p = warp_sum(p);
        acc[r] = fmaf(p, wsc * xs[size_t(kb) * xrows + m], acc[r]);
      }
    }
    const bool store = head.tile_val == nullptr || head.store_logits;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const int m = m0 + r;
      if (m >= M || n >= N) continue;
      if (store && lane == 0) out[size_t(m) * ld + n] = acc[r];
      const float v = acc[r];
      if (v == v && (v > bestv[r] || (v == bestv[r] && n < besti[r]))) bestv[r] = v, besti[r] = n;
    }
  }
  if (head.tile_val == nullptr) return;
  if (lane == 0)
    for (int r = 0; r < 8; ++r) red_val[warp][r] = bestv[r], red_idx[warp][r] = besti[r];
  __syncthreads();
  if (threadIdx.x < 8 && m0 + threadIdx.x < M) {
    const int r = threadIdx.x;
    float v = red_val[0][r];
    int id = red_idx[0][r];
    for (int q = 1; q < 8; ++q)
      if (red_val[q][r] > v || (red_val[q][r] == v && red_idx[q][r] < id)) v = red_val[q][r], id = red_idx[q][r];
    head.tile_val[size_t(blockIdx.x) * head.rows_alloc + m0 + r] = v;
    head.tile_idx[size_t(blockIdx.x) * head.rows_alloc + m0 + r] = id;
  }
}

// ---------------------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int encode_2d(CUtensorMap* map, void* base, uint64_t inner, uint64_t rows, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from the driver");
    return LING_B200_ERR_CUDA;
  }
  const cuuint64_t dims[2] = {inner, rows};
  const cuuint64_t strides[1] = {inner};  // bytes between rows
  const cuuint32_t box[2] = {kBlockK, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with code " + std::to_string(int(r)));
    return LING_B200_ERR_CUDA;
  }
  return LING_B200_OK;
}

template <int NT>
int init_tc() {
  LB_CUDA(cudaFuncSetAttribute(gemm_fp8_tcgen05_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               int(gemm_smem_bytes(NT))));
  return LING_B200_OK;
}

template <int NT>
int launch_tc(const GemmCall& c, cudaStream_t stream) {
  const size_t smem = gemm_smem_bytes(NT);
  const Fp8Matrix& W = *c.W;
  const Fp8Acts& X = *c.X;
  HeadArgs h{nullptr, nullptr, 0, 0};
  if (c.head) h = HeadArgs{c.head->tile_val, c.head->tile_idx, c.head->rows_alloc, c.head->store_logits ? 1 : 0};
  const int splits = c.head ? 1 : W.splits;
  SwigluArgs sw{nullptr, 0, 0, nullptr, nullptr, 0, 0};
  if (c.swiglu) {
    if (c.head || c.swiglu->up_col0 % kTileN != 0 || c.swiglu->up_col0 < c.swiglu->I || !c.swiglu->tickets) {
      set_error("gemm: the fused activation needs the up columns on a tile boundary behind the gate columns");
      return LING_B200_ERR_ARG;
    }
    sw = SwigluArgs{c.swiglu->tickets, c.swiglu->I, c.swiglu->up_col0, c.swiglu->codes, c.swiglu->scales, c.swiglu->K_pad, c.swiglu->rows_alloc};
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ceil_div(c.M, NT), splits, W.N_pad / kTileN);
  cfg.blockDim = dim3(gemm_threads(NT));
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  const bool pdl = pdl_enabled();
  cfg.numAttrs = pdl ? 1 : 0;
  // L2 prefetch budget of one GEMM before its dependency wait: 16 MB of weight tiles beyond the pipeline stages, spread
  // over its CTAs (measured on the 27B shapes: 0 MB 8.75 ms per step, 16 MB 8.72, 40 MB 8.96, 80 MB 9.18), and every
  // pipeline stage filled before the wait
  const int ctas = int(cfg.gridDim.z * cfg.gridDim.y);
  constexpr int kL2PrefetchMb = 16, pre_stages = 30;
  const int l2_slabs = std::min(64, int((size_t(kL2PrefetchMb) << 20) / (size_t(ctas) * kABytes)));
  LB_CUDA(cudaLaunchKernelEx(&cfg, gemm_fp8_tcgen05_kernel<NT>, W.map, X.map[NT / 32 - 1], (const float*)W.scales,
                             (const float*)X.scales, c.out, c.ld, c.split_stride, c.M, W.N, W.N_pad, W.KB, splits,
                             X.rows_alloc, h, c.err_flag, pdl ? 1 + pre_stages : 0, pdl && cfg.gridDim.x == 1 ? l2_slabs : 0,
                             c.timeline, sw));
  LB_LAUNCH("gemm_fp8_tcgen05_kernel");
  return LING_B200_OK;
}

}  // namespace

// Opts the kernels into their dynamic shared memory; called once per device before the first launch (never inside a
// stream capture).
int gemm_init() {
  if (const int r = init_tc<32>()) return r;
  if (const int r = init_tc<64>()) return r;
  if (const int r = init_tc<96>()) return r;
  return init_tc<128>();
}

int encode_tile_map(CUtensorMap* map, void* base, uint64_t row_bytes, uint64_t rows, uint32_t box_rows) {
  return encode_2d(map, base, row_bytes, rows, box_rows);
}

int encode_linear_map(CUtensorMap* map, void* base, uint64_t row_bytes, uint64_t rows, uint32_t box_bytes) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from the driver");
    return LING_B200_ERR_CUDA;
  }
  const cuuint64_t dims[2] = {row_bytes / 8, rows};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {box_bytes / 8, 1};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled (linear) failed with code " + std::to_string(int(r)));
    return LING_B200_ERR_CUDA;
  }
  return LING_B200_OK;
}

int make_weight_map(Fp8Matrix& w) { return encode_2d(&w.map, w.codes, uint64_t(w.K_pad), uint64_t(w.N_pad), kTileN); }

int make_acts_maps(Fp8Acts& x) {
  for (int i = 0; i < 4; ++i) {
    const int nt = 32 * (i + 1);
    if (const int r = encode_2d(&x.map[i], x.codes, uint64_t(x.K_pad), uint64_t(x.rows_alloc), uint32_t(nt))) return r;
  }
  return LING_B200_OK;
}

int tensor_peak_launch(int ctas, int iters, int* err_flag, cudaStream_t stream) {
  constexpr int smem = (128 + 256) * 128 + 1024 + 64;
  static bool attr = false;
  if (!attr) {
    LB_CUDA(cudaFuncSetAttribute(tensor_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    attr = true;
  }
  tensor_peak_kernel<<<ctas, 128, smem, stream>>>(iters, err_flag);
  LB_LAUNCH("tensor_peak_kernel");
  return LING_B200_OK;
}

int wait_probe_launch(unsigned long long limit_ns, int* err_flag, unsigned long long* waited_ns, cudaStream_t stream) {
  wait_probe_kernel<<<1, 32, 0, stream>>>(limit_ns, err_flag, waited_ns);
  LB_LAUNCH("wait_probe_kernel");
  return LING_B200_OK;
}

// Up to 128 rows: the smallest tile that holds them.  Beyond: the GEMM's time is its padded rows (tiles x tile rows) times the
// tile's cost per row -- measured at 2048 rows, where no tile pads: in projection 320 us with 96-row tiles, 360 with 128; out
// projection 178 / 216; gate|up 605 / 620; per row 0.336 us at 96, 0.344 at 64 on the gate|up shape -- so the tile with the least
// weighted padding: 142 rows run as 2 x 96 (68 us) rather than 2 x 128 (88), 260 as 3 x 96 (99 vs 130), 300 as 5 x 64 (111 vs
// 130), 2048 as 32 x 64 rather than 16 x 128 (22 x 96 would pad past the buffers' 128-row granularity).  The result does not depend on the choice (a row's arithmetic is the same in
// every tile size).
int token_tile(int M) {
  if (M <= 128) return M <= 32 ? 32 : M <= 64 ? 64 : M <= 96 ? 96 : 128;
  // (never more padded rows than 128-row tiles would have: the activation buffers are allocated in whole 128-row tiles)
  const int limit = round_up(M, 128);
  int best = 128;
  double best_cost = double(limit) * 1.08;
  for (const auto& [nt, per_row] : {std::pair<int, double>{96, 1.0}, {64, 1.05}}) {
    const double cost = double(round_up(M, nt)) * per_row;
    if (round_up(M, nt) <= limit && cost < best_cost) best = nt, best_cost = cost;
  }
  return best;
}

int choose_splits(int N_pad, int KB, int sm_count) {
  const int tiles = N_pad / kTileN;
  // Two CTAs are resident per SM for the narrow token tiles: as many splits as keep tiles x splits within one wave
  // (2 x SMs), at least four K blocks per split so that the prologue and the partial-sum traffic stay small, at most
  // kMaxPlanes-many planes for the consumers to add.
  int s = (2 * sm_count) / tiles;
  s = std::min(s, KB / 4);
  s = std::max(s, 1);
  return std::min(s, 8);
}

int gemm_launch(const GemmCall& c, cudaStream_t stream) {
  const Fp8Matrix& W = *c.W;
  const Fp8Acts& X = *c.X;
  if (W.K_pad != X.K_pad || c.M < 1 || c.M > X.rows_alloc) {
    set_error("gemm: shape mismatch");
    return LING_B200_ERR_ARG;
  }
  if (c.impl == 1) {
    HeadArgs h{nullptr, nullptr, 0, 0};
    if (c.head) h = HeadArgs{c.head->tile_val, c.head->tile_idx, c.head->rows_alloc, c.head->store_logits ? 1 : 0};
    const dim3 grid(W.N_pad / kTileN, ceil_div(c.M, 8));
    LB_CUDA(launch_kernel(gemm_fp8_simt_kernel, grid, dim3(256), size_t(0), stream, (const uint8_t*)W.codes,
                          (const float*)W.scales, (const uint8_t*)X.codes, (const float*)X.scales, c.out, c.ld, c.M, W.N, W.N_pad,
                          W.K_pad, W.KB, X.rows_alloc, h));
    return LING_B200_OK;
  }
  switch (c.force_tile > 0 ? c.force_tile : token_tile(c.M)) {
    case 32: return launch_tc<32>(c, stream);
    case 64: return launch_tc<64>(c, stream);
    case 96: return launch_tc<96>(c, stream);
    default: return launch_tc<128>(c, stream);
  }
}

}  // namespace lb
