// nvfp4.cu -- the NVFP4 GEMMs of the prefill chunk and the quantizers that feed them (see nvfp4.h) for sm_100a.
//
// GEMM kernel shape (persistent: one CTA per SM walks the 128 x 256 output tiles, token tiles fastest):
//   warp 0   producer (one lane): per stage of 256 K values, TMA tiles of the activations (128 rows x 128 B) and of the
//            weights (2 x 128 rows x 128 B) into 128B-swizzled shared memory, and the three row groups' block scales
//            (2 KiB each, already in the order tcgen05.cp reads) by bulk copy; all counted on the stage's mbarrier.
//   warp 1   MMA issuer (one lane): copies the stage's block scales into tensor memory (tcgen05.cp 32x128b.warpx4: each
//            512-byte atom becomes four TMEM columns, replicated over the four lane quarters), then four
//            tcgen05.mma kind::mxf4nvf4.block_scale (M 128, N 256, K 64, scale vector 16) into the 256-column
//            accumulator; tcgen05.commit releases the stage and, after the last stage, hands the tile to the epilogue.
//   warps 2-17 epilogue (four per TMEM lane quarter, a quarter of the columns each): tcgen05.ld of the tile; plain form: alpha * acc to y (or added to it); fused form: the gate and up
//            halves of the tile become silu(alpha * gate) * (alpha2 * up), rounded to BF16 and written as the next GEMM's
//            NVFP4 operand (16 features = one block scale, all in one thread).
// TMEM: columns 0-255 accumulator, 256-271 activation scales of the stage, 272-303 weight scales.  One accumulator: an
// epilogue warp reads its columns into registers, hands the accumulator back, and does its arithmetic and stores while
// the next tile's MMAs run (what stays exposed is the TMEM read).
// Every wait is bounded; a wait that runs out records a code in the device error word and the CTA unwinds.
#include "nvfp4.h"

#include <atomic>
#include <mutex>

#include "../../include/ling_b200.h"
#include "gemm.h"
#include "tc.cuh"

namespace lb {

namespace {
using namespace tc;

constexpr int kStages = 4;
constexpr int kRowBytes = kFp4StageK / 2;         // 128
constexpr int kABytes = kFp4TileM * kRowBytes;    // 16 KiB
constexpr int kBBytes = kFp4TileN * kRowBytes;    // 32 KiB
constexpr int kSfGroup = (kFp4StageK / 64) * 512;  // one 128-row group's scales of a stage: 2 KiB
constexpr int kStageBytes = kABytes + kBBytes + 3 * kSfGroup;
constexpr int kSfaCol = 256, kSfbCol = 272, kTmemCols = 512;
constexpr int kEpiWarps = 16;  // four per TMEM lane quarter, each draining a quarter of the tile's columns
constexpr int kThreads = 64 + 32 * kEpiWarps;
constexpr size_t kSmemBytes = size_t(kStages) * kStageBytes + 1024 /* alignment slack */ + 256 /* barriers */;
static_assert(kStageBytes % 1024 == 0, "swizzled tiles start on 1024-byte boundaries");

// Instruction descriptor, kind::mxf4nvf4: A = B = E2M1 (format 1), both K-major, scale format UE4M3 (bit 23 clear),
// M = 128, N = n; the scale-factor ids select bytes of a TMEM column for narrower scale vectors and stay 0 here.
__host__ __device__ constexpr uint32_t umma_idesc_nvfp4(int n) {
  return (1u << 7) | (1u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(128 >> 4) << 24);
}
__device__ __forceinline__ void umma_nvfp4(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n" ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
      : "memory");
}
// Shared-memory descriptor of one scale atom for tcgen05.cp: 32 rows of 16 bytes, no swizzle, 8-row groups 128 bytes apart.
__device__ __forceinline__ uint64_t sf_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= uint64_t((smem_addr & 0x3FFFFu) >> 4);
  d |= uint64_t(128 >> 4) << 32;  // stride byte offset
  d |= uint64_t(1) << 46;         // descriptor version (sm_100)
  return d;
}
__device__ __forceinline__ void sf_copy(uint32_t tmem_col, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_col), "l"(desc) : "memory");
}
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// Two floats to two E2M1 codes in a byte (lo in the low nibble), round to nearest even, saturating.
__device__ __forceinline__ uint32_t e2m1x2(float lo, float hi) {
  uint16_t out;
  asm("{\n .reg .b8 b;\n cvt.rn.satfinite.e2m1x2.f32 b, %1, %2;\n mov.b16 %0, {b, b};\n}" : "=h"(out) : "f"(hi), "f"(lo));
  return out & 0xffu;
}

// One block of 16 values (already rounded to BF16) under the global scale: the block's E4M3 scale and eight code bytes.
__device__ __forceinline__ uint8_t encode_block(const float (&v)[16], float gscale, uint2& codes) {
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[j]));
  const uint8_t sc = to_e4m3(gscale * (amax * (1.f / 6.f)));
  const float sv = from_e4m3(sc);
  const float os = sv != 0.f ? 1.f / (sv * (1.f / gscale)) : 0.f;
  uint32_t w[2] = {0u, 0u};
#pragma unroll
  for (int j = 0; j < 8; ++j) w[j >> 2] |= e2m1x2(v[2 * j] * os, v[2 * j + 1] * os) << (8 * (j & 3));
  codes = make_uint2(w[0], w[1]);
  return sc;
}

struct GemmArgs {
  const uint8_t* sfa;
  const uint8_t* sfb0;
  const uint8_t* sfb1;
  int M, N;             // rows; output columns (features in the fused form)
  int k_stages;         // K_pad / 256
  int tiles_m, tiles_n;
  int b_step, b1_off;   // first weight row of tile n: n * b_step in map B0, n * b_step + b1_off in map B1
  int g_mul, g1_off;    // scale row group of tile n: n * g_mul of sfb0, n * g_mul + g1_off of sfb1
  float alpha, alpha2, gscale_out;
  float* y;
  int ldy, accumulate;
  uint8_t* q_out;
  uint8_t* sf_out;
  int sf_out_tiled, out_atoms;
  int* err_flag;
  unsigned long long* stats;  // optional cycle sums over all CTAs: [0] issuer waiting for stages, [1] issuer waiting for the
                              // epilogue, [2] epilogue busy (one warp), [3] whole CTA
};

// One epilogue warp's part of a finished tile: TMEM lanes = token rows (this thread's row), columns = the tile's weight rows;
// `part` selects which of the tile's eight column groups this warp drains (8 / (kEpiWarps / 4) of them).  The warp first
// reads ALL of its columns into registers and calls release() -- the accumulator is then free for the next tile's MMAs --
// and only then does the arithmetic and the stores, which so run under the next tile's main loop.
template <bool SWIGLU, typename Release>
__device__ __forceinline__ void drain_tile(const GemmArgs& p, uint32_t taddr, int row, int tn, int part, Release release) {
  constexpr int kGroups = 8 / (kEpiWarps / 4);  // column groups per warp
  if constexpr (SWIGLU) {
    const int f0 = tn * 128;  // the tile's first feature: columns 0-127 its gate products, 128-255 its up products
    uint32_t g[kGroups][16], u[kGroups][16];
#pragma unroll
    for (int i = 0; i < kGroups; ++i) {
      tmem_ld16(taddr + 16 * (kGroups * part + i), g[i]);
      tmem_ld16(taddr + 128 + 16 * (kGroups * part + i), u[i]);
    }
    tmem_ld_wait();
    release();
#pragma unroll
    for (int i = 0; i < kGroups; ++i) {
      float v[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = bf16_round(silu(__uint_as_float(g[i][j]) * p.alpha) * (__uint_as_float(u[i][j]) * p.alpha2));
      uint2 codes;
      const uint8_t sc = encode_block(v, p.gscale_out, codes);
      if (row < p.M) {
        const int f = f0 + 16 * (kGroups * part + i);
        *reinterpret_cast<uint2*>(p.q_out + size_t(row) * (p.N / 2) + f / 2) = codes;
        p.sf_out[p.sf_out_tiled ? fp4_sf_offset(row, f / 16, p.out_atoms) : size_t(row) * (p.N / 16) + f / 16] = sc;
      }
    }
  } else {
    const int n0 = tn * kFp4TileN;
    uint32_t v[kGroups][32];
#pragma unroll
    for (int i = 0; i < kGroups; ++i) tmem_ld32(taddr + 32 * (kGroups * part + i), v[i]);
    tmem_ld_wait();
    release();
#pragma unroll
    for (int i = 0; i < kGroups; ++i) {
      const int c = kGroups * part + i;
      if (row < p.M && n0 + 32 * c < p.N) {
        float4* dst = reinterpret_cast<float4*>(p.y + size_t(row) * p.ldy + n0 + 32 * c);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float4 o = make_float4(__uint_as_float(v[i][4 * j]) * p.alpha, __uint_as_float(v[i][4 * j + 1]) * p.alpha,
                                 __uint_as_float(v[i][4 * j + 2]) * p.alpha, __uint_as_float(v[i][4 * j + 3]) * p.alpha);
          if (p.accumulate) {
            const float4 old = dst[j];
            o.x += old.x, o.y += old.y, o.z += old.z, o.w += old.w;
          }
          dst[j] = o;
        }
      }
    }
  }
}

template <bool SWIGLU>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_nvfp4_tcgen05_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB0,
                              const __grid_constant__ CUtensorMap mapB1, const GemmArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* empty = full + kStages;
  uint64_t* tmem_full = empty + kStages;
  uint64_t* tmem_empty = tmem_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles = p.tiles_m * p.tiles_n;
  const int k_atoms = p.k_stages * 4;
  const long long t_start = clock64();

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&mapA)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&mapB0)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&mapB1)) : "memory");
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(tmem_full, 1);
    mbar_init(tmem_empty, kEpiWarps);
    *abort_flag = 0;
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

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      const uint64_t pol_w = policy_evict_last();  // both operands are re-read by other tiles: keep them in L2
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
        const int tm = t % p.tiles_m, tn = t / p.tiles_m;
        const uint8_t* sa = p.sfa + size_t(tm) * k_atoms * 512;
        const uint8_t* sb0 = p.sfb0 + size_t(tn * p.g_mul) * k_atoms * 512;
        const uint8_t* sb1 = p.sfb1 + size_t(tn * p.g_mul + p.g1_off) * k_atoms * 512;
        for (int ks = 0; ks < p.k_stages; ++ks, ++it) {
          const int s = it % kStages;
          ok = mbar_wait(&empty[s], ((it / kStages) & 1) ^ 1, abort_flag);
          if (!ok) {
            dev_fail(p.err_flag, kDevWaitEmpty);
            *abort_flag = 1;
            break;
          }
          uint8_t* st = smem + s * kStageBytes;
          mbar_expect_tx(&full[s], kStageBytes);
          tma_load_2d(st, &mapA, &full[s], ks * kRowBytes, tm * kFp4TileM, pol_w);
          tma_load_2d(st + kABytes, &mapB0, &full[s], ks * kRowBytes, tn * p.b_step, pol_w);
          tma_load_2d(st + kABytes + kBBytes / 2, &mapB1, &full[s], ks * kRowBytes, tn * p.b_step + p.b1_off, pol_w);
          bulk_load(st + kABytes + kBBytes, sa + size_t(ks) * kSfGroup, kSfGroup, &full[s]);
          bulk_load(st + kABytes + kBBytes + kSfGroup, sb0 + size_t(ks) * kSfGroup, kSfGroup, &full[s]);
          bulk_load(st + kABytes + kBBytes + 2 * kSfGroup, sb1 + size_t(ks) * kSfGroup, kSfGroup, &full[s]);
        }
      }
      // every copy this lane issued has landed before it leaves (also when a role gave up)
      for (int j = (it > kStages ? it - kStages : 0); j < it; ++j) mbar_wait(&full[j % kStages], (j / kStages) & 1, nullptr);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_nvfp4(kFp4TileN);
      int it = 0, ti = 0;
      bool ok = true;
      long long w_full = 0, w_empty = 0;
      for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++ti) {
        long long c0 = clock64();
        if (!mbar_wait(tmem_empty, (ti & 1) ^ 1, abort_flag)) {
          dev_fail(p.err_flag, kDevWaitTmemEmpty);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        w_empty += clock64() - c0;
        for (int ks = 0; ks < p.k_stages; ++ks, ++it) {
          const int s = it % kStages;
          c0 = clock64();
          if (!mbar_wait(&full[s], (it / kStages) & 1, abort_flag)) {
            dev_fail(p.err_flag, kDevWaitFull);
            *abort_flag = 1;
            ok = false;
            break;
          }
          w_full += clock64() - c0;
          tc_fence_after();
          const uint32_t st = smem_u32(smem + s * kStageBytes);
          const uint32_t sf = st + kABytes + kBBytes;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            sf_copy(tmem_base + kSfaCol + 4 * k, sf_desc(sf + 512 * k));
            sf_copy(tmem_base + kSfbCol + 8 * k, sf_desc(sf + kSfGroup + 512 * k));
            sf_copy(tmem_base + kSfbCol + 8 * k + 4, sf_desc(sf + 2 * kSfGroup + 512 * k));
          }
          const uint64_t adesc = umma_desc_sw128(st), bdesc = umma_desc_sw128(st + kABytes);
#pragma unroll
          for (int k = 0; k < 4; ++k)  // K = 64 values = 32 bytes per instruction
            umma_nvfp4(tmem_base, adesc + uint64_t(k * 2), bdesc + uint64_t(k * 2), idesc, tmem_base + kSfaCol + 4 * k,
                       tmem_base + kSfbCol + 8 * k, (ks > 0 || k > 0) ? 1u : 0u);
          umma_commit(&empty[s]);
        }
        if (ok) umma_commit(tmem_full);
      }
      if (p.stats) {
        atomicAdd(p.stats, (unsigned long long)w_full);
        atomicAdd(p.stats + 1, (unsigned long long)w_empty);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (TMEM lane quarter = warp % 4)
    const int quarter = warp & 3, part = (warp - 2) >> 2;
    int ti = 0;
    long long busy = 0;
    for (int t = blockIdx.x; t < tiles; t += gridDim.x, ++ti) {
      const int tm = t % p.tiles_m, tn = t / p.tiles_m;
      if (!mbar_wait(tmem_full, ti & 1, abort_flag)) {
        dev_fail(p.err_flag, kDevWaitTmemFull);
        *abort_flag = 1;
        break;
      }
      const long long c0 = clock64();
      tc_fence_after();
      const int row = tm * kFp4TileM + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16);
      drain_tile<SWIGLU>(p, taddr, row, tn, part, [&] {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tmem_empty);
      });
      busy += clock64() - c0;
    }
    if (p.stats && warp == 2 && lane == 0) atomicAdd(p.stats + 2, (unsigned long long)busy);
  }
  tc_fence_before();
  __syncthreads();
  if (p.stats && threadIdx.x == 0) atomicAdd(p.stats + 3, (unsigned long long)(clock64() - t_start));
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------- two-CTA form
// The same GEMM with the MMA spanning a pair of CTAs (a cluster of two, tcgen05 cta_group::2): the pair's tile is 256 token
// rows x 256 weight rows; each CTA keeps its own 128 token rows of A and HALF of B (128 weight rows) in shared memory, the
// tensor cores of both read both halves.  Per CTA and stage 38 KiB arrive instead of 54, and the shared-memory reads of B
// halve: the one-CTA tile is bound by exactly that traffic.  Every CTA issues its own ordinary TMA loads into its own shared
// memory, completing on the LEADER's mbarrier (cta_group::2); the leader (cluster rank 0) arms it for both
// CTAs' bytes, copies the scales and issues the MMAs for the pair; tcgen05.commit with a cluster mask releases the stage in
// both CTAs and hands both accumulators to the two epilogues.  Fused form: the leader's half of B is the gate rows, the
// peer's the up rows of the same 128 features.
constexpr int kPairStages = 5;
constexpr int kPairStageBytes = kABytes + kBBytes / 2 + 3 * kSfGroup;  // 38 KiB: A, half of B, scales of A and of both B halves
constexpr size_t kPairSmemBytes = size_t(kPairStages) * kPairStageBytes + 1024 + 256;
static_assert(kPairStageBytes % 1024 == 0, "swizzled tiles start on 1024-byte boundaries");

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {  // the same offset in another CTA of the cluster
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load of a CTA pair: lands in this CTA's shared memory, completes on the barrier at `bar_cluster_addr` (the leader's).
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x, int y, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void umma_nvfp4_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n" ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
      : "memory");
}
__device__ __forceinline__ void sf_copy_pair(uint32_t tmem_col, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(tmem_col), "l"(desc) : "memory");
}
// Arrives (once the pair's earlier tcgen05 operations are done) on the barrier at this offset in both CTAs of the pair.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_u32(bar)),
               "h"(uint16_t(3))
               : "memory");
}
__host__ __device__ constexpr uint32_t umma_idesc_nvfp4_pair(int n) {  // M = 256 over the pair
  return (1u << 7) | (1u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(256 >> 4) << 24);
}

// The block scales travel as tensor-map tiles too (the completion must reach the leader's barrier, which the plain bulk copy
// cannot address): the scale array of an operand seen as [row groups][k_atoms * 64] 8-byte words, one box = 256 words = the
// 2 KiB of one row group's stage.
template <bool SWIGLU>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_nvfp4_pair_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB0,
                           const __grid_constant__ CUtensorMap mapB1, const __grid_constant__ CUtensorMap mapSA,
                           const __grid_constant__ CUtensorMap mapSB0, const __grid_constant__ CUtensorMap mapSB1, const GemmArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kPairStages * kPairStageBytes);  // used in the leader only
  uint64_t* empty = full + kPairStages;
  uint64_t* tmem_full = empty + kPairStages;
  uint64_t* tmem_empty = tmem_full + 1;  // used in the leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int tiles = p.tiles_m * p.tiles_n;  // tiles_m counts 256-row pair tiles here
  const long long t_start = clock64();

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(tmem_full, 1);
    mbar_init(tmem_empty, 2 * kEpiWarps);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {  // both CTAs, the same warp and the same slot
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    tc_fence_before();
  }
  __syncthreads();
  cluster_sync();  // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (each CTA loads its own operands)
    if (lane == 0) {
      const uint64_t pol = policy_evict_last();
      const CUtensorMap* mapB = leader ? &mapB0 : &mapB1;
      int it = 0;
      bool ok = true;
      for (int t = pair; t < tiles && ok; t += pairs) {
        const int tm = t % p.tiles_m, tn = t / p.tiles_m;
        const int arow = tm * 256 + int(rank) * 128;
        const int brow = tn * p.b_step + (leader ? 0 : p.b1_off);
        const int ga = arow >> 7, gb0 = tn * p.g_mul, gb1 = tn * p.g_mul + p.g1_off;
        for (int ks = 0; ks < p.k_stages; ++ks, ++it) {
          const int s = it % kPairStages;
          ok = mbar_wait(&empty[s], ((it / kPairStages) & 1) ^ 1, abort_flag);
          if (!ok) {
            dev_fail(p.err_flag, kDevWaitEmpty);
            *abort_flag = 1;
            break;
          }
          uint8_t* st = smem + s * kPairStageBytes;
          const uint32_t bar = map_to_cta(smem_u32(&full[s]), 0);
          if (leader) mbar_expect_tx(&full[s], 2 * kPairStageBytes);
          tma_load_2d_pair(st, &mapA, bar, ks * kRowBytes, arow, pol);
          tma_load_2d_pair(st + kABytes, mapB, bar, ks * kRowBytes, brow, pol);
          tma_load_2d_pair(st + kABytes + kBBytes / 2, &mapSA, bar, ks * 256, ga, pol);
          tma_load_2d_pair(st + kABytes + kBBytes / 2 + kSfGroup, &mapSB0, bar, ks * 256, gb0, pol);
          tma_load_2d_pair(st + kABytes + kBBytes / 2 + 2 * kSfGroup, &mapSB1, bar, ks * 256, gb1, pol);
        }
      }
      // The leader waits for every stage it armed (both CTAs' copies have then landed); the peer's copies complete on the
      // leader's barriers, so the closing cluster barrier below is what keeps the peer's shared memory alive until then.
      if (leader)
        for (int j = (it > kPairStages ? it - kPairStages : 0); j < it; ++j) mbar_wait(&full[j % kPairStages], (j / kPairStages) & 1, nullptr);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (the leader, for the pair)
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = umma_idesc_nvfp4_pair(kFp4TileN);
      int it = 0, ti = 0;
      bool ok = true;
      long long w_full = 0, w_empty = 0;
      for (int t = pair; t < tiles && ok; t += pairs, ++ti) {
        long long c0 = clock64();
        if (!mbar_wait(tmem_empty, (ti & 1) ^ 1, abort_flag)) {
          dev_fail(p.err_flag, kDevWaitTmemEmpty);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        w_empty += clock64() - c0;
        for (int ks = 0; ks < p.k_stages; ++ks, ++it) {
          const int s = it % kPairStages;
          c0 = clock64();
          if (!mbar_wait(&full[s], (it / kPairStages) & 1, abort_flag)) {
            dev_fail(p.err_flag, kDevWaitFull);
            *abort_flag = 1;
            ok = false;
            break;
          }
          w_full += clock64() - c0;
          tc_fence_after();
          const uint32_t st = smem_u32(smem + s * kPairStageBytes);
          const uint32_t sf = st + kABytes + kBBytes / 2;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            sf_copy_pair(tmem_base + kSfaCol + 4 * k, sf_desc(sf + 512 * k));
            sf_copy_pair(tmem_base + kSfbCol + 8 * k, sf_desc(sf + kSfGroup + 512 * k));
            sf_copy_pair(tmem_base + kSfbCol + 8 * k + 4, sf_desc(sf + 2 * kSfGroup + 512 * k));
          }
          const uint64_t adesc = umma_desc_sw128(st), bdesc = umma_desc_sw128(st + kABytes);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_nvfp4_pair(tmem_base, adesc + uint64_t(k * 2), bdesc + uint64_t(k * 2), idesc, tmem_base + kSfaCol + 4 * k,
                            tmem_base + kSfbCol + 8 * k, (ks > 0 || k > 0) ? 1u : 0u);
          umma_commit_pair(&empty[s]);
        }
        if (ok) umma_commit_pair(tmem_full);
      }
      if (p.stats) {
        atomicAdd(p.stats, (unsigned long long)w_full);
        atomicAdd(p.stats + 1, (unsigned long long)w_empty);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue: each CTA drains its own 128 rows
    const int quarter = warp & 3, part = (warp - 2) >> 2;
    const uint32_t empty_bar = map_to_cta(smem_u32(tmem_empty), 0);
    int ti = 0;
    long long busy = 0;
    for (int t = pair; t < tiles; t += pairs, ++ti) {
      const int tm = t % p.tiles_m, tn = t / p.tiles_m;
      if (!mbar_wait(tmem_full, ti & 1, abort_flag)) {
        dev_fail(p.err_flag, kDevWaitTmemFull);
        *abort_flag = 1;
        break;
      }
      const long long c0 = clock64();
      tc_fence_after();
      const int row = tm * 256 + int(rank) * 128 + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16);
      drain_tile<SWIGLU>(p, taddr, row, tn, part, [&] {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(empty_bar);
      });
      busy += clock64() - c0;
    }
    if (p.stats && leader && warp == 2 && lane == 0) atomicAdd(p.stats + 2, (unsigned long long)busy);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();  // neither CTA leaves while the other may still signal its barriers or read its shared memory
  if (p.stats && leader && threadIdx.x == 0) atomicAdd(p.stats + 3, (unsigned long long)(clock64() - t_start));
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------- tensor peak
// The NVFP4 tensor pipe's rate on this GPU, measured rather than quoted: every CTA issues `iters` groups of four
// tcgen05.mma kind::mxf4nvf4.block_scale (M 128, N 256, K 64 each) on operand tiles and block scales that stay resident in
// shared / tensor memory; no loads, no epilogue.  The denominator of the NVFP4 GEMMs' roofline fraction (mode 0).  Modes 1
// and 2 add the GEMM's per-stage scale copies (shared memory -> tensor memory) to every group, to price them.
__global__ void __launch_bounds__(128, 1) fp4_tensor_peak_kernel(int iters, int mode, int* err_flag) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* sf = smem + kABytes + kBBytes;  // [3 groups][4 atoms][512]
  uint64_t* bar = reinterpret_cast<uint64_t*>(sf + 3 * kSfGroup);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 2);
  for (int i = threadIdx.x; i < kABytes + kBBytes; i += blockDim.x) smem[i] = uint8_t((i * 2654435761u) >> 24);  // every code
  for (int i = threadIdx.x; i < 3 * kSfGroup; i += blockDim.x) sf[i] = uint8_t(0x30 + ((i * 2654435761u) >> 29));  // 0.5 .. 0.94
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    mbar_init(bar + 1, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) {
    constexpr uint32_t idesc = umma_idesc_nvfp4(kFp4TileN);
    const uint32_t st = smem_u32(smem), sfa = smem_u32(sf);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      sf_copy(tmem_base + kSfaCol + 4 * k, sf_desc(sfa + 512 * k));
      sf_copy(tmem_base + kSfbCol + 8 * k, sf_desc(sfa + kSfGroup + 512 * k));
      sf_copy(tmem_base + kSfbCol + 8 * k + 4, sf_desc(sfa + 2 * kSfGroup + 512 * k));
    }
    const uint64_t adesc = umma_desc_sw128(st), bdesc = umma_desc_sw128(st + kABytes);
    for (int i = 0; i < iters; ++i) {
      // mode 1: the GEMM's twelve scale copies before every group, into the one scale region; mode 2: into two regions in turn
      const uint32_t so = mode == 2 ? uint32_t(i & 1) * 48u : 0u;
      if (mode == 4) {  // the same 48 scale columns written by six 128-lane x 256-bit copies (a source replicated in shared memory)
#pragma unroll
        for (int k = 0; k < 6; ++k) {
          uint64_t dsc = uint64_t(((st + 4096u * k) & 0x3FFFFu) >> 4) | (uint64_t(128 >> 4) << 16) | (uint64_t(256 >> 4) << 32) | (uint64_t(1) << 46);
          asm volatile("tcgen05.cp.cta_group::1.128x256b [%0], %1;" ::"r"(tmem_base + kSfaCol + 8 * k), "l"(dsc) : "memory");
        }
      }
      if (mode == 1 || mode == 2) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          sf_copy(tmem_base + so + kSfaCol + 4 * k, sf_desc(sfa + 512 * k));
          sf_copy(tmem_base + so + kSfbCol + 8 * k, sf_desc(sfa + kSfGroup + 512 * k));
          sf_copy(tmem_base + so + kSfbCol + 8 * k + 4, sf_desc(sfa + 2 * kSfGroup + 512 * k));
        }
      }
#pragma unroll
      for (int k = 0; k < 4; ++k)
        umma_nvfp4(tmem_base, adesc + uint64_t(k * 2), bdesc + uint64_t(k * 2), idesc, tmem_base + so + kSfaCol + 4 * k,
                   tmem_base + so + kSfbCol + 8 * k, (i > 0 || k > 0) ? 1u : 0u);
    }
    umma_commit(bar);
    if (!mbar_wait(bar, 0, nullptr)) dev_fail(err_flag, kDevWaitTmemFull);
  } else if (threadIdx.x == 32 && mode == 3) {
    // mode 3: the same twelve copies per group, but issued by a thread of another warp into a second scale region while
    // thread 0 issues MMAs that read the first: do copies and MMAs from different issuers run side by side?
    const uint32_t sfa = smem_u32(sf);
    for (int i = 0; i < iters; ++i) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        sf_copy(tmem_base + 48 + kSfaCol + 4 * k, sf_desc(sfa + 512 * k));
        sf_copy(tmem_base + 48 + kSfbCol + 8 * k, sf_desc(sfa + kSfGroup + 512 * k));
        sf_copy(tmem_base + 48 + kSfbCol + 8 * k + 4, sf_desc(sfa + 2 * kSfGroup + 512 * k));
      }
    }
    umma_commit(bar + 1);
    if (!mbar_wait(bar + 1, 0, nullptr)) dev_fail(err_flag, kDevWaitTmemFull);
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------- quantizers
__device__ __forceinline__ void store_block(uint8_t* q, uint8_t* sf, bool tiled, int row, int blk, int K, int k_atoms, uint2 codes,
                                            uint8_t sc) {
  *reinterpret_cast<uint2*>(q + size_t(row) * (K / 2) + size_t(blk) * 8) = codes;
  sf[tiled ? fp4_sf_offset(row, blk, k_atoms) : size_t(row) * (K / 16) + blk] = sc;
}

// One thread per block of 16 values.
template <bool SILU>
__global__ void __launch_bounds__(256)
    quant_act_nvfp4_kernel(const float* __restrict__ x, const float* __restrict__ up, int M, int K, float gscale,
                           uint8_t* __restrict__ q, uint8_t* __restrict__ sf, int tiled, int k_atoms) {
  const int bpr = K / 16;
  const size_t blocks = size_t(M) * bpr;
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < blocks; i += size_t(gridDim.x) * blockDim.x) {
    const int row = int(i / bpr), blk = int(i % bpr);
    const float4* src = reinterpret_cast<const float4*>(x + i * 16);
    float v[16];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float4 f = src[j];
      if constexpr (SILU) {
        const float4 u = reinterpret_cast<const float4*>(up + i * 16)[j];
        f = make_float4(silu(f.x) * u.x, silu(f.y) * u.y, silu(f.z) * u.z, silu(f.w) * u.w);
      }
      v[4 * j] = bf16_round(f.x), v[4 * j + 1] = bf16_round(f.y), v[4 * j + 2] = bf16_round(f.z), v[4 * j + 3] = bf16_round(f.w);
    }
    uint2 codes;
    const uint8_t sc = encode_block(v, gscale, codes);
    store_block(q, sf, tiled != 0, row, blk, K, k_atoms, codes, sc);
  }
}

// The DeltaNet mixer's gated RMSNorm in front of its out projection (src/core/kernels.cu:543-554) straight into NVFP4:
// y = core * rstd(core over the head's 128 values) * w * silu(z), rounded to BF16 and encoded.  A thread holds a block of 16
// values, eight neighbouring threads a head.
__global__ void __launch_bounds__(256)
    gated_norm_quant_nvfp4_kernel(const float* __restrict__ core, const float* __restrict__ z, const __nv_bfloat16* __restrict__ w, int M,
                                  int K, float eps, float gscale, uint8_t* __restrict__ q, uint8_t* __restrict__ sf, int tiled, int k_atoms) {
  const int bpr = K / 16;
  const size_t blocks = size_t(M) * bpr;
  const size_t span = (blocks + 31) / 32 * 32;  // whole warps stay in the loop together (the shuffles name every lane)
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < span; i += size_t(gridDim.x) * blockDim.x) {
    const bool real = i < blocks;
    const int row = int((real ? i : 0) / bpr), blk = int((real ? i : 0) % bpr);
    float v[16], ss = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 f = real ? reinterpret_cast<const float4*>(core + i * 16)[j] : make_float4(0.f, 0.f, 0.f, 0.f);
      v[4 * j] = f.x, v[4 * j + 1] = f.y, v[4 * j + 2] = f.z, v[4 * j + 3] = f.w;
      ss = fmaf(f.x, f.x, fmaf(f.y, f.y, fmaf(f.z, f.z, fmaf(f.w, f.w, ss))));
    }
    ss += __shfl_xor_sync(0xffffffffu, ss, 1), ss += __shfl_xor_sync(0xffffffffu, ss, 2), ss += __shfl_xor_sync(0xffffffffu, ss, 4);
    if (!real) continue;
    const float rstd = rsqrtf(ss / 128.f + eps);
    const int d0 = (blk % 8) * 16;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 zz = reinterpret_cast<const float4*>(z + i * 16)[j];
      const float zv[4] = {zz.x, zz.y, zz.z, zz.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) v[4 * j + e] = bf16_round(v[4 * j + e] * rstd * __bfloat162float(w[d0 + 4 * j + e]) * silu(zv[e]));
    }
    uint2 codes;
    const uint8_t sc = encode_block(v, gscale, codes);
    store_block(q, sf, tiled != 0, row, blk, K, k_atoms, codes, sc);
  }
}

// One CTA per row, a thread per block of 16 (H / 16 threads, whole warps): the sum of squares from float4s that are all
// requested before the first is used (per-thread fp32 partials in the order of the strided loop this replaces, then the block),
// then each thread normalizes, rounds and encodes its block, whose values the first pass left in L1.
__global__ void __launch_bounds__(1024)
    rmsnorm_quant_nvfp4_kernel(const float* __restrict__ x, const __nv_bfloat16* __restrict__ w, float* __restrict__ out, int H,
                               float eps, float gscale, uint8_t* __restrict__ q, uint8_t* __restrict__ sf, int tiled, int k_atoms) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  const float4* src = reinterpret_cast<const float4*>(x + size_t(row) * H);
  float ss = 0.f;
  for (int i0 = threadIdx.x; i0 < H / 4; i0 += 8 * blockDim.x) {
    float4 f[8];
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (i0 + k * int(blockDim.x) < H / 4) f[k] = src[i0 + k * blockDim.x];
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (i0 + k * int(blockDim.x) < H / 4) ss = fmaf(f[k].x, f[k].x, fmaf(f[k].y, f[k].y, fmaf(f[k].z, f[k].z, fmaf(f[k].w, f[k].w, ss))));
  }
  const float rstd = rsqrtf(block_sum(ss, red) / float(H) + eps);
  for (int blk = threadIdx.x; blk < H / 16; blk += blockDim.x) {
    float v[16];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 f = src[blk * 4 + j];
      const int c = blk * 16 + 4 * j;
      const uint2 wr = *reinterpret_cast<const uint2*>(w + c);
      const __nv_bfloat162 w01 = *reinterpret_cast<const __nv_bfloat162*>(&wr.x), w23 = *reinterpret_cast<const __nv_bfloat162*>(&wr.y);
      float4 n;
      n.x = f.x * rstd * (1.f + __low2float(w01)), n.y = f.y * rstd * (1.f + __high2float(w01));
      n.z = f.z * rstd * (1.f + __low2float(w23)), n.w = f.w * rstd * (1.f + __high2float(w23));
      if (out) reinterpret_cast<float4*>(out + size_t(row) * H)[blk * 4 + j] = n;
      v[4 * j] = bf16_round(n.x), v[4 * j + 1] = bf16_round(n.y), v[4 * j + 2] = bf16_round(n.z), v[4 * j + 3] = bf16_round(n.w);
    }
    uint2 codes;
    const uint8_t sc = encode_block(v, gscale, codes);
    store_block(q, sf, tiled != 0, row, blk, H, k_atoms, codes, sc);
  }
}

__global__ void weight_amax_kernel(const __nv_bfloat16* __restrict__ w, size_t n, unsigned* __restrict__ amax_bits) {
  float m = 0.f;
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x)
    m = fmaxf(m, fabsf(__bfloat162float(w[i])));
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) atomicMax(amax_bits, __float_as_uint(m));  // non-negative floats order like their bits
}

// One thread per block of 16 weights.  The code of a value is the number of midpoints below its magnitude, so a value on
// a midpoint takes the smaller of its two neighbours.
__global__ void __launch_bounds__(256)
    quant_weight_nvfp4_kernel(const __nv_bfloat16* __restrict__ w, int N, int K, const unsigned* __restrict__ amax_bits,
                              uint8_t* __restrict__ q, uint8_t* __restrict__ sf, int tiled, int k_atoms, float* __restrict__ scale2) {
  const float mx = __uint_as_float(*amax_bits);
  const float g = mx > 0.f ? mx / (448.f * 6.f) : 1.f;
  if (blockIdx.x == 0 && threadIdx.x == 0) *scale2 = g;
  const int bpr = K / 16;
  const size_t blocks = size_t(N) * bpr;
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < blocks; i += size_t(gridDim.x) * blockDim.x) {
    const int row = int(i / bpr), blk = int(i % bpr);
    float v[16], bm = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      v[j] = __bfloat162float(w[i * 16 + j]);
      bm = fmaxf(bm, fabsf(v[j]));
    }
    const uint8_t sc = to_e4m3(fmaxf(bm / 6.f / g, 0x1p-9f));
    const float s = from_e4m3(sc) * g;
    uint32_t words[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float a = fabsf(v[j] / s);
      uint32_t c = (a > 0.25f) + (a > 0.75f) + (a > 1.25f) + (a > 1.75f) + (a > 2.5f) + (a > 3.5f) + (a > 5.f);
      if (v[j] < 0.f && c > 0) c |= 8u;
      words[j >> 3] |= c << (4 * (j & 7));
    }
    store_block(q, sf, tiled != 0, row, blk, K, k_atoms, make_uint2(words[0], words[1]), sc);
  }
}

__global__ void sf_retile_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int rows, int bpr, int k_atoms, int to_tiled) {
  const size_t n = size_t(rows) * bpr;
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) {
    const size_t t = fp4_sf_offset(int(i / bpr), int(i % bpr), k_atoms);
    if (to_tiled) dst[t] = src[i];
    else dst[i] = src[t];
  }
}

int grid_for(size_t items) { return int(std::min<size_t>((items + 255) / 256, 148 * 16)); }

bool shape_ok(int rows, int K, const char* what) {
  if (rows < 1 || K < 16 || K % 16) {
    set_error(std::string(what) + ": rows must be positive and K a positive multiple of 16");
    return false;
  }
  return true;
}

}  // namespace

static std::atomic<int> g_pair_mode{0};
int fp4_set_pair_mode(int mode) { return g_pair_mode.exchange(mode); }

int fp4_init() {
  static std::once_flag once;
  static int rc = LING_B200_OK;
  std::call_once(once, [] {
    if (cudaFuncSetAttribute(gemm_nvfp4_tcgen05_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSmemBytes)) != cudaSuccess ||
        cudaFuncSetAttribute(gemm_nvfp4_tcgen05_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSmemBytes)) != cudaSuccess ||
        cudaFuncSetAttribute(gemm_nvfp4_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kPairSmemBytes)) != cudaSuccess ||
        cudaFuncSetAttribute(gemm_nvfp4_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kPairSmemBytes)) != cudaSuccess) {
      set_error("cudaFuncSetAttribute failed for the NVFP4 GEMM");
      rc = LING_B200_ERR_CUDA;
    }
  });
  return rc;
}

int make_fp4_map(Fp4Operand& o) {
  if (o.K % 32) {
    set_error("NVFP4 operand: K must be a multiple of 32 (16-byte rows for the tensor map)");
    return LING_B200_ERR_ARG;
  }
  if (const int r = encode_tile_map(&o.map, o.codes, uint64_t(o.K / 2), uint64_t(o.rows), 128)) return r;
  return encode_linear_map(&o.sf_map, o.sf, uint64_t(fp4_k_atoms(o.K)) * 512, uint64_t(round_up(o.rows, kFp4TileN) / 128), kSfGroup);
}

int fp4_gemm_launch(const Fp4GemmCall& c, cudaStream_t stream) {
  const Fp4Operand &X = *c.X, &W = *c.W;
  const bool fused = c.W2 != nullptr;
  if (X.K != W.K || W.rows % 128 || X.K % 128 || (fused && (c.W2->K != W.K || c.W2->rows != W.rows))) {
    set_error("NVFP4 GEMM: N % 128 and K % 128 must be 0 and the operands' K must agree");
    return LING_B200_ERR_ARG;
  }
  if (X.rows < 1) return LING_B200_OK;
  if (const int r = fp4_init()) return r;
  GemmArgs p{};
  p.sfa = X.sf, p.sfb0 = W.sf, p.sfb1 = fused ? c.W2->sf : W.sf;
  p.M = X.rows, p.N = W.rows;
  p.k_stages = ceil_div(X.K, kFp4StageK);
  p.tiles_m = ceil_div(X.rows, kFp4TileM);
  p.tiles_n = fused ? W.rows / 128 : ceil_div(W.rows, kFp4TileN);
  p.b_step = fused ? 128 : 256, p.b1_off = fused ? 0 : 128;
  p.g_mul = fused ? 1 : 2, p.g1_off = fused ? 0 : 1;
  p.alpha = c.alpha, p.alpha2 = c.alpha2, p.gscale_out = c.gscale_out;
  p.y = c.y, p.ldy = c.ldy, p.accumulate = c.accumulate ? 1 : 0;
  p.q_out = c.q_out, p.sf_out = c.sf_out, p.sf_out_tiled = c.sf_out_tiled ? 1 : 0, p.out_atoms = fp4_k_atoms(W.rows);
  p.err_flag = c.err_flag, p.stats = c.stats;
  if (!fused && (c.ldy % 4 || (reinterpret_cast<uintptr_t>(c.y) & 15))) {
    set_error("NVFP4 GEMM: y must be 16-byte aligned and ldy a multiple of 4");
    return LING_B200_ERR_ARG;
  }
  int sms = 148;
  int dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const bool pair = c.pair >= 0 ? c.pair > 0 : g_pair_mode.load() > 0;
  if (pair) {
    p.tiles_m = ceil_div(X.rows, 2 * kFp4TileM);
    const int pairs = std::max(1, std::min((c.ctas > 0 ? c.ctas : sms) / 2, p.tiles_m * p.tiles_n));
    const Fp4Operand& B1 = fused ? *c.W2 : W;
    LB_CUDA(launch_kernel_cluster(fused ? gemm_nvfp4_pair_kernel<true> : gemm_nvfp4_pair_kernel<false>, dim3(2 * pairs), dim3(kThreads),
                                  kPairSmemBytes, 2, stream, X.map, W.map, B1.map, X.sf_map, W.sf_map, B1.sf_map, p));
    LB_LAUNCH("gemm_nvfp4_pair_kernel");
    return LING_B200_OK;
  }
  const int ctas = std::min(c.ctas > 0 ? c.ctas : sms, p.tiles_m * p.tiles_n);
  if (fused)
    gemm_nvfp4_tcgen05_kernel<true><<<ctas, kThreads, kSmemBytes, stream>>>(X.map, W.map, c.W2->map, p);
  else
    gemm_nvfp4_tcgen05_kernel<false><<<ctas, kThreads, kSmemBytes, stream>>>(X.map, W.map, W.map, p);
  LB_LAUNCH("gemm_nvfp4_tcgen05_kernel");
  return LING_B200_OK;
}

int fp4_quant_act_launch(const float* x, const float* up, int M, int K, float gscale, uint8_t* q, uint8_t* sf, bool tiled,
                         cudaStream_t stream) {
  if (!shape_ok(M, K, "quant_act_nvfp4")) return LING_B200_ERR_ARG;
  const int g = grid_for(size_t(M) * (K / 16));
  if (up) quant_act_nvfp4_kernel<true><<<g, 256, 0, stream>>>(x, up, M, K, gscale, q, sf, tiled ? 1 : 0, fp4_k_atoms(K));
  else quant_act_nvfp4_kernel<false><<<g, 256, 0, stream>>>(x, nullptr, M, K, gscale, q, sf, tiled ? 1 : 0, fp4_k_atoms(K));
  LB_LAUNCH("quant_act_nvfp4_kernel");
  return LING_B200_OK;
}

int fp4_gated_norm_quant_launch(const float* core, const float* z, const __nv_bfloat16* w, int M, int K, float eps, float gscale,
                                uint8_t* q, uint8_t* sf, bool tiled, cudaStream_t stream) {
  if (!shape_ok(M, K, "gated_norm_quant_nvfp4") || K % 128 != 0) return LING_B200_ERR_ARG;
  gated_norm_quant_nvfp4_kernel<<<grid_for(size_t(M) * (K / 16)), 256, 0, stream>>>(core, z, w, M, K, eps, gscale, q, sf, tiled ? 1 : 0,
                                                                                   fp4_k_atoms(K));
  LB_LAUNCH("gated_norm_quant_nvfp4_kernel");
  return LING_B200_OK;
}

int fp4_rmsnorm_quant_launch(const float* x, const __nv_bfloat16* w, float* out, int M, int H, float eps, float gscale, uint8_t* q,
                             uint8_t* sf, bool tiled, cudaStream_t stream) {
  if (!shape_ok(M, H, "rmsnorm_quant")) return LING_B200_ERR_ARG;
  const int threads = std::min(1024, std::max(64, (H / 16 + 31) / 32 * 32));
  rmsnorm_quant_nvfp4_kernel<<<M, threads, 0, stream>>>(x, w, out, H, eps, gscale, q, sf, tiled ? 1 : 0, fp4_k_atoms(H));
  LB_LAUNCH("rmsnorm_quant_nvfp4_kernel");
  return LING_B200_OK;
}

int fp4_quant_weight_launch(const __nv_bfloat16* w, int N, int K, uint8_t* q, uint8_t* sf, bool tiled, float* scale2,
                            unsigned* amax_bits, cudaStream_t stream) {
  if (!shape_ok(N, K, "quantize_nvfp4")) return LING_B200_ERR_ARG;
  weight_amax_kernel<<<grid_for(size_t(N) * K / 8), 256, 0, stream>>>(w, size_t(N) * K, amax_bits);
  LB_LAUNCH("weight_amax_kernel");
  quant_weight_nvfp4_kernel<<<grid_for(size_t(N) * (K / 16)), 256, 0, stream>>>(w, N, K, amax_bits, q, sf, tiled ? 1 : 0,
                                                                               fp4_k_atoms(K), scale2);
  LB_LAUNCH("quant_weight_nvfp4_kernel");
  return LING_B200_OK;
}

int fp4_tensor_peak_launch(int ctas, int iters, int mode, int* err_flag, cudaStream_t stream) {
  constexpr int smem = kABytes + kBBytes + 3 * kSfGroup + 1024 + 128;
  static std::once_flag once;
  static cudaError_t attr = cudaSuccess;
  std::call_once(once, [] { attr = cudaFuncSetAttribute(fp4_tensor_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); });
  LB_CUDA(attr);
  fp4_tensor_peak_kernel<<<ctas, 128, smem, stream>>>(iters, mode, err_flag);
  LB_LAUNCH("fp4_tensor_peak_kernel");
  return LING_B200_OK;
}

int fp4_sf_tile_launch(const uint8_t* rowmajor, uint8_t* tiled, int rows, int K, cudaStream_t stream) {
  sf_retile_kernel<<<grid_for(size_t(rows) * (K / 16)), 256, 0, stream>>>(rowmajor, tiled, rows, K / 16, fp4_k_atoms(K), 1);
  LB_LAUNCH("sf_retile_kernel");
  return LING_B200_OK;
}
int fp4_sf_untile_launch(const uint8_t* tiled, uint8_t* rowmajor, int rows, int K, cudaStream_t stream) {
  sf_retile_kernel<<<grid_for(size_t(rows) * (K / 16)), 256, 0, stream>>>(tiled, rowmajor, rows, K / 16, fp4_k_atoms(K), 0);
  LB_LAUNCH("sf_retile_kernel");
  return LING_B200_OK;
}

}  // namespace lb
