// attention_tc.cu -- tree-masked attention over the paged FP8 cache on the 5th-generation tensor cores (sm_100a).
//
// The same flash-decoding contract as attention_kernel in kernels.cu (work items per (sequence, kv head, 512-key chunk),
// per (chunk slot, query row) the unnormalized output and (max, denominator), merged by attn_combine_kernel), rebuilt
// around tcgen05.mma kind::f16 with the accumulators in TMEM:
//
//   item     (sequence, kv head, key chunk, 128 query rows): the query rows of a kv head are (token row, q head of the
//            group) pairs; 128 rows are the MMA's M, one TMEM lane per row.
//   operands FP16 in 128B-swizzled K-major shared-memory tiles, written by the CTA's own threads: Q from global memory,
//            K and V converted once per 64-key tile from the E4M3 codes that cp.async staged (cvt.f16x2.e4m3x2; every
//            converted value then serves all 128 rows), P by the softmax threads.
//   S = Q.K^T for a sub-chunk of 256 keys sits in TMEM columns 0..255 (four 64-key tiles, D/16 MMAs of N = 64 each),
//            so the softmax of a sub-chunk sees its whole row: exact maximum, no rescaling between tiles.
//   softmax  thread = (query row = TMEM lane, half of the sub-chunk's keys): two passes over its 128 scores (tcgen05.ld),
//            per-position K scale (log2 domain) and the mask applied in fp32, probabilities times the V scale written
//            as FP16 into the A tiles; the two halves of a row meet through shared memory.
//   O += P.V into TMEM columns 256..256+D (MMA N = D); between the two sub-chunks of a chunk the rows whose maximum
//            grew are rescaled in TMEM (tcgen05.ld / tcgen05.st).
//   overlap  in the operand loops warp 0 only issues MMAs and warps 1-7 stage and convert; operand buffers are double, so
//            the tensor core works on tile t while tile t + 1 is converted (named barriers between the two roles,
//            tcgen05.commit on one mbarrier per buffer); cp.async runs two to three tiles ahead.
// Every wait is bounded; a wait that runs out records a code in the device error word and the CTA frees its TMEM and
// leaves.  No TMA, no cluster, no multicast.
#include "kernels.h"
#include "tc.cuh"

namespace lb {
namespace {
using namespace tc;

constexpr int kTcRows = kAttnTcRows;  // query rows per item = the MMA's M
constexpr int kTcKeys = 64;      // keys per operand tile
constexpr int kTcSub = 256;      // keys per sub-chunk = S columns in TMEM
constexpr int kTcPages = kAttnChunk / 16 + 4;  // page ids of one chunk (pages hold 16 positions or more; a tail chunk starts unaligned)
constexpr int kTcThreads = 256;  // warps 0-3 also run the softmax (one per TMEM lane quarter)
constexpr int kTcStage = 4;      // 16 KiB-class slots of the FP8 staging ring
constexpr float kLog2e = 1.4426950408889634f, kLn2 = 0.6931471805599453f;

__device__ __forceinline__ void cp16(void* dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp4(void* dst, const void* src, int src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
// 2^x for x <= 0 (also -inf -> 0); results below the normal range flush to zero, which a probability may
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t h2_bits(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}
// 16 E4M3 codes -> 16 FP16 values (two 16-byte chunks), codes at or past `valid` cleared first
__device__ __forceinline__ void convert16(const uint4& in, int valid, uint4& lo, uint4& hi) {
  uint32_t w[4] = {in.x, in.y, in.z, in.w};
  if (valid < 16) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int left = valid - 4 * i;  // valid bytes of word i
      w[i] = left >= 4 ? w[i] : left <= 0 ? 0u : (w[i] & ((1u << (8 * left)) - 1u));
    }
  }
  lo = make_uint4(e4m3x2_to_h2(uint16_t(w[0])), e4m3x2_to_h2(uint16_t(w[0] >> 16)), e4m3x2_to_h2(uint16_t(w[1])),
                  e4m3x2_to_h2(uint16_t(w[1] >> 16)));
  hi = make_uint4(e4m3x2_to_h2(uint16_t(w[2])), e4m3x2_to_h2(uint16_t(w[2] >> 16)), e4m3x2_to_h2(uint16_t(w[3])),
                  e4m3x2_to_h2(uint16_t(w[3] >> 16)));
}

// Named barriers of the operand loops: id 1 = the staging/converting warps among themselves; ids 2 and 3 (by operand
// buffer) = "tile converted": the converting warps arrive, the issuing warp waits.  Counts are whole warps.
constexpr int kTcWorkers = kTcThreads - 32;  // warps 1-7 stage and convert; warp 0 issues the MMAs
__device__ __forceinline__ void named_sync(int id, int count) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory"); }
__device__ __forceinline__ void named_arrive(int id, int count) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory"); }

template <int D>
struct TcSmem {
  static constexpr int KB = D / 64;                        // 128-byte K blocks of a D-wide FP16 row
  static constexpr size_t kQV = size_t(D) * 256;           // Q [KB][128][128 B]  /  V^T FP16 x 2 [D][128 B]
  static constexpr size_t kKP = kQV > 65536 ? kQV : 65536; // K FP16 x 2 [KB][64][128 B]  /  P [4][128][128 B]
  static constexpr size_t kSlot = size_t(D) * 64;          // one staged FP8 tile: K [64][D] or V [D][64]
  static constexpr size_t kStageBytes = kTcStage * kSlot;
  static constexpr size_t kBytes = kQV + kKP + kStageBytes + 5 * kTcSub * 4 /* scales, per-key coefficients */ +
                                   2 * kTcRows * 4 /* halves' exchange */ + 64 /* barriers */ + 1024 /* alignment */;
};

template <int D, int G>
__global__ void __launch_bounds__(kTcThreads, 1)
    attention_tc_kernel(const __half* __restrict__ q, StepBuffers sb, ModelDims d, int al, KvPoolDev kv, float* __restrict__ part_o,
                        float* __restrict__ part_ml, int chunk_slots, PrefetchPlan plan, unsigned long long* stamps) {
  // stamps (debugging aid, or nullptr): %globaltimer of block 0's first item: [0] entry, [1] set-up done, then per sub-chunk
  // [2 + 4 sub ..]: Q loaded, S complete, softmax done, O issued; [10] item stored
  const bool stamp = stamps != nullptr && blockIdx.x == 0 && threadIdx.x == 0;
  if (stamp) stamps[0] = global_ns();
  pdl_sync();  // first statement: see common.cuh
  using L = TcSmem<D>;
  constexpr int KB = L::KB, RMAX = kTreeRows * G;
  constexpr uint32_t kScol = 0, kOcol = kTcSub;  // TMEM columns of S and O
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* qv = smem;                   // Q tiles, later the two V^T tiles
  uint8_t* kp = qv + L::kQV;            // the two K tiles, later the four P tiles
  uint8_t* stage = kp + L::kKP;         // FP8 staging ring
  float* ksc = reinterpret_cast<float*>(stage + L::kStageBytes);  // [256] K scales of the sub-chunk
  float* vsc = ksc + kTcSub;                                      // [256]
  float2* kcoef = reinterpret_cast<float2*>(vsc + kTcSub);        // [256] per key: score scale (log2 domain), additive mask
  float* vcoef = reinterpret_cast<float*>(kcoef + kTcSub);        // [256] per key: V scale x kPScale
  float* redm = vcoef + kTcSub;                                   // [2][128] the halves' row maxima / denominators
  uint64_t* bar = reinterpret_cast<uint64_t*>(redm + 2 * kTcRows);  // [2] MMA completion, one per operand buffer
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 2);
  __shared__ int cbase[LING_B200_MAX_SEQS + 1], ibase[LING_B200_MAX_SEQS + 1];
  __shared__ volatile int failed;  // a bounded wait ran out: no further waits, no output; every thread still takes every barrier
  __shared__ int chunk_sh;         // keys per chunk of this step (attn_chunk_keys)
  __shared__ int pages_sm[2][kTcPages];
  int items_done = 0;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool worker = warp > 0;  // operand loops: warps 1-7 stage and convert, warp 0 issues (all eight run the softmax)
  const int wtid = tid - 32;
  const int nseq = *sb.n_seqs;
  if (tid == 0) {
    const int chunk = attn_chunk_keys(sb, nseq, d.Hkv, G, kTcRows, int(gridDim.x));
    chunk_sh = chunk;
    int cb = 0, ib = 0;
    for (int s = 0; s < nseq; ++s) {
      cbase[s] = cb, ibase[s] = ib;
      const int nch = (sb.seqs[s].pos + chunk - 1) / chunk + 1;
      const int nrg = (sb.seqs[s].n_rows * G + kTcRows - 1) / kTcRows;
      cb += nch, ib += d.Hkv * nch * nrg;
    }
    cbase[nseq] = cb, ibase[nseq] = ib;
    mbar_init(&bar[0], 1);
    mbar_init(&bar[1], 1);
    failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int chunk = chunk_sh;
  const float inv_sqrt_d = rsqrtf(float(D));
  const int pt = d.page_tokens, lp = 31 - __clz(pt), pmask = pt - 1;
  if (stamp) stamps[1] = global_ns();
  uint32_t mma_count = 0;  // MMA groups committed so far (same value in every thread): group n uses bar[n & 1]

  // Waits until MMA group n has completed (n < mma_count).  Bounded; on expiry every thread sees `failed`.
  auto wait_group = [&](uint32_t n) {
    if (failed) return;
    if (!mbar_wait(&bar[n & 1], (n >> 1) & 1, nullptr)) {
      dev_fail(sb.err, kDevWaitTmemFull);
      failed = 1;
    }
    tc_fence_after();
  };

  // a CTA without an item asks the weights of the GEMMs behind this kernel into L2 (HBM is nearly idle while it runs)
  if (int(blockIdx.x) >= ibase[nseq]) prefetch_plan_share(plan, int(blockIdx.x) - ibase[nseq], int(gridDim.x) - ibase[nseq]);
  for (int item = blockIdx.x; item < ibase[nseq]; item += gridDim.x) {
    int s = 0;
    while (ibase[s + 1] <= item) ++s;
    const SeqDev sq = sb.seqs[s];
    const int nch = (sq.pos + chunk - 1) / chunk + 1;
    const int nrg = (sq.n_rows * G + kTcRows - 1) / kTcRows;
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
    const int R = sq.n_rows * G, r_begin = rg * kTcRows, r0 = sb.row0[s];
    const int* table = kv.tables + size_t(sq.slot) * d.max_pages;
    const uint8_t* kcodes = kv.codes + kv_slot_index(d, al, 0, hk, 0, 0) * D;
    const uint8_t* vcodes = kv.codes + kv_slot_index(d, al, 1, hk, 0, 0) * D;
    const float* kscales = kv.scales + kv_slot_index(d, al, 0, hk, 0, 0);
    const float* vscales = kv.scales + kv_slot_index(d, al, 1, hk, 0, 0);
    // The chunk's page ids, looked up once per item into shared memory (two sets, alternating by item, so that a thread
    // still staging the previous item's last tile is not overtaken): a lookup per staged tile was a dependent global load
    // ahead of every tile's copies.  The first use is behind the block barrier that opens the sub-chunk loop.
    int* pages = pages_sm[items_done & 1];
    const int page0 = key_base >> lp;
    for (int i = tid; i <= ((key_base + max(key_hi, 1) - 1) >> lp) - page0 && i < kTcPages; i += kTcThreads) {
      const int page = table[page0 + i];
      pages[i] = (page < 0 || page > d.pool_pages) ? 0 : page;  // an unmapped position lands in the reserved page
    }
    ++items_done;
    auto page_of = [&](int pos) { return pages[min((pos >> lp) - page0, kTcPages - 1)]; };
    // cp.async of one 64-key tile's codes into a staging slot: K as [key][D], V as [D][64 keys]; one commit group each.
    // A position at or past key_hi is zero-filled.
    // K: two threads per key (one page lookup each), eight 16-byte pieces of the key's D bytes per thread for D = 256
    auto stage_k = [&](int k0, uint8_t* dst, bool scales, int sc_off) {
      constexpr int PK = D / 16, TPK = PK >= 8 ? 2 : 1, PPT = PK / TPK;  // pieces per key, threads per key, pieces per thread
      if (wtid < kTcKeys * TPK) {
        const int key = wtid / TPK, part0 = (wtid % TPK) * PPT;
        const bool valid = k0 + key < key_hi;
        const int pos = key_base + k0 + key;
        const size_t at = valid ? (size_t(page_of(pos)) << lp) + (pos & pmask) : 0;
        const uint8_t* src = kcodes + at * D + part0 * 16;
        uint8_t* to = dst + size_t(key) * D + part0 * 16;
#pragma unroll
        for (int i = 0; i < PPT; ++i) cp16(to + i * 16, src + i * 16, valid ? 16 : 0);
        if (scales && part0 == 0) {
          cp4(ksc + sc_off + key, kscales + at, valid ? 4 : 0);
          cp4(vsc + sc_off + key, vscales + at, valid ? 4 : 0);
        }
      }
      cp_commit();
    };
    // V: a thread's 16 positions (one page lookup) are the same for all its dims
    auto stage_v = [&](int k0, uint8_t* dst) {
      static_assert(kTcWorkers % 4 == 0, "a thread keeps its 16-position piece across dims");
      const int kc = (wtid & 3) * 16;
      const bool valid = k0 + kc < key_hi;
      const int pos = key_base + k0 + kc;
      const uint8_t* src = vcodes + (valid ? (size_t(page_of(pos)) << lp) * D + (pos & pmask) : 0);
      for (int dd = wtid >> 2; dd < D; dd += kTcWorkers / 4)
        cp16(dst + size_t(dd) * 64 + kc, src + (valid ? size_t(dd) << lp : 0), valid ? 16 : 0);
      cp_commit();
    };

    float m_run = -INFINITY, l_run = 0.f;  // this thread's row: running maximum (log2 domain) and its half of the denominator
    const int q4 = warp & 3, half = warp >> 2;
    const int row = q4 * 32 + lane;        // row inside the item = TMEM lane
    uint32_t anc = 0xffffffffu;
    if (tail) anc = r_begin + row < R ? sb.anc[r0 + (r_begin + row) / G] : 0u;
    const int nsub = (key_hi + kTcSub - 1) / kTcSub;

    for (int sub = 0; sub < nsub; ++sub) {
      const int sub0 = sub * kTcSub;                                   // first key of the sub-chunk inside the chunk
      const int nt = min(kTcSub / kTcKeys, (key_hi - sub0 + kTcKeys - 1) / kTcKeys);  // its 64-key tiles
      // everything of the previous sub-chunk (and item) has been consumed: all MMA groups are complete
      if (mma_count >= 1) wait_group(mma_count - 1);
      if (mma_count >= 2) wait_group(mma_count - 2);
      __syncthreads();
      // ---- Q into its swizzled tiles by cp.async (rows past R zero-filled), K tiles 0 and 1 on their way -- unless the
      // previous sub-chunk's P.V loop already sent for them
      const bool k_prefetched = sub > 0;  // (a sub-chunk with a successor always has four tiles)
      if (worker) {
        for (int idx = wtid; idx < kTcRows * (D / 8); idx += kTcWorkers) {
          const int r = idx / (D / 8), piece = idx % (D / 8), rr = r_begin + r;
          const __half* src = rr < R ? q + (size_t(r0 + rr / G) * d.Hq + hk * G + rr % G) * D + piece * 8 : q;
          cp16(qv + size_t(piece >> 3) * (kTcRows * 128) + sw128_offset(r, piece & 7), src, rr < R ? 16 : 0);
        }
        if (!k_prefetched) {
          stage_k(sub0, stage, true, 0);  // one group with the Q copies
          if (nt > 1) stage_k(sub0 + kTcKeys, stage + L::kSlot, true, kTcKeys);
          else cp_commit();
          if (nt > 2) stage_k(sub0 + 2 * kTcKeys, stage + 2 * L::kSlot, true, 2 * kTcKeys);
          else cp_commit();
        } else {
          cp_commit();  // the Q copies alone, after the three K groups
        }
      }
      if (stamp && item == int(blockIdx.x) && sub < 2) stamps[2 + 4 * sub] = global_ns();
      // ---- S = Q.K^T, tile by tile; staging slot t & 3 holds K tile t
      const uint32_t first_qk = mma_count;
      for (int t = 0; t < nt; ++t) {
        uint8_t* kt = kp + size_t(t & 1) * (size_t(KB) * kTcKeys * 128);
        if (worker) {
          // tile t's group has landed (this thread's copies): the copies run three tiles ahead, and tile t + 3 is sent for
          // after the barrier, when every thread is done with the staging slot it reuses (tile t - 1's).  With prefetched K
          // tiles the Q group is the youngest.
          if (t == 0 && k_prefetched) cp_wait<0>();
          else cp_wait<2>();
          named_sync(1, kTcWorkers);
          if (t + 3 < nt) stage_k(sub0 + (t + 3) * kTcKeys, stage + size_t((t + 3) & 3) * L::kSlot, true, (t + 3) * kTcKeys);
          else cp_commit();
          if (mma_count >= first_qk + 2) wait_group(mma_count - 2);  // the MMAs that read this K buffer two tiles ago
          const uint8_t* src = stage + size_t(t & 3) * L::kSlot;
          for (int idx = wtid; idx < kTcKeys * (D / 16); idx += kTcWorkers) {
            const int key = idx / (D / 16), part = idx % (D / 16);
            uint4 lo, hi;
            convert16(*reinterpret_cast<const uint4*>(src + size_t(key) * D + part * 16), 16, lo, hi);
            uint8_t* blk = kt + size_t(part >> 2) * (kTcKeys * 128);
            *reinterpret_cast<uint4*>(blk + sw128_offset(key, (part & 3) * 2)) = lo;
            *reinterpret_cast<uint4*>(blk + sw128_offset(key, (part & 3) * 2 + 1)) = hi;
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          named_arrive(2 + (t & 1), kTcThreads);
        } else {
          named_sync(2 + (t & 1), kTcThreads);  // the tile (and, at t = 0, Q) is in shared memory, fenced for the tensor core
          if (lane == 0) {
            tc_fence_after();
            constexpr uint32_t idesc = umma_idesc_f16(kTcKeys);
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) {
              const uint64_t adesc = umma_desc_sw128(smem_u32(qv + size_t(kb) * (kTcRows * 128)));
              const uint64_t bdesc = umma_desc_sw128(smem_u32(kt + size_t(kb) * (kTcKeys * 128)));
#pragma unroll
              for (int k = 0; k < 4; ++k)  // K = 16 halves = 32 bytes per instruction
                umma_f16(tmem_base + kScol + uint32_t(t * kTcKeys), adesc + uint64_t(k * 2), bdesc + uint64_t(k * 2), idesc,
                         (kb | k) ? 1u : 0u);
            }
            umma_commit(&bar[mma_count & 1]);
          }
          __syncwarp();
        }
        ++mma_count;
      }
      // ---- the V tiles start moving while the softmax runs; staging slots are free once their K tile was converted
      cp_wait<0>();
      __syncthreads();
      if (worker) {
        stage_v(sub0, stage);
        if (nt > 1) stage_v(sub0 + kTcKeys, stage + L::kSlot);
        else cp_commit();
        if (nt > 2) stage_v(sub0 + 2 * kTcKeys, stage + 2 * L::kSlot);
        else cp_commit();
      }
      // per key of the sub-chunk: score scale in the log2 domain and an additive mask (0, or -inf outside the chunk's
      // keys), and the V scale the probabilities carry
      for (int k = tid; k < nt * kTcKeys; k += kTcThreads) {
        const int kk = sub0 + k;
        kcoef[k] = make_float2(ksc[k] * inv_sqrt_d * kLog2e, (kk >= key_lo && kk < key_hi) ? 0.f : -INFINITY);
        vcoef[k] = vsc[k] * kPScale;
      }
      // every S tile is complete
      wait_group(mma_count - 1);
      if (mma_count >= first_qk + 2) wait_group(mma_count - 2);
      __syncthreads();
      if (stamp && item == int(blockIdx.x) && sub < 2) stamps[3 + 4 * sub] = global_ns();
      // ---- softmax of the sub-chunk: a thread per (row, half of the keys): warps w and w + 4 share TMEM lane quarter w,
      // the first takes keys 0..127, the second 128..255; a quarter without a real row does nothing
      const int c_lo = half * 4, c_hi = min(c_lo + 4, 2 * nt);  // this thread's 32-key groups
      const bool live = r_begin + q4 * 32 < R;                 // warp-uniform
      const uint32_t taddr = tmem_base + (uint32_t(q4 * 32) << 16) + kScol;
      float mx = -INFINITY;
      if (live) {
        for (int c = c_lo; c < c_hi; ++c) {
          uint32_t v[32];
          tmem_ld32(taddr + c * 32, v);
          tmem_ld_wait();
          if (!tail) {
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              const float4 kc = *reinterpret_cast<const float4*>(kcoef + c * 32 + j);  // two keys
              mx = fmaxf(mx, fmaxf(fmaf(__uint_as_float(v[j]), kc.x, kc.y), fmaf(__uint_as_float(v[j + 1]), kc.z, kc.w)));
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float2 kc = kcoef[c * 32 + j];
              const bool vis = (anc >> ((sub0 + c * 32 + j - key_lo) & 31)) & 1u;
              mx = fmaxf(mx, vis ? fmaf(__uint_as_float(v[j]), kc.x, kc.y) : -INFINITY);
            }
          }
        }
        redm[half * kTcRows + row] = mx;
      }
      __syncthreads();
      float corr = 1.f;
      if (live) {
        const float mnew = fmaxf(m_run, fmaxf(redm[row], redm[kTcRows + row]));
        const float muse = mnew == -INFINITY ? 0.f : mnew;
        corr = exp2f(m_run - muse);  // 2^-inf = 0 for a row that has seen nothing yet
        m_run = mnew;
        // rows whose maximum grew: rescale the output accumulated over the earlier sub-chunk (each warp half of the columns)
        if (sub > 0 && __any_sync(0xffffffffu, corr != 1.f)) {
          const uint32_t oaddr = tmem_base + (uint32_t(q4 * 32) << 16) + kOcol;
#pragma unroll 1
          for (int c = half; c < D / 32; c += 2) {
            uint32_t v[32];
            tmem_ld32(oaddr + c * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * corr);
            tmem_st32(oaddr + c * 32, v);
          }
          tmem_st_wait();
        }
        float lsum = 0.f;
        for (int c = c_lo; c < c_hi; ++c) {
          uint32_t v[32];
          tmem_ld32(taddr + c * 32, v);
          tmem_ld_wait();
          uint32_t pk[16];
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const float4 k01 = *reinterpret_cast<const float4*>(kcoef + c * 32 + j);      // keys j, j + 1
            const float4 k23 = *reinterpret_cast<const float4*>(kcoef + c * 32 + j + 2);  // keys j + 2, j + 3
            const float4 vc = *reinterpret_cast<const float4*>(vcoef + c * 32 + j);
            float s2[4] = {fmaf(__uint_as_float(v[j]), k01.x, k01.y), fmaf(__uint_as_float(v[j + 1]), k01.z, k01.w),
                           fmaf(__uint_as_float(v[j + 2]), k23.x, k23.y), fmaf(__uint_as_float(v[j + 3]), k23.z, k23.w)};
            if (tail) {
#pragma unroll
              for (int e = 0; e < 4; ++e)
                if (!((anc >> ((sub0 + c * 32 + j + e - key_lo) & 31)) & 1u)) s2[e] = -INFINITY;
            }
            const float p0 = ex2_approx(s2[0] - muse), p1 = ex2_approx(s2[1] - muse), p2 = ex2_approx(s2[2] - muse),
                        p3 = ex2_approx(s2[3] - muse);
            lsum += (p0 + p1) + (p2 + p3);
            pk[j >> 1] = h2_bits(p0 * vc.x, p1 * vc.y);
            pk[(j >> 1) + 1] = h2_bits(p2 * vc.z, p3 * vc.w);
          }
          // 32 keys = four 16-byte chunks of this row in P tile c / 2
          uint8_t* ptile = kp + size_t(c >> 1) * (kTcRows * 128);
#pragma unroll
          for (int x = 0; x < 4; ++x)
            *reinterpret_cast<uint4*>(ptile + sw128_offset(row, (c & 1) * 4 + x)) = make_uint4(pk[4 * x], pk[4 * x + 1], pk[4 * x + 2], pk[4 * x + 3]);
        }
        l_run = l_run * corr + lsum;  // this thread's half of the keys; the halves are added at the end
        tc_fence_before();
      }
      if (stamp && item == int(blockIdx.x) && sub < 2) stamps[4 + 4 * sub] = global_ns();
      // ---- O += P.V, tile by tile; staging slot t & 3 holds V tile t, the Q region the two V^T operand tiles
      const uint32_t first_pv = mma_count;
      // the P tiles are written and fenced, the S reads are done
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncthreads();
      for (int t = 0; t < nt; ++t) {
        uint8_t* vt = qv + size_t(t & 1) * (size_t(D) * 128);
        if (worker) {
          cp_wait<2>();
          named_sync(1, kTcWorkers);
          // after the barrier tile t - 1's slot is free: V tile t + 3, or the next sub-chunk's K tiles 0..2 (its scales go to
          // ksc / vsc, which the softmax no longer reads: it copied them into kcoef / vcoef)
          if (t + 3 < nt) stage_v(sub0 + (t + 3) * kTcKeys, stage + size_t((t + 3) & 3) * L::kSlot);
          else if (sub + 1 < nsub && t >= 1) stage_k(sub0 + kTcSub + (t - 1) * kTcKeys, stage + size_t(t - 1) * L::kSlot, true, (t - 1) * kTcKeys);
          else cp_commit();
          if (mma_count >= first_pv + 2) wait_group(mma_count - 2);
          const uint8_t* src = stage + size_t(t & 3) * L::kSlot;
          const int tile0 = sub0 + t * kTcKeys;
          for (int idx = wtid; idx < D * 4; idx += kTcWorkers) {
            const int dd = idx >> 2, piece = idx & 3;
            uint4 lo, hi;
            convert16(*reinterpret_cast<const uint4*>(src + size_t(dd) * 64 + piece * 16), key_hi - (tile0 + piece * 16), lo, hi);
            *reinterpret_cast<uint4*>(vt + sw128_offset(dd, piece * 2)) = lo;
            *reinterpret_cast<uint4*>(vt + sw128_offset(dd, piece * 2 + 1)) = hi;
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          named_arrive(2 + (t & 1), kTcThreads);
        } else {
          named_sync(2 + (t & 1), kTcThreads);
          if (lane == 0) {
            tc_fence_after();
            constexpr uint32_t idesc = umma_idesc_f16(D);
            const uint64_t adesc = umma_desc_sw128(smem_u32(kp + size_t(t) * (kTcRows * 128)));
            const uint64_t bdesc = umma_desc_sw128(smem_u32(vt));
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_f16(tmem_base + kOcol, adesc + uint64_t(k * 2), bdesc + uint64_t(k * 2), idesc, (sub | t | k) ? 1u : 0u);
            umma_commit(&bar[mma_count & 1]);
          }
          __syncwarp();
        }
        ++mma_count;
      }
      if (stamp && item == int(blockIdx.x) && sub < 2) stamps[5 + 4 * sub] = global_ns();
    }
    cp_wait<0>();
    // ---- the item's output: unnormalized sums and (max, denominator) per real row
    if (mma_count >= 1) wait_group(mma_count - 1);
    if (mma_count >= 2) wait_group(mma_count - 2);
    if (half == 1) redm[row] = l_run;  // the second half's share of the denominator
    __syncthreads();
    // O goes through shared memory (everything there is dead now) so that the global stores are whole rows: a thread holds
    // one row, and 32 rows a kilobyte apart per store instruction would serialize in the load/store unit
    float* osm = reinterpret_cast<float*>(smem);  // [128][D + 4]
    if (!failed && r_begin + q4 * 32 < R) {
      const int rr = r_begin + row;
      const uint32_t oaddr = tmem_base + (uint32_t(q4 * 32) << 16) + kOcol;
#pragma unroll 1
      for (int c = half; c < D / 32; c += 2) {
        uint32_t v[32];
        tmem_ld32(oaddr + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<uint4*>(osm + size_t(row) * (D + 4) + c * 32 + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
      }
      if (half == 0 && rr < R) {
        float* pm = part_ml + (size_t(slot_idx) * RMAX + rr) * 2;
        pm[0] = m_run * kLn2, pm[1] = l_run + redm[row];  // the maximum back in the natural-log domain the merge works in
      }
      tc_fence_before();
    }
    __syncthreads();
    if (!failed) {
      const int nreal = min(kTcRows, R - r_begin);
      float* po = part_o + (size_t(slot_idx) * RMAX + r_begin) * D;
      for (int idx = tid; idx < nreal * (D / 4); idx += kTcThreads) {
        const int r = idx / (D / 4), c4 = (idx % (D / 4)) * 4;
        *reinterpret_cast<float4*>(po + size_t(r) * D + c4) = *reinterpret_cast<const float4*>(osm + size_t(r) * (D + 4) + c4);
      }
    }
    if (stamp && item == int(blockIdx.x)) stamps[10] = global_ns();
    __syncthreads();  // the TMEM reads are done before the next item's MMAs overwrite S and O
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

template <int D, int G>
int launch_tc_attention(const __half* q, const StepBuffers& sb, const ModelDims& d, int al, const KvPoolDev& kv, float* part_o,
                        float* part_ml, int chunk_slots, int grid, const PrefetchPlan& plan, unsigned long long* stamps, cudaStream_t s) {
  LB_CUDA(launch_kernel(attention_tc_kernel<D, G>, dim3(grid), dim3(kTcThreads), TcSmem<D>::kBytes, s, q, sb, d, al, kv, part_o, part_ml,
                        chunk_slots, plan, stamps));
  LB_LAUNCH("attention_tc_kernel");
  return LING_B200_OK;
}

}  // namespace

int attention_tc_init() {
  LB_CUDA(cudaFuncSetAttribute(attention_tc_kernel<256, 6>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(TcSmem<256>::kBytes)));
  LB_CUDA(cudaFuncSetAttribute(attention_tc_kernel<64, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(TcSmem<64>::kBytes)));
  LB_CUDA(cudaFuncSetAttribute(attention_tc_kernel<128, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(TcSmem<128>::kBytes)));
  LB_CUDA(cudaFuncSetAttribute(attention_tc_kernel<128, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(TcSmem<128>::kBytes)));
  return LING_B200_OK;
}

bool attention_tc_supported(const ModelDims& d) {
  const int G = d.Hkv > 0 ? d.Hq / d.Hkv : 0;
  return (d.D == 256 && G == 6) || (d.D == 64 && G == 4) || (d.D == 128 && (G == 4 || G == 8));
}

int attention_tc_launch(const __half* q, const StepBuffers& sb, const ModelDims& d, int al, const KvPoolDev& kv, float* part_o,
                        float* part_ml, int chunk_slots, int grid, const PrefetchPlan& plan, unsigned long long* stamps, cudaStream_t s) {
  const int G = d.Hq / d.Hkv;
  if (d.D == 256 && G == 6) return launch_tc_attention<256, 6>(q, sb, d, al, kv, part_o, part_ml, chunk_slots, grid, plan, stamps, s);
  if (d.D == 64 && G == 4) return launch_tc_attention<64, 4>(q, sb, d, al, kv, part_o, part_ml, chunk_slots, grid, plan, stamps, s);
  if (d.D == 128 && G == 4) return launch_tc_attention<128, 4>(q, sb, d, al, kv, part_o, part_ml, chunk_slots, grid, plan, stamps, s);
  if (d.D == 128 && G == 8) return launch_tc_attention<128, 8>(q, sb, d, al, kv, part_o, part_ml, chunk_slots, grid, plan, stamps, s);
  set_error("attention: unsupported (head_dim, q heads per kv head); built: (256,6), (64,4), (128,4), (128,8)");
  return LING_B200_ERR_UNSUPPORTED;
}

}  // namespace lb
