// gdn_chunk.cu -- the gated delta rule over many tokens of one sequence (a prefill chunk), in its chunked (WY) form.
//
// The verify step's kernels walk a tree's few rows token by token; 4096 rows of a prefill chunk would be 4096 dependent
// steps per head.  Unrolled over a chunk of T = 32 tokens with start state S0 [Dk][Dv], cumulative log-decay G_i and
// gamma_i = exp(G_i), the recurrence S_i = a_i S_(i-1) + k_i beta_i (v_i - a_i S_(i-1)^T k_i)^T, o_i = S_i^T q_i becomes
//   A_ij   = beta_i exp(G_i - G_j) k_i . k_j  (j < i),        Tinv = (I + A)^-1  (forward substitution, fp32)
//   U      = Tinv (beta v),   W = Tinv (beta gamma k),        Delta = U - W S0
//   O      = diag(gamma) Q S0 + [exp(G_i - G_j) q_i . k_j]_(j <= i) Delta
//   S_next = gamma_T S0 + K'^T Delta,   k'_i = (gamma_T / gamma_i) k_i
// (the reference's chunk_gdn_kernel, src/core/prefill_gdn.cu:75-142, restated).  Every product is a small matrix product
// with a 32-row operand: they run as FP16 m16n8k16 MMAs with fp32 accumulation from shared memory -- tiles of 32 rows are
// below the 64-row minimum of tcgen05.mma, and the chain of chunks is bound by its dependent steps, not by tensor
// throughput.  The state stays in fp32 registers (the accumulator layout of its own update) and is multiplied as an FP16
// copy; q and k arrive un-normalized (the conv's output) and are L2-normalized here, q also scaled by 1/sqrt(Dk).
// Two kernels: A, P, Tinv, U and W do not depend on the state, so one CTA per (chunk, value head) prepares them for every chunk at
// once (the GPU is full), and one CTA of 16 warps per value head then walks the chunks in order with only the state-dependent
// products left (two barriers a chunk), the prepared records arriving by cp.async three chunks ahead.  Key and value dimension 128.
#include <cuda_fp16.h>

#include "gdn_chunk.h"

namespace lb {
namespace {

constexpr int kD = 128, kT = 32, kThreads = 512, kPrepThreads = 256;
constexpr int kLdD = 136;  // halves per row of a [*][128] tile: rows 68 words apart, the 8 x 4 fragment loads hit 32 banks
constexpr int kLdT = 40;   // halves per row of a [*][32] tile

// What the state-independent half leaves per (chunk, value head) for the state-dependent half, in the padded layouts the MMAs
// read from shared memory (so the record is copied there as it is): 46720 bytes.
struct ChunkTiles {
  __half q[kT * kLdD];     // q^ [i][d]
  __half w[kT * kLdD];     // W = Tinv (beta gamma k^) [i][d]
  __half p[kT * kLdT];     // exp(G_i - G_j) q_i . k_j, j <= i
  __half kpT[kD * kLdT];   // k'^T [d][j]
};
struct ChunkRecord {
  ChunkTiles t;
  float u[kT * kD];        // U = Tinv (beta v) [i][c]
  float gam[kT];           // gamma_i
};
static_assert(sizeof(ChunkRecord) % 16 == 0 && sizeof(ChunkTiles) % 16 == 0, "records are copied in 16-byte pieces");

struct PrepSmem {  // the prepare kernel's working tiles (the record's q, w, p, kpT are built in `t`; u goes straight to global memory)
  ChunkTiles t;
  __half k[kT * kLdD];     // k^ [i][d]
  __half bvT[kD * kLdT];   // (beta v)^T [c][j]
  __half bgkT[kD * kLdT];  // (beta gamma k^)^T [d][j]
  __half tinv[kT * kLdT];  // Tinv [i][j]
  float a[kT][kT + 1];     // A, fp32 for the substitution
  float G[kT], gam[kT], beta[kT];
};

constexpr int kStages = 3;  // records in flight in the apply kernel
struct ApplySmem {
  ChunkRecord rec[kStages];
  __half sT[kD * kLdD];    // S0^T [c][d], the state's FP16 copy
  __half dT[kD * kLdT];    // Delta^T [c][j]
};

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// ldmatrix.x4: four 8 x 8 FP16 matrices; lane l supplies the address of row l % 8 of matrix l / 8 (16 bytes, 16-byte aligned),
// and receives from each matrix the pair at (row l / 4, columns 2 (l % 4), + 1) -- the fragment layout of mma.m16n8k16.
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], const __half* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(uint32_t(__cvta_generic_to_shared(p))));
}
// The A fragment (16 x 16) of a row-major [m][k] tile at (m0, k0): matrices rows 0-7 / 8-15 at k0, then the same at k0 + 8.
__device__ __forceinline__ void frag_a(uint32_t (&a)[4], const __half* A, int lda, int m0, int k0, int lane) {
  ldsm4(a, A + (m0 + (lane & 7) + 8 * ((lane >> 3) & 1)) * lda + k0 + 8 * (lane >> 4));
}
// The B fragments of two consecutive k steps (k0 .. k0 + 31) for the 8 columns n0 .. n0 + 7 of an [n][k] tile (k contiguous):
// b[0], b[1] belong to k0, b[2], b[3] to k0 + 16.
__device__ __forceinline__ void frag_b2(uint32_t (&b)[4], const __half* B, int ldb, int n0, int k0, int lane) {
  ldsm4(b, B + (n0 + (lane & 7)) * ldb + k0 + 8 * (lane >> 3));
}
// c[t] (rows 16 t .. 16 t + 15 of the MT row tiles from mt0 on, columns n0 .. n0 + 7) += A . B^T over K (a multiple of 32);
// A [m][k], B [n][k], both with k contiguous.  The row tiles share the B fragments.
template <int MT, int K>
__device__ __forceinline__ void tiles_mma(float (&c)[MT][4], const __half* A, int lda, int mt0, const __half* B, int ldb, int n0, int lane) {
#pragma unroll
  for (int k0 = 0; k0 < K; k0 += 32) {
    uint32_t b[4];
    frag_b2(b, B, ldb, n0, k0, lane);
#pragma unroll
    for (int t = 0; t < MT; ++t) {
      uint32_t a[4];
      frag_a(a, A, lda, (mt0 + t) * 16, k0, lane);
      mma16816(c[t], a[0], a[1], a[2], a[3], b[0], b[1]);
      frag_a(a, A, lda, (mt0 + t) * 16, k0 + 16, lane);
      mma16816(c[t], a[0], a[1], a[2], a[3], b[2], b[3]);
    }
  }
}
__device__ __forceinline__ void copy16(void* dst, const void* src, bool real) {  // zero-filled when the row does not exist
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(uint32_t(__cvta_generic_to_shared(dst))), "l"(src), "r"(real ? 16 : 0) : "memory");
}
__device__ __forceinline__ uint32_t h2(float lo, float hi) {
  const __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// The state-independent half, one CTA of 8 warps per (chunk, value head): L2 norms, the decays, A and P, the substitution, U and
// W.  6144 independent CTAs for 4096 rows of the 27B model: this half fills the GPU.
__global__ void __launch_bounds__(kPrepThreads)
    gdn_chunk_prepare_kernel(const float* __restrict__ post, const float* __restrict__ g, const float* __restrict__ beta, int M, int Hk, int HV,
                             ChunkRecord* __restrict__ records) {
  pdl_sync();  // first statement: see common.cuh
  extern __shared__ __align__(16) unsigned char raw_smem[];
  PrepSmem& sm = *reinterpret_cast<PrepSmem*>(raw_smem);
  const int chunk = blockIdx.x, hv = blockIdx.y, h = hv / (HV / Hk), tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gq = lane >> 2, tq = lane & 3;
  const int C = 2 * Hk * kD + HV * kD, c0 = chunk * kT, n = min(kT, M - c0);
  // rows past n: k = v = 0, beta = 0, g = 0 -- they change nothing and are not stored
  // ---- gates: every warp scans the log-decays (lane i ends with G_i); warp 0 keeps them for the later phases
  float G = lane < n ? g[size_t(c0 + lane) * HV + hv] : 0.f;
  const float b_lane = lane < n ? beta[size_t(c0 + lane) * HV + hv] : 0.f;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float up = __shfl_up_sync(0xffffffffu, G, o);
    if (lane >= o) G += up;
  }
  const float G_last = __shfl_sync(0xffffffffu, G, kT - 1);
  if (warp == 0) sm.G[lane] = G, sm.gam[lane] = __expf(G), sm.beta[lane] = b_lane;
  // ---- q^, k^ (four rows a warp, in two pairs; lane l holds the elements l, l + 32, l + 64, l + 96), k^ scaled for W and the state
  for (int pr = 0; pr < 2; ++pr) {
    const int i0 = 4 * warp + 2 * pr;
    float kx[2][4], bg[2], kp[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int i = i0 + r;
      float qv[4], kv[4], sq = 0.f, sk = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float* row = post + size_t(c0 + min(i, n - 1)) * C;
        qv[e] = i < n ? row[h * kD + lane + 32 * e] : 0.f, kv[e] = i < n ? row[Hk * kD + h * kD + lane + 32 * e] : 0.f;
        sq = fmaf(qv[e], qv[e], sq), sk = fmaf(kv[e], kv[e], sk);
      }
      sq = warp_sum(sq), sk = warp_sum(sk);
      const float cq = rsqrtf(sq + 1e-6f) * rsqrtf(float(kD)), ck = rsqrtf(sk + 1e-6f);
      const float Gi = __shfl_sync(0xffffffffu, G, i), bi = __shfl_sync(0xffffffffu, b_lane, i);
      bg[r] = bi * __expf(Gi), kp[r] = __expf(G_last - Gi);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        kx[r][e] = kv[e] * ck;
        sm.t.q[i * kLdD + lane + 32 * e] = __float2half_rn(qv[e] * cq);
        sm.k[i * kLdD + lane + 32 * e] = __float2half_rn(kx[r][e]);
      }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {  // the two rows of a transposed tile as one 32-bit store
      *reinterpret_cast<uint32_t*>(sm.bgkT + (lane + 32 * e) * kLdT + i0) = h2(bg[0] * kx[0][e], bg[1] * kx[1][e]);
      *reinterpret_cast<uint32_t*>(sm.t.kpT + (lane + 32 * e) * kLdT + i0) = h2(kp[0] * kx[0][e], kp[1] * kx[1][e]);
    }
  }
  for (int idx = tid; idx < (kT / 2) * kD; idx += kPrepThreads) {
    const int i = (idx / kD) * 2, c = idx % kD;
    const float b0 = __shfl_sync(0xffffffffu, b_lane, i), b1 = __shfl_sync(0xffffffffu, b_lane, i + 1);  // (i is warp-uniform: 128 columns a row pair)
    const float v0 = i < n ? post[size_t(c0 + i) * C + 2 * Hk * kD + hv * kD + c] : 0.f;
    const float v1 = i + 1 < n ? post[size_t(c0 + i + 1) * C + 2 * Hk * kD + hv * kD + c] : 0.f;
    *reinterpret_cast<uint32_t*>(sm.bvT + c * kLdT + i) = h2(b0 * v0, b1 * v1);
  }
  __syncthreads();
  // ---- K K^T (warps 0-3, two tiles each) and Q K^T (warps 4-7)
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int t8 = (warp & 3) * 2 + half, m0 = (t8 >> 2) * 16, n0 = (t8 & 3) * 8;
    float acc[1][4] = {};
    tiles_mma<1, kD>(acc, warp < 4 ? sm.k : sm.t.q, kLdD, t8 >> 2, sm.k, kLdD, n0, lane);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = m0 + gq + (e >> 1) * 8, j = n0 + 2 * tq + (e & 1);
      const float decay = __expf(sm.G[i] - sm.G[j]);  // <= 1 for j <= i
      if (warp < 4) sm.a[i][j] = j < i ? sm.beta[i] * decay * acc[0][e] : 0.f;
      else sm.t.p[i * kLdT + j] = __float2half_rn(j <= i ? decay * acc[0][e] : 0.f);
    }
  }
  __syncthreads();
  // ---- Tinv = (I + A)^-1 by forward substitution: lane l of warp 0 solves column l, x_i = [i == l] - sum_(j < i) A_ij x_j
  if (warp == 0) {
    float x[kT];
#pragma unroll
    for (int i = 0; i < kT; ++i) {
      float part[4] = {i == lane ? 1.f : 0.f, 0.f, 0.f, 0.f};  // four interleaved sums: a quarter of the dependent chain
#pragma unroll
      for (int j = 0; j < i; ++j) part[j & 3] = fmaf(-sm.a[i][j], x[j], part[j & 3]);
      x[i] = (part[0] + part[1]) + (part[2] + part[3]);
      sm.tinv[i * kLdT + lane] = __float2half_rn(x[i]);
    }
  }
  __syncthreads();
  // ---- U = Tinv (beta v) and W = Tinv (beta gamma k): warp w takes the columns 16 w .. 16 w + 15
  ChunkRecord* out = records + size_t(chunk) * HV + hv;
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) {
    const int n0 = warp * 16 + nt * 8;
    float u[2][4] = {}, wv[2][4] = {};
    tiles_mma<2, kT>(u, sm.tinv, kLdT, 0, sm.bvT, kLdT, n0, lane);
    tiles_mma<2, kT>(wv, sm.tinv, kLdT, 0, sm.bgkT, kLdT, n0, lane);
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
      *reinterpret_cast<float2*>(out->u + (mt * 16 + gq) * kD + n0 + 2 * tq) = make_float2(u[mt][0], u[mt][1]);
      *reinterpret_cast<float2*>(out->u + (mt * 16 + gq + 8) * kD + n0 + 2 * tq) = make_float2(u[mt][2], u[mt][3]);
      *reinterpret_cast<uint32_t*>(sm.t.w + (mt * 16 + gq) * kLdD + n0 + 2 * tq) = h2(wv[mt][0], wv[mt][1]);
      *reinterpret_cast<uint32_t*>(sm.t.w + (mt * 16 + gq + 8) * kLdD + n0 + 2 * tq) = h2(wv[mt][2], wv[mt][3]);
    }
  }
  __syncthreads();
  // ---- the record's shared-memory tiles out (q, w, p, kpT: the record's first bytes) and the decays
  const uint4* src = reinterpret_cast<const uint4*>(&sm.t);
  uint4* dst = reinterpret_cast<uint4*>(&out->t);
  for (int idx = tid; idx < int(sizeof(ChunkTiles) / 16); idx += kPrepThreads) dst[idx] = src[idx];
  if (tid < kT) out->gam[tid] = sm.gam[tid];
}

// The state-dependent half, per value head walking the chunks in order: Delta = U - W S0, O = diag(gamma) Q S0 + P Delta,
// S = gamma_T S0 + K'^T Delta.  Every value column is independent of the others, so a head's 128 columns are split over
// gridDim.y CTAs (blockDim.x / 32 warps of 8 columns each): 48 heads alone leave two thirds of the SMs idle, and a chunk's
// time is mostly its mma.sync instructions.  The records arrive by cp.async three chunks ahead; two barriers per chunk.
__global__ void __launch_bounds__(kThreads, 1)
    gdn_chunk_apply_kernel(const ChunkRecord* __restrict__ records, int M, int HV, float* __restrict__ state, float* __restrict__ core) {
  pdl_sync();  // first statement: see common.cuh
  extern __shared__ __align__(16) unsigned char raw_smem[];
  ApplySmem& sm = *reinterpret_cast<ApplySmem*>(raw_smem);
  const int hv = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, threads = blockDim.x;
  const int col0 = int(blockIdx.y) * (threads >> 5) * 8;  // this CTA's first value column of the head
  const int gq = lane >> 2, tq = lane & 3;
  const int n_chunks = (M + kT - 1) / kT;
  float* st = state + size_t(hv) * kD * kD;
  // The state in the accumulator layout of its update: warp w owns the value columns 8 w .. 8 w + 7, S[mt][*] the key rows
  // 16 mt + gq (two of them: +8) at columns 8 w + 2 tq, + 1.
  float S[8][4];
#pragma unroll
  for (int mt = 0; mt < 8; ++mt) {
    const int d = mt * 16 + gq, c = col0 + warp * 8 + 2 * tq;
    const float2 lo = *reinterpret_cast<const float2*>(st + size_t(d) * kD + c);
    const float2 hi = *reinterpret_cast<const float2*>(st + size_t(d + 8) * kD + c);
    S[mt][0] = lo.x, S[mt][1] = lo.y, S[mt][2] = hi.x, S[mt][3] = hi.y;
  }
  auto publish_state = [&] {  // the FP16 copy, transposed: sT[c][d]
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) {
      const int d = mt * 16 + gq, c = warp * 8 + 2 * tq;
      sm.sT[c * kLdD + d] = __float2half_rn(S[mt][0]), sm.sT[(c + 1) * kLdD + d] = __float2half_rn(S[mt][1]);
      sm.sT[c * kLdD + d + 8] = __float2half_rn(S[mt][2]), sm.sT[(c + 1) * kLdD + d + 8] = __float2half_rn(S[mt][3]);
    }
  };
  publish_state();
  auto fetch = [&](int chunk) {  // one cp.async group per chunk (an empty group past the end keeps the count uniform)
    if (chunk < n_chunks) {
      const char* src = reinterpret_cast<const char*>(records + size_t(chunk) * HV + hv);
      char* dst = reinterpret_cast<char*>(&sm.rec[chunk % kStages]);
      for (int idx = tid; idx < int(sizeof(ChunkRecord) / 16); idx += threads) copy16(dst + idx * 16, src + idx * 16, true);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  fetch(0);
  fetch(1);
  for (int ch = 0; ch < n_chunks; ++ch) {
    const int c0 = ch * kT, n = min(kT, M - c0);
    asm volatile("cp.async.wait_group 1;" ::: "memory");  // this chunk's record has landed (the next one may still be on its way)
    __syncthreads();  // ... for every thread; the state's copy of the previous chunk is published; its readers of rec / dT are done
    fetch(ch + 2);    // into the stage chunk ch - 1 used
    const ChunkRecord& r = sm.rec[ch % kStages];
    // ---- Q S0 and W S0 (every warp: its 8 value columns, both row halves), Delta = U - W S0 transposed to shared memory
    float qs[2][4] = {};
    tiles_mma<2, kD>(qs, r.t.q, kLdD, 0, sm.sT, kLdD, warp * 8, lane);
    {
      float ws[2][4] = {};
      tiles_mma<2, kD>(ws, r.t.w, kLdD, 0, sm.sT, kLdD, warp * 8, lane);
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        const int i = mt * 16 + gq, c = warp * 8 + 2 * tq;  // (column inside the CTA: the shared-memory tiles hold the CTA's columns)
        const float2 ua = *reinterpret_cast<const float2*>(r.u + i * kD + col0 + c), ub = *reinterpret_cast<const float2*>(r.u + (i + 8) * kD + col0 + c);
        sm.dT[c * kLdT + i] = __float2half_rn(ua.x - ws[mt][0]), sm.dT[(c + 1) * kLdT + i] = __float2half_rn(ua.y - ws[mt][1]);
        sm.dT[c * kLdT + i + 8] = __float2half_rn(ub.x - ws[mt][2]), sm.dT[(c + 1) * kLdT + i + 8] = __float2half_rn(ub.y - ws[mt][3]);
      }
    }
    __syncthreads();  // Delta is complete; nobody reads the state's FP16 copy any more
    // ---- O = diag(gamma) Q S0 + P Delta; S = gamma_T S + K'^T Delta
    {
      float pd[2][4] = {};
      tiles_mma<2, kT>(pd, r.t.p, kLdT, 0, sm.dT, kLdT, warp * 8, lane);
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        const int i = mt * 16 + gq, c = col0 + warp * 8 + 2 * tq;
        if (i < n)
          *reinterpret_cast<float2*>(core + size_t(c0 + i) * HV * kD + size_t(hv) * kD + c) =
              make_float2(fmaf(r.gam[i], qs[mt][0], pd[mt][0]), fmaf(r.gam[i], qs[mt][1], pd[mt][1]));
        if (i + 8 < n)
          *reinterpret_cast<float2*>(core + size_t(c0 + i + 8) * HV * kD + size_t(hv) * kD + c) =
              make_float2(fmaf(r.gam[i + 8], qs[mt][2], pd[mt][2]), fmaf(r.gam[i + 8], qs[mt][3], pd[mt][3]));
      }
    }
    const float gT = r.gam[kT - 1];
    {
      float acc[8][4] = {};
      tiles_mma<8, kT>(acc, r.t.kpT, kLdT, 0, sm.dT, kLdT, warp * 8, lane);
#pragma unroll
      for (int mt = 0; mt < 8; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) S[mt][e] = fmaf(gT, S[mt][e], acc[mt][e]);
    }
    publish_state();
  }
  asm volatile("cp.async.wait_all;" ::: "memory");
#pragma unroll
  for (int mt = 0; mt < 8; ++mt) {
    const int d = mt * 16 + gq, c = col0 + warp * 8 + 2 * tq;
    *reinterpret_cast<float2*>(st + size_t(d) * kD + c) = make_float2(S[mt][0], S[mt][1]);
    *reinterpret_cast<float2*>(st + size_t(d + 8) * kD + c) = make_float2(S[mt][2], S[mt][3]);
  }
}

// conv_prefill_kernel + conv_window_kernel (src/core/prefill_gdn.cu:34-72): the four-tap causal conv over M rows in parallel,
// out of place, the first rows' taps from the session's window, then SiLU; the window afterwards holds the last three raw inputs.
constexpr int kConvRows = 16;  // rows a thread walks: every raw input is read once (plus three a tile for the taps before it)
__global__ void __launch_bounds__(256)
    conv_rows_kernel(const float* __restrict__ pre, const __nv_bfloat16* __restrict__ w, const float* __restrict__ win, int M, int C,
                     float* __restrict__ post) {
  pdl_sync();  // first statement: see common.cuh
  const int c4 = blockIdx.x * blockDim.x + threadIdx.x, t0 = blockIdx.y * kConvRows;
  if (c4 * 4 >= C) return;
  const int c = c4 * 4;
  float wt[4][4], x[3][4];  // [channel][tap], [age: oldest first][channel]
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const uint2 wr = *reinterpret_cast<const uint2*>(w + size_t(c + e) * 4);
    const __nv_bfloat162 w01 = *reinterpret_cast<const __nv_bfloat162*>(&wr.x), w23 = *reinterpret_cast<const __nv_bfloat162*>(&wr.y);
    wt[e][0] = __low2float(w01), wt[e][1] = __high2float(w01), wt[e][2] = __low2float(w23), wt[e][3] = __high2float(w23);
  }
#pragma unroll
  for (int j = 0; j < 3; ++j) {
    const int tt = t0 - 3 + j;
    if (tt >= 0) {
      const float4 v = *reinterpret_cast<const float4*>(pre + size_t(tt) * C + c);
      x[j][0] = v.x, x[j][1] = v.y, x[j][2] = v.z, x[j][3] = v.w;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) x[j][e] = win[(c + e) * 3 + 3 + tt];
    }
  }
  for (int t = t0; t < min(t0 + kConvRows, M); ++t) {
    const float4 v = *reinterpret_cast<const float4*>(pre + size_t(t) * C + c);
    const float cur[4] = {v.x, v.y, v.z, v.w};
    float o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      o[e] = silu(wt[e][0] * x[0][e] + wt[e][1] * x[1][e] + wt[e][2] * x[2][e] + wt[e][3] * cur[e]);
      x[0][e] = x[1][e], x[1][e] = x[2][e], x[2][e] = cur[e];
    }
    *reinterpret_cast<float4*>(post + size_t(t) * C + c) = make_float4(o[0], o[1], o[2], o[3]);
  }
}
__global__ void __launch_bounds__(256) conv_window_kernel(const float* __restrict__ pre, float* __restrict__ win, int M, int C) {
  pdl_sync();  // first statement: see common.cuh
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s[3];
#pragma unroll
  for (int j = 0; j < 3; ++j) {
    const int tt = M - 3 + j;
    s[j] = tt >= 0 ? pre[size_t(tt) * C + c] : win[c * 3 + 3 + tt];
  }
#pragma unroll
  for (int j = 0; j < 3; ++j) win[c * 3 + j] = s[j];
}

}  // namespace

// The gating projections of a prefill chunk on tensor cores (a = xn . W_a^T, b = xn . W_b^T, then g = -exp(A_log) softplus(a +
// dt_bias), beta = sigmoid(b): src/core/kernels.cu:200-253,385-395): 4096 rows x 96 outputs x 5120 is two billion multiply-adds,
// 240 us on the CUDA cores.  The fp32 rows are split into two BF16 terms (x = hi + lo, |lo| <= 2^-9 |x|): with BF16 weights both
// products are exact in fp32, so the sum differs from the fp32 one by the accumulation order and by 2^-17 of a term.  A CTA takes
// 32 rows and every output; its eight warps split the hidden dimension and meet in shared memory.  The k index of an MMA step
// is permuted (lane t of the fragment layout supplies the columns 4 t .. 4 t + 3 of the step's 16) so that a lane's A values are
// one 16-byte load and its B values one 8-byte load.
constexpr int kGateRows = 32, kGateCols = 96, kGateWarps = 8;
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void split_bf16(float x, float y, uint32_t& hi, uint32_t& lo) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
  const __nv_bfloat162 l = __floats2bfloat162_rn(x - __low2float(h), y - __high2float(h));
  hi = *reinterpret_cast<const uint32_t*>(&h), lo = *reinterpret_cast<const uint32_t*>(&l);
}
__global__ void __launch_bounds__(kGateWarps * 32)
    ab_gating_mma_kernel(const float* __restrict__ xn, const __nv_bfloat16* __restrict__ wa, const __nv_bfloat16* __restrict__ wb,
                         const __nv_bfloat16* __restrict__ A_log, const __nv_bfloat16* __restrict__ dt_bias, float* __restrict__ g,
                         float* __restrict__ beta, int M, int H, int HV, int col0) {
  pdl_sync();  // first statement: see common.cuh
  extern __shared__ __align__(16) float gate_red[];  // [warps][32 rows][97]
  constexpr int LDR = kGateCols + 1, NTL = kGateCols / 8;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, gq = lane >> 2, tq = lane & 3;
  const int m0 = blockIdx.x * kGateRows, ncols = min(kGateCols, 2 * HV - col0);
  const int kw = H / kGateWarps, k_lo = warp * kw;
  // this lane's rows of x (clamped: a row past M contributes to outputs that are not written) and rows of W per column tile
  const float* xr[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) xr[i] = xn + size_t(min(m0 + (i >> 1) * 16 + (i & 1) * 8 + gq, M - 1)) * H + 4 * tq;
  const __nv_bfloat16* wr[NTL];
#pragma unroll
  for (int nt = 0; nt < NTL; ++nt) {
    const int c = min(col0 + nt * 8 + gq, 2 * HV - 1);
    wr[nt] = (c < HV ? wa + size_t(c) * H : wb + size_t(c - HV) * H) + 4 * tq;
  }
  float acc[2][NTL][4] = {};
  for (int k = k_lo; k < k_lo + kw; k += 16) {
    uint32_t ah[2][4], al[2][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
      const float4 top = *reinterpret_cast<const float4*>(xr[2 * mt] + k), bot = *reinterpret_cast<const float4*>(xr[2 * mt + 1] + k);
      split_bf16(top.x, top.y, ah[mt][0], al[mt][0]), split_bf16(bot.x, bot.y, ah[mt][1], al[mt][1]);
      split_bf16(top.z, top.w, ah[mt][2], al[mt][2]), split_bf16(bot.z, bot.w, ah[mt][3], al[mt][3]);
    }
#pragma unroll
    for (int nt = 0; nt < NTL; ++nt) {
      const uint2 b = __ldg(reinterpret_cast<const uint2*>(wr[nt] + k));
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        mma_bf16(acc[mt][nt], ah[mt][0], ah[mt][1], ah[mt][2], ah[mt][3], b.x, b.y);
        mma_bf16(acc[mt][nt], al[mt][0], al[mt][1], al[mt][2], al[mt][3], b.x, b.y);
      }
    }
  }
  float* mine = gate_red + size_t(warp) * kGateRows * LDR;
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int nt = 0; nt < NTL; ++nt) {
      const int r = mt * 16 + gq, c = nt * 8 + 2 * tq;
      mine[r * LDR + c] = acc[mt][nt][0], mine[r * LDR + c + 1] = acc[mt][nt][1];
      mine[(r + 8) * LDR + c] = acc[mt][nt][2], mine[(r + 8) * LDR + c + 1] = acc[mt][nt][3];
    }
  __syncthreads();
  for (int i = threadIdx.x; i < kGateRows * kGateCols; i += blockDim.x) {
    const int r = i / kGateCols, c = i % kGateCols, m = m0 + r, col = col0 + c;
    if (m >= M || c >= ncols) continue;
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < kGateWarps; ++w) tot += gate_red[(size_t(w) * kGateRows + r) * LDR + c];
    if (col < HV) {
      const float xx = tot + __bfloat162float(dt_bias[col]);
      const float sp = xx <= 20.f ? log1pf(__expf(xx)) : xx;
      g[size_t(m) * HV + col] = -__expf(__bfloat162float(A_log[col])) * sp;
    } else {
      beta[size_t(m) * HV + col - HV] = 1.f / (1.f + __expf(-tot));
    }
  }
}

int gdn_chunk_init() {
  LB_CUDA(cudaFuncSetAttribute(ab_gating_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kGateWarps * kGateRows * (kGateCols + 1) * 4)));
  LB_CUDA(cudaFuncSetAttribute(gdn_chunk_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(sizeof(PrepSmem))));
  LB_CUDA(cudaFuncSetAttribute(gdn_chunk_apply_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(sizeof(ApplySmem))));
  return LING_B200_OK;
}

size_t gdn_chunk_scratch_bytes(int M, int HV) { return size_t(ceil_div(std::max(M, 1), kT)) * std::max(HV, 1) * sizeof(ChunkRecord); }

int gdn_chunk_launch(const float* post, const float* g, const float* beta, int M, int Hk, int HV, int Dk, int Dv, float* state, float* core,
                     void* scratch, cudaStream_t s) {
  if (Dk != kD || Dv != kD || M < 1 || Hk < 1 || HV % Hk != 0 || !scratch) return LING_B200_ERR_ARG;
  ChunkRecord* rec = static_cast<ChunkRecord*>(scratch);
  LB_CUDA(launch_kernel(gdn_chunk_prepare_kernel, dim3(ceil_div(M, kT), HV), dim3(kPrepThreads), sizeof(PrepSmem), s, post, g, beta, M, Hk, HV, rec));
  LB_LAUNCH("gdn_chunk_prepare_kernel");
  // a head's columns over as many CTAs as still run in one wave (one CTA per SM: its shared memory): 48 heads x 2 CTAs of 8 warps
  // (measured at 4096 rows x 48 heads: 661 us with one CTA a head, 459 with two, 531 with four = 192 CTAs for 148 SMs)
  const int parts = HV <= 37 ? 4 : HV <= 74 ? 2 : 1;
  LB_CUDA(launch_kernel(gdn_chunk_apply_kernel, dim3(HV, parts), dim3(kThreads / parts), sizeof(ApplySmem), s, (const ChunkRecord*)rec, M, HV, state, core));
  LB_LAUNCH("gdn_chunk_apply_kernel");
  return LING_B200_OK;
}

// g, beta [M][HV] from the normalized rows xn [M][H] (fp32) and the two BF16 projections [HV][H]; H a multiple of 128.
int ab_gating_mma_launch(const float* xn, const __nv_bfloat16* wa, const __nv_bfloat16* wb, const __nv_bfloat16* A_log, const __nv_bfloat16* dt_bias,
                         float* g, float* beta, int M, int H, int HV, cudaStream_t s) {
  if (M < 1 || HV < 1 || H % (kGateWarps * 16) != 0) return LING_B200_ERR_ARG;
  for (int col0 = 0; col0 < 2 * HV; col0 += kGateCols) {  // 96 outputs a launch (the 27B model's 48 + 48 in one)
    LB_CUDA(launch_kernel(ab_gating_mma_kernel, dim3(ceil_div(M, kGateRows)), dim3(kGateWarps * 32), size_t(kGateWarps) * kGateRows * (kGateCols + 1) * 4, s,
                          xn, wa, wb, A_log, dt_bias, g, beta, M, H, HV, col0));
    LB_LAUNCH("ab_gating_mma_kernel");
  }
  return LING_B200_OK;
}

int conv_rows_launch(const float* pre, const __nv_bfloat16* w, float* window, int M, int C, float* post, cudaStream_t s) {
  if (M < 1 || C < 1) return LING_B200_ERR_ARG;
  if (C % 4 != 0) return LING_B200_ERR_ARG;
  LB_CUDA(launch_kernel(conv_rows_kernel, dim3(ceil_div(C / 4, 256), ceil_div(M, kConvRows)), dim3(256), size_t(0), s, pre, w, (const float*)window,
                        M, C, post));
  LB_LAUNCH("conv_rows_kernel");
  LB_CUDA(launch_kernel(conv_window_kernel, dim3(ceil_div(C, 256)), dim3(256), size_t(0), s, pre, window, M, C));
  LB_LAUNCH("conv_window_kernel");
  return LING_B200_OK;
}

}  // namespace lb
