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
// One CTA of 16 warps per value head walks the chunks in order.  Key and value dimension 128.
#include <cuda_fp16.h>

#include "gdn_chunk.h"

namespace lb {
namespace {

constexpr int kD = 128, kT = 32, kThreads = 512;
constexpr int kLdD = 136;  // halves per row of a [*][128] tile: rows 68 words apart, the 8 x 4 fragment loads hit 32 banks
constexpr int kLdT = 40;   // halves per row of a [*][32] tile

struct ChunkSmem {
  __half q[kT * kLdD];     // q^ [i][d]
  __half k[kT * kLdD];     // k^ [i][d]
  __half w[kT * kLdD];     // W [i][d]
  __half bvT[kD * kLdT];   // (beta v)^T [c][j]
  __half bgkT[kD * kLdT];  // (beta gamma k^)^T [d][j]
  __half kpT[kD * kLdT];   // k'^T [d][j]
  __half dT[kD * kLdT];    // Delta^T [c][j]
  __half sT[kD * kLdD];    // S0^T [c][d]
  __half tinv[kT * kLdT];  // Tinv [i][j]
  __half p[kT * kLdT];     // exp(G_i - G_j) q_i . k_j, j <= i
  float a[kT][kT + 1];     // A, fp32 for the substitution
  float G[kT], gam[kT], beta[kT];
  // the next chunk's raw rows, copied in (cp.async) while the current chunk is computed
  float rq[kT * kD], rk[kT * kD], rv[kT * kD], rg[kT], rb[kT];
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
__device__ __forceinline__ void copy4(void* dst, const void* src, bool real) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(uint32_t(__cvta_generic_to_shared(dst))), "l"(src), "r"(real ? 4 : 0) : "memory");
}
__device__ __forceinline__ void copies_done() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ uint32_t h2(float lo, float hi) {
  const __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

__global__ void __launch_bounds__(kThreads, 1)
    gdn_chunk_kernel(const float* __restrict__ post, const float* __restrict__ g, const float* __restrict__ beta, int M, int Hk, int HV,
                     float* __restrict__ state, float* __restrict__ core) {
  pdl_sync();  // first statement: see common.cuh
  extern __shared__ __align__(16) unsigned char raw_smem[];
  ChunkSmem& sm = *reinterpret_cast<ChunkSmem*>(raw_smem);
  const int hv = blockIdx.x, h = hv / (HV / Hk), tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gq = lane >> 2, tq = lane & 3;
  const int C = 2 * Hk * kD + HV * kD;
  float* st = state + size_t(hv) * kD * kD;
  // The state in the accumulator layout of its update: warp w owns the value columns 8 w .. 8 w + 7, S[mt][*] the key rows
  // 16 mt + gq (two of them: +8) at columns 8 w + 2 tq, + 1.
  float S[8][4];
#pragma unroll
  for (int mt = 0; mt < 8; ++mt) {
    const int d = mt * 16 + gq, c = warp * 8 + 2 * tq;
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
  // Requests the raw rows of the chunk that starts at row r0: q, k (this key head) and v (this value head), g and beta.
  auto fetch_chunk = [&](int r0) {
    const int rows = min(kT, M - r0);
    for (int idx = tid; idx < 3 * kT * (kD / 4); idx += kThreads) {
      const int part = idx / (kT * (kD / 4)), i = (idx / (kD / 4)) % kT, e = (idx % (kD / 4)) * 4;
      const bool real = i < rows;
      const float* row = post + size_t(r0 + (real ? i : 0)) * C;
      const float* src = part == 0 ? row + h * kD + e : part == 1 ? row + Hk * kD + h * kD + e : row + 2 * Hk * kD + hv * kD + e;
      copy16((part == 0 ? sm.rq : part == 1 ? sm.rk : sm.rv) + i * kD + e, src, real);
    }
    if (tid < 2 * kT) {
      const int i = tid % kT;
      const bool real = i < rows;
      copy4((tid < kT ? sm.rg : sm.rb) + i, (tid < kT ? g : beta) + size_t(r0 + (real ? i : 0)) * HV + hv, real);
    }
  };
  fetch_chunk(0);

  for (int c0 = 0; c0 < M; c0 += kT) {
    const int n = min(kT, M - c0);  // rows past n: k = v = 0, beta = 0, g = 0 -- they change nothing and are not stored
    copies_done();
    __syncthreads();  // the chunk's raw rows are in shared memory; the previous chunk's readers of the tiles are done
    // ---- gates: every warp scans the log-decays (lane i ends with G_i); warp 0 also keeps them for the later phases
    float G = sm.rg[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, G, o);
      if (lane >= o) G += up;
    }
    const float G_last = __shfl_sync(0xffffffffu, G, kT - 1);
    if (warp == 0) sm.G[lane] = G, sm.gam[lane] = __expf(G), sm.beta[lane] = sm.rb[lane];
    // ---- q^, k^ (two rows a warp; lane l holds the elements l, l + 32, l + 64, l + 96), k^ scaled for W and for the state update
    {
      const int i0 = 2 * warp;
      float kx[2][4], bg[2], kp[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int i = i0 + r;
        float qv[4], kv[4], sq = 0.f, sk = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          qv[e] = sm.rq[i * kD + lane + 32 * e], kv[e] = sm.rk[i * kD + lane + 32 * e];
          sq = fmaf(qv[e], qv[e], sq), sk = fmaf(kv[e], kv[e], sk);
        }
        sq = warp_sum(sq), sk = warp_sum(sk);
        const float cq = rsqrtf(sq + 1e-6f) * rsqrtf(float(kD)), ck = rsqrtf(sk + 1e-6f);
        const float Gi = __shfl_sync(0xffffffffu, G, i);
        bg[r] = sm.rb[i] * __expf(Gi), kp[r] = __expf(G_last - Gi);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          kx[r][e] = kv[e] * ck;
          sm.q[i * kLdD + lane + 32 * e] = __float2half_rn(qv[e] * cq);
          sm.k[i * kLdD + lane + 32 * e] = __float2half_rn(kx[r][e]);
        }
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {  // the two rows of a transposed tile as one 32-bit store
        *reinterpret_cast<uint32_t*>(sm.bgkT + (lane + 32 * e) * kLdT + i0) = h2(bg[0] * kx[0][e], bg[1] * kx[1][e]);
        *reinterpret_cast<uint32_t*>(sm.kpT + (lane + 32 * e) * kLdT + i0) = h2(kp[0] * kx[0][e], kp[1] * kx[1][e]);
      }
    }
    for (int idx = tid; idx < (kT / 2) * kD; idx += kThreads) {
      const int i = (idx / kD) * 2, c = idx % kD;
      *reinterpret_cast<uint32_t*>(sm.bvT + c * kLdT + i) = h2(sm.rb[i] * sm.rv[i * kD + c], sm.rb[i + 1] * sm.rv[(i + 1) * kD + c]);
    }
    __syncthreads();
    if (c0 + kT < M) fetch_chunk(c0 + kT);  // lands while this chunk is computed
    // ---- Q S0 (every warp: its 8 value columns, both row halves), K K^T (warps 0-7) and Q K^T (warps 8-15)
    float qs[2][4] = {};
    tiles_mma<2, kD>(qs, sm.q, kLdD, 0, sm.sT, kLdD, warp * 8, lane);
    {
      const int t8 = warp & 7, m0 = (t8 >> 2) * 16, n0 = (t8 & 3) * 8;
      float acc[1][4] = {};
      tiles_mma<1, kD>(acc, warp < 8 ? sm.k : sm.q, kLdD, t8 >> 2, sm.k, kLdD, n0, lane);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = m0 + gq + (e >> 1) * 8, j = n0 + 2 * tq + (e & 1);
        const float decay = __expf(sm.G[i] - sm.G[j]);  // <= 1 for j <= i
        if (warp < 8) sm.a[i][j] = j < i ? sm.beta[i] * decay * acc[0][e] : 0.f;
        else sm.p[i * kLdT + j] = __float2half_rn(j <= i ? decay * acc[0][e] : 0.f);
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
    // ---- U = Tinv (beta v) (kept in registers), W = Tinv (beta gamma k) (to shared memory)
    float u[2][4] = {};
    tiles_mma<2, kT>(u, sm.tinv, kLdT, 0, sm.bvT, kLdT, warp * 8, lane);
    {
      float wv[2][4] = {};
      tiles_mma<2, kT>(wv, sm.tinv, kLdT, 0, sm.bgkT, kLdT, warp * 8, lane);
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        *reinterpret_cast<uint32_t*>(sm.w + (mt * 16 + gq) * kLdD + warp * 8 + 2 * tq) = h2(wv[mt][0], wv[mt][1]);
        *reinterpret_cast<uint32_t*>(sm.w + (mt * 16 + gq + 8) * kLdD + warp * 8 + 2 * tq) = h2(wv[mt][2], wv[mt][3]);
      }
    }
    __syncthreads();
    // ---- Delta = U - W S0, transposed to shared memory
    {
      float ws[2][4] = {};
      tiles_mma<2, kD>(ws, sm.w, kLdD, 0, sm.sT, kLdD, warp * 8, lane);
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        const int i = mt * 16 + gq, c = warp * 8 + 2 * tq;
        sm.dT[c * kLdT + i] = __float2half_rn(u[mt][0] - ws[mt][0]), sm.dT[(c + 1) * kLdT + i] = __float2half_rn(u[mt][1] - ws[mt][1]);
        sm.dT[c * kLdT + i + 8] = __float2half_rn(u[mt][2] - ws[mt][2]), sm.dT[(c + 1) * kLdT + i + 8] = __float2half_rn(u[mt][3] - ws[mt][3]);
      }
    }
    __syncthreads();
    // ---- O = diag(gamma) Q S0 + P Delta; S = gamma_T S + K'^T Delta
    {
      float pd[2][4] = {};
      tiles_mma<2, kT>(pd, sm.p, kLdT, 0, sm.dT, kLdT, warp * 8, lane);
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        const int i = mt * 16 + gq, c = warp * 8 + 2 * tq;
        if (i < n)
          *reinterpret_cast<float2*>(core + size_t(c0 + i) * HV * kD + size_t(hv) * kD + c) =
              make_float2(fmaf(sm.gam[i], qs[mt][0], pd[mt][0]), fmaf(sm.gam[i], qs[mt][1], pd[mt][1]));
        if (i + 8 < n)
          *reinterpret_cast<float2*>(core + size_t(c0 + i + 8) * HV * kD + size_t(hv) * kD + c) =
              make_float2(fmaf(sm.gam[i + 8], qs[mt][2], pd[mt][2]), fmaf(sm.gam[i + 8], qs[mt][3], pd[mt][3]));
      }
    }
    const float gT = sm.gam[kT - 1];
    {
      float acc[8][4] = {};
      tiles_mma<8, kT>(acc, sm.kpT, kLdT, 0, sm.dT, kLdT, warp * 8, lane);
#pragma unroll
      for (int mt = 0; mt < 8; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) S[mt][e] = fmaf(gT, S[mt][e], acc[mt][e]);
    }
    __syncthreads();  // every reader of sT and of the chunk's tiles is done
    publish_state();
  }
#pragma unroll
  for (int mt = 0; mt < 8; ++mt) {
    const int d = mt * 16 + gq, c = warp * 8 + 2 * tq;
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

int gdn_chunk_init() {
  LB_CUDA(cudaFuncSetAttribute(gdn_chunk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(sizeof(ChunkSmem))));
  return LING_B200_OK;
}

int gdn_chunk_launch(const float* post, const float* g, const float* beta, int M, int Hk, int HV, int Dk, int Dv, float* state, float* core,
                     cudaStream_t s) {
  if (Dk != kD || Dv != kD || M < 1 || Hk < 1 || HV % Hk != 0) return LING_B200_ERR_ARG;
  LB_CUDA(launch_kernel(gdn_chunk_kernel, dim3(HV), dim3(kThreads), sizeof(ChunkSmem), s, post, g, beta, M, Hk, HV, state, core));
  LB_LAUNCH("gdn_chunk_kernel");
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
