// ref_cuda_shim.cu -- C wrappers around the REFERENCE's own CUDA kernels (src/core/kernels.cu, topk.cu, draft_kernels.cu, prefill_gdn.cu of
// dreamference/ling-engine), compiled for sm_100a from where the sources lie into oracle/_ref/libling_refcuda.so (see
// oracle/Makefile, target ref_cuda).  TEST INFRASTRUCTURE ONLY.  Nothing of the reference is copied into this repository:
// this file includes the reference's header and calls its launchers on device copies of host buffers, so that the CPU
// oracle's fp32 math (conv over trees, gating, the gated delta rule, gated RMSNorm, head norms + rotation, top-K, the candidate selector's lattice) and the
// product's kernels can be compared with what the reference itself computes on the same GPU.
//
// The reference's kernels are built for its 27B shapes only (DeltaNet key/value dim 128, attention head dim 256 with six
// query heads per KV head), keep the KV cache in BF16 and take at most 32 rows of one sequence; the wrappers mirror that.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "core/kernels.cuh"

namespace {
namespace K = ling::kernels;

std::string g_err;

struct Dev {  // device allocations freed on scope exit
  std::vector<void*> p;
  ~Dev() {
    for (void* q : p) cudaFree(q);
  }
  template <typename T>
  T* get(size_t n) {
    void* q = nullptr;
    if (cudaMalloc(&q, (n ? n : 1) * sizeof(T)) != cudaSuccess) throw std::runtime_error("cudaMalloc failed");
    cudaMemset(q, 0, (n ? n : 1) * sizeof(T));
    p.push_back(q);
    return static_cast<T*>(q);
  }
  template <typename T>
  T* put(const T* host, size_t n) {
    T* q = get<T>(n);
    if (cudaMemcpy(q, host, n * sizeof(T), cudaMemcpyHostToDevice) != cudaSuccess) throw std::runtime_error("H2D copy failed");
    return q;
  }
  __nv_bfloat16* put_bf16(const float* host, size_t n) {
    std::vector<__nv_bfloat16> h(n);
    for (size_t i = 0; i < n; ++i) h[i] = __float2bfloat16(host[i]);
    return put(h.data(), n);
  }
};

template <typename T>
void fetch(T* host, const T* dev, size_t n) {
  if (cudaMemcpy(host, dev, n * sizeof(T), cudaMemcpyDeviceToHost) != cudaSuccess) throw std::runtime_error("D2H copy failed");
}
void sync() {
  const cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) throw std::runtime_error(std::string("CUDA: ") + cudaGetErrorString(e));
}

template <typename F>
int guarded(F&& body) {
  try {
    body();
    return 0;
  } catch (const std::exception& e) {
    g_err = e.what();
    return 1;
  }
}
}  // namespace

// sparse_head.cu's draft_head_rows calls the rows-path GEMMs of stream_gemm.cu, which does not build for sm_100a; the shim
// never calls draft_head_rows, so these only satisfy the linker.
namespace ling::kernels {
void to_half_rows(const float*, int, int, __half*, float*, cudaStream_t) { throw std::runtime_error("to_half_rows: not built here"); }
void stream_gemm_nvfp4(const __half*, const float*, int, const uint8_t*, const uint8_t*, float, float*, int, int, cudaStream_t) {
  throw std::runtime_error("stream_gemm_nvfp4: not built here");
}
void stream_gemm_gather_nvfp4(const __half*, const float*, int, const uint8_t*, const uint8_t*, float, const int*, const int*, int, float*, int,
                              cudaStream_t) {
  throw std::runtime_error("stream_gemm_gather_nvfp4: not built here");
}
}  // namespace ling::kernels

extern "C" {

const char* refcuda_last_error() { return g_err.c_str(); }
int refcuda_tree_desc_bytes() { return int(sizeof(K::TreeDesc)); }

// gdn_conv_tree + gdn_recurrent_tree (src/core/kernels.cu:365-383,455-477) for one sequence: td is the host TreeDesc.
int refcuda_gdn_tree(int Hk, int HV, const void* td, const float* pre, const float* convw, const float* g, const float* beta,
                     const float* state, const float* conv, float* post, float* core) {
  return guarded([&] {
    K::TreeDesc t;
    std::memcpy(&t, td, sizeof t);
    const int M = t.n, C = 2 * Hk * 128 + HV * 128, Vs = HV * 128;
    Dev d;
    K::TreeDesc* d_td = d.put(&t, 1);
    float* d_pre = d.put(pre, size_t(M) * C);
    float* d_post = d.get<float>(size_t(M) * C);
    float* d_core = d.get<float>(size_t(M) * Vs);
    K::gdn_conv_tree(d_pre, d_post, d.put(conv, size_t(C) * 3), d.put_bf16(convw, size_t(C) * 4), M, C, d_td, 0);
    K::gdn_recurrent_tree(d_post, d.put(g, size_t(M) * HV), d.put(beta, size_t(M) * HV), d.put(state, size_t(HV) * 128 * 128), d_core,
                          Hk, HV, d_td, t.ngdn, 0);
    sync();
    fetch(post, d_post, size_t(M) * C);
    fetch(core, d_core, size_t(M) * Vs);
  });
}

// Engine::commit's two launches for one DeltaNet layer (src/core/speculate.cpp:516-529): gdn_conv in place over the n
// accepted rows' raw inputs (the window advances), gdn_recurrent over their conv outputs with the state written in place.
int refcuda_gdn_commit(int Hk, int HV, int n, const float* pre_rows, const float* post_rows, const float* g_rows,
                       const float* beta_rows, const float* convw, float* state, float* conv) {
  return guarded([&] {
    const int C = 2 * Hk * 128 + HV * 128;
    Dev d;
    float* d_state = d.put(state, size_t(HV) * 128 * 128);
    float* d_conv = d.put(conv, size_t(C) * 3);
    K::gdn_conv(d.put(pre_rows, size_t(n) * C), d_conv, d.put_bf16(convw, size_t(C) * 4), n, C, 0);
    K::gdn_recurrent(d.put(post_rows, size_t(n) * C), d.put(g_rows, size_t(n) * HV), d.put(beta_rows, size_t(n) * HV), d_state, d_state,
                     d.get<float>(size_t(n) * HV * 128), n, Hk, HV, 0);
    sync();
    fetch(state, d_state, size_t(HV) * 128 * 128);
    fetch(conv, d_conv, size_t(C) * 3);
  });
}

// gdn_gating (src/core/kernels.cu:385-395).
int refcuda_gdn_gating(const float* a, const float* b, const float* A_log, const float* dt_bias, float* g, float* beta, int M, int HV) {
  return guarded([&] {
    Dev d;
    float* d_g = d.get<float>(size_t(M) * HV);
    float* d_b = d.get<float>(size_t(M) * HV);
    K::gdn_gating(d.put(a, size_t(M) * HV), d.put(b, size_t(M) * HV), d.put_bf16(A_log, HV), d.put_bf16(dt_bias, HV), d_g, d_b, M, HV, 0);
    sync();
    fetch(g, d_g, size_t(M) * HV);
    fetch(beta, d_b, size_t(M) * HV);
  });
}

// gated_rmsnorm (src/core/kernels.cu:543-554): rows of length D.
int refcuda_gated_rmsnorm(const float* x, const float* z, const float* w, float* out, int rows, int D, float eps) {
  return guarded([&] {
    Dev d;
    float* d_o = d.get<float>(size_t(rows) * D);
    K::gated_rmsnorm(d.put(x, size_t(rows) * D), d.put(z, size_t(rows) * D), d.put_bf16(w, D), d_o, rows, D, eps, 0);
    sync();
    fetch(out, d_o, size_t(rows) * D);
  });
}

// attn_prepare (src/core/kernels.cu:558-582, src/core/attention_body.cuh:54-99) for M rows of one sequence at position
// pos0 (rope delta rdelta; td: the host TreeDesc of a tree verify, or NULL for a chain).  Out: q and gate [M][Hq][D], and
// the M new cache entries of K (normed, rotated) and V, [M][Hkv][D], widened from the BF16 the reference stores.
int refcuda_attn_prepare(const float* q_gate, const float* k, const float* v, const float* q_norm, const float* k_norm, int pos0,
                         int rdelta, int M, int Hq, int Hkv, int D, int rot, float theta, float eps, const void* td, float* q_out,
                         float* gate_out, float* k_new, float* v_new) {
  return guarded([&] {
    Dev d;
    K::TreeDesc t;
    K::TreeDesc* d_td = nullptr;
    if (td) {
      std::memcpy(&t, td, sizeof t);
      d_td = d.put(&t, 1);
    }
    const size_t per = size_t(Hkv) * D, cache = size_t(pos0 + M) * per;  // the default layout: [position][kv head][D]
    __nv_bfloat16* kc = d.get<__nv_bfloat16>(cache);
    __nv_bfloat16* vc = d.get<__nv_bfloat16>(cache);
    float* d_q = d.get<float>(size_t(M) * Hq * D);
    float* d_gate = d.get<float>(size_t(M) * Hq * D);
    K::DevPos pos(pos0);
    K::attn_prepare(d.put(q_gate, size_t(M) * Hq * 2 * D), d.put(k, size_t(M) * per), d.put(v, size_t(M) * per), d.put_bf16(q_norm, D),
                    d.put_bf16(k_norm, D), pos.with_rope(rdelta, nullptr), M, Hq, Hkv, D, rot, theta, eps, d_q, d_gate, kc, vc, 0, d_td);
    sync();
    fetch(q_out, d_q, size_t(M) * Hq * D);
    fetch(gate_out, d_gate, size_t(M) * Hq * D);
    std::vector<__nv_bfloat16> hk(size_t(M) * per), hv(size_t(M) * per);
    fetch(hk.data(), kc + size_t(pos0) * per, hk.size());
    fetch(hv.data(), vc + size_t(pos0) * per, hv.size());
    for (size_t i = 0; i < hk.size(); ++i) k_new[i] = __bfloat162float(hk[i]), v_new[i] = __bfloat162float(hv[i]);
  });
}

// attention_rows (src/core/kernels.cu:919-936; body src/core/attention_body.cuh:262-525) for M rows of one sequence at
// position pos0 over the caches kcache / vcache [pos0 + M][Hkv][D] (values given in fp32, stored as BF16: pass values that
// BF16 holds exactly), td as above.  out [M][Hq][D].
int refcuda_attention_rows(const float* q, const float* kcache, const float* vcache, int pos0, int M, int Hq, int Hkv, int D,
                           const void* td, float* out) {
  return guarded([&] {
    Dev d;
    K::TreeDesc t;
    K::TreeDesc* d_td = nullptr;
    if (td) {
      std::memcpy(&t, td, sizeof t);
      d_td = d.put(&t, 1);
    }
    const size_t cache = size_t(pos0 + M) * Hkv * D;
    float* d_out = d.get<float>(size_t(M) * Hq * D);
    float* scratch = d.get<float>(K::attention_rows_scratch_floats(M, Hq, D, pos0 + M));
    K::attention_rows(d.put(q, size_t(M) * Hq * D), d.put_bf16(kcache, cache), d.put_bf16(vcache, cache), K::DevPos(pos0), M, Hq, Hkv, D,
                      scratch, d_out, 0, 0, d_td);
    sync();
    fetch(out, d_out, size_t(M) * Hq * D);
  });
}

// topk_rows with K = 1 (src/core/topk.cu:83-129).
int refcuda_top1(const float* logits, int rows, int V, int* ids, float* vals) {
  return guarded([&] {
    Dev d;
    int* d_i = d.get<int>(rows);
    float* d_v = d.get<float>(rows);
    K::topk_rows(d.put(logits, size_t(rows) * V), rows, V, 1, d.get<float>(K::topk_scratch_floats(rows, 1)), d_v, d_i, 0);
    sync();
    fetch(ids, d_i, rows);
    fetch(vals, d_v, rows);
  });
}

// topk_rows for any K <= 64 (src/core/topk.cu:83-129): values descending, ties to the lower index.
int refcuda_topk(const float* logits, int rows, int V, int K_, int* ids, float* vals) {
  return guarded([&] {
    Dev d;
    int* d_i = d.get<int>(size_t(rows) * K_);
    float* d_v = d.get<float>(size_t(rows) * K_);
    K::topk_rows(d.put(logits, size_t(rows) * V), rows, V, K_, d.get<float>(K::topk_scratch_floats(rows, K_)), d_v, d_i, 0);
    sync();
    fetch(ids, d_i, size_t(rows) * K_);
    fetch(vals, d_v, size_t(rows) * K_);
  });
}

// sparse_head_select (src/core/sparse_head.cu:183-230): p [M][256] fp32, us [N][256] given as fp32 and rounded to BF16 here, one
// mask of N bytes; rows [cap] (ascending ids) and their count.
int refcuda_sparse_select(const float* p, int M, const float* us, int N, const unsigned char* mask, int dynamic, int cap, int* rows,
                          int* nrows) {
  return guarded([&] {
    Dev d;
    int* d_rows = d.get<int>(size_t(N));
    int* d_n = d.get<int>(1);
    K::SelMasks ms{};
    ms.n = 1;
    ms.m[0] = d.put(mask, size_t(N));
    K::sparse_head_select(d.put(p, size_t(M) * 256), M, d.put_bf16(us, size_t(N) * 256), N, 256, ms, dynamic, cap,
                          d.get<unsigned char>(K::sparse_head_scratch_bytes(N)), d_rows, d_n, 0);
    sync();
    fetch(nrows, d_n, 1);
    fetch(rows, d_rows, size_t(*nrows));
  });
}

// selector_lattice (src/core/draft_kernels.cu:328-351): hp [E][256], cand / unary [E][16], the two codebooks [vocab][256]
// given as fp32 and rounded to BF16 here, scores [E][16][16].
int refcuda_selector_lattice(const float* hp, const int* cand, const float* unary, const float* P, const float* S, int vocab,
                             int anchor, int E, float* scores) {
  return guarded([&] {
    Dev d;
    float* d_s = d.get<float>(size_t(E) * 256);
    K::selector_lattice(d.put(hp, size_t(E) * 256), d.put(cand, size_t(E) * 16), d.put(unary, size_t(E) * 16),
                        d.put_bf16(P, size_t(vocab) * 256), d.put_bf16(S, size_t(vocab) * 256), anchor, E, d_s, 0);
    sync();
    fetch(scores, d_s, size_t(E) * 256);
  });
}

// gdn_conv_prefill + gdn_recurrent_prefill (src/core/prefill_gdn.cu): the reference's own prefill DeltaNet core over M rows.
int refcuda_gdn_prefill(int Hk, int HV, int M, const float* pre, const float* convw, const float* g, const float* beta, float* state,
                        float* conv, float* post, float* core) {
  return guarded([&] {
    Dev d;
    const int C = 2 * Hk * 128 + HV * 128;
    float* d_state = d.put(state, size_t(HV) * 128 * 128);
    float* d_conv = d.put(conv, size_t(C) * 3);
    float* d_post = d.get<float>(size_t(M) * C);
    float* d_core = d.get<float>(size_t(M) * HV * 128);
    K::gdn_conv_prefill(d.put(pre, size_t(M) * C), d_post, d_conv, d.put_bf16(convw, size_t(C) * 4), M, C, 0);
    K::gdn_recurrent_prefill(d_post, d.put(g, size_t(M) * HV), d.put(beta, size_t(M) * HV), d_state, d_core, M, Hk, HV, 0, 0);
    sync();
    fetch(state, d_state, size_t(HV) * 128 * 128);
    fetch(conv, d_conv, size_t(C) * 3);
    fetch(post, d_post, size_t(M) * C);
    fetch(core, d_core, size_t(M) * HV * 128);
  });
}

}  // extern "C"
