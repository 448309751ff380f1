// kernel_abi.cu -- kernel-level entry points of the C ABI: each runs one of the step's kernels on host buffers (copy in,
// launch, copy out), the way the reference's model-free kernel tests drive its kernel layer on random data
// (tests/stream_tests.cu, tests/tree_tests.cu in the reference project).  They allocate and free their own scratch.
#include <vector>

#include "abi_util.h"
#include "draft_head.h"
#include "gdn_chunk.h"
#include "chain.h"
#include "gemm.h"
#include "kernels.h"

using namespace lb;

namespace {

struct GemmSetup {
  Fp8Matrix W;
  Fp8Acts X;
  float* out = nullptr;
  int* err = nullptr;
};

int setup_gemm(Scratch& sc, GemmSetup& g, int M, int N, int K, int splits) {
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
  Fp8Matrix& W = g.W;
  W.N = N, W.K = K, W.N_pad = round_up(N, kTileN), W.K_pad = round_up(K, kBlockK), W.KB = W.K_pad / kBlockK;
  W.splits = splits > 0 ? std::min(splits, W.KB) : choose_splits(W.N_pad, W.KB, sms);
  W.codes = sc.get<uint8_t>(size_t(W.N_pad) * W.K_pad);
  W.scales = sc.get<float>(size_t(W.KB) * W.N_pad);
  Fp8Acts& X = g.X;
  X.K = K, X.K_pad = W.K_pad, X.KB = W.KB, X.rows_alloc = round_up(M, 128);
  X.codes = sc.get<uint8_t>(size_t(X.rows_alloc) * X.K_pad);
  X.scales = sc.get<float>(size_t(X.KB) * X.rows_alloc);
  g.out = sc.get<float>(size_t(W.splits) * X.rows_alloc * W.N_pad);
  g.err = sc.get<int>(1);
  LB_PTR(W.codes && W.scales && X.codes && X.scales && g.out && g.err);
  LB_TRY(make_weight_map(W));
  return make_acts_maps(X);
}

}  // namespace

extern "C" {

int ling_b200_gemm_fp8_host(int device, int impl, int splits, const float* x, const float* w, float* y, int M, int N, int K) {
  if (!x || !w || !y || M < 1 || N < 1 || K < 1 || M > LING_B200_MAX_ROWS) {
    set_error("gemm_fp8_host: bad argument");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(check_device(device));
  Scratch sc;
  GemmSetup g;
  LB_TRY(setup_gemm(sc, g, M, N, K, splits));
  float* dw = sc.put(w, size_t(N) * K);
  float* dx = sc.put(x, size_t(M) * K);
  LB_PTR(dw && dx);
  LB_TRY(quant_weight_launch(dw, 0, 0.f, 0, g.W.codes, g.W.scales, 0, N, K, g.W.N_pad, g.W.K_pad, 0));
  LB_TRY(quant_acts_launch(dx, M, QuantOut{g.X.codes, g.X.scales, K, g.X.K_pad, g.X.rows_alloc}, 0));
  // With dependent launch the GEMM loads weight tiles before its dependency wait, on the understanding that no kernel
  // just ahead of it writes the weights: the quantizers must have completed before it is launched.
  LB_CUDA(cudaStreamSynchronize(0));
  GemmCall c;
  c.W = &g.W, c.X = &g.X, c.M = M, c.out = g.out, c.ld = g.W.N_pad;
  c.split_stride = size_t(g.X.rows_alloc) * g.W.N_pad;
  c.impl = impl, c.err_flag = g.err;
  LB_TRY(gemm_launch(c, 0));
  LB_CUDA(cudaDeviceSynchronize());
  int err = 0;
  LB_CUDA(cudaMemcpy(&err, g.err, 4, cudaMemcpyDeviceToHost));
  if (err) {
    set_error("gemm: device error word = " + std::to_string(err));
    return LING_B200_ERR_DEVICE_FLAG;
  }
  const int planes = impl == 1 ? 1 : g.W.splits;
  std::vector<float> host(size_t(planes) * c.split_stride);
  LB_CUDA(cudaMemcpy(host.data(), g.out, host.size() * 4, cudaMemcpyDeviceToHost));
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      float v = 0.f;
      for (int p = 0; p < planes; ++p) v += host[size_t(p) * c.split_stride + size_t(m) * g.W.N_pad + n];  // plane order
      y[size_t(m) * N + n] = v;
    }
  return LING_B200_OK;
}

int ling_b200_gemm_fp8_bench(int device, int impl, int splits, int M, int N, int K, int iters, float* ms_per_launch) {
  if (M < 1 || N < 1 || K < 1 || iters < 1 || !ms_per_launch || M > LING_B200_MAX_ROWS) {
    set_error("gemm_fp8_bench: bad argument");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(check_device(device));
  Scratch sc;
  GemmSetup g;
  LB_TRY(setup_gemm(sc, g, M, N, K, splits));
  float* dx = sc.get<float>(size_t(M) * K, false);
  LB_PTR(dx);
  LB_TRY(fill_f32_launch(stream_key(1, 7), 1.f, dx, size_t(M) * K, 0));
  LB_TRY(quant_weight_launch(nullptr, stream_key(1, 9), 0.02f, 1, g.W.codes, g.W.scales, 0, N, K, g.W.N_pad, g.W.K_pad, 0));
  LB_TRY(quant_acts_launch(dx, M, QuantOut{g.X.codes, g.X.scales, K, g.X.K_pad, g.X.rows_alloc}, 0));
  LB_CUDA(cudaStreamSynchronize(0));  // the weights are complete before a GEMM that may read them ahead of its dependency wait
  GemmCall c;
  c.W = &g.W, c.X = &g.X, c.M = M, c.out = g.out, c.ld = g.W.N_pad;
  c.split_stride = size_t(g.X.rows_alloc) * g.W.N_pad;
  c.impl = (impl & 0xff) == 2 ? 0 : (impl & 0xff), c.err_flag = g.err;
  c.force_tile = impl >> 8;  // (impl | tile << 8: the token tile forced, for tile-size comparisons)
  impl &= 0xff;
  cudaEvent_t a, b;
  LB_CUDA(cudaEventCreate(&a));
  LB_CUDA(cudaEventCreate(&b));
  // impl 2: the same GEMM as a one-GEMM chain (chain.cu) for rows <= 32: what the persistent kernel's GEMM part costs alone
  ChainProgram P;
  unsigned* counters = nullptr;
  if (impl == 2) {
    LB_TRY(chain_init());
    counters = sc.get<unsigned>(kChainCounterWords);
    int* n_rows = sc.put(&M, 1);
    LB_PTR(counters && n_rows);
    P.n_gemm = 1, P.norm_gemm = -1, P.n_rows = n_rows, P.rows_grid = std::min(32, round_up(M, 32)), P.counters = counters, P.err_flag = g.err;
    ChainGemm& G = P.g[0];
    G.mapW = g.W.map, G.mapX = g.X.map[0], G.ws = g.W.scales, G.xs = g.X.scales, G.out = g.out, G.split_stride = c.split_stride;
    G.N = g.W.N, G.N_pad = g.W.N_pad, G.KB = g.W.KB, G.splits = g.W.splits, G.xrows = g.X.rows_alloc;
    if (M > 32 || !chain_supported(P, 148)) {
      set_error("gemm_fp8_bench: the chain kernel does not cover this shape");
      return LING_B200_ERR_UNSUPPORTED;
    }
  }
  auto one = [&]() -> int { return impl == 2 ? chain_launch(P, 148, 0) : gemm_launch(c, 0); };
  for (int i = 0; i < 3; ++i) LB_TRY(one());
  LB_CUDA(cudaEventRecord(a, 0));
  for (int i = 0; i < iters; ++i) LB_TRY(one());
  LB_CUDA(cudaEventRecord(b, 0));
  LB_CUDA(cudaEventSynchronize(b));
  float ms = 0.f;
  LB_CUDA(cudaEventElapsedTime(&ms, a, b));
  cudaEventDestroy(a), cudaEventDestroy(b);
  int err = 0;
  LB_CUDA(cudaMemcpy(&err, g.err, 4, cudaMemcpyDeviceToHost));
  if (err) {
    set_error("gemm: device error word = " + std::to_string(err));
    return LING_B200_ERR_DEVICE_FLAG;
  }
  *ms_per_launch = ms / iters;
  return LING_B200_OK;
}

// The FP8 tensor pipe's sustained rate (tensor_peak_kernel): one CTA per SM, `iters` MMA groups each, timed with CUDA
// events after a warm-up launch; dense TFLOP/s = 2 * 128 * 256 * 128 * iters * SMs / time.
int ling_b200_fp8_tensor_peak(int device, int iters, float* tflops, float* ms) {
  if (!tflops || iters < 1 || iters > (1 << 22)) {
    set_error("fp8_tensor_peak: bad argument");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(check_device(device));
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  Scratch sc;
  int* err = sc.get<int>(1);
  LB_PTR(err);
  cudaEvent_t a, b;
  LB_CUDA(cudaEventCreate(&a));
  LB_CUDA(cudaEventCreate(&b));
  LB_TRY(tensor_peak_launch(sms, iters, err, 0));
  LB_CUDA(cudaEventRecord(a, 0));
  LB_TRY(tensor_peak_launch(sms, iters, err, 0));
  LB_CUDA(cudaEventRecord(b, 0));
  LB_CUDA(cudaEventSynchronize(b));
  float t = 0.f;
  LB_CUDA(cudaEventElapsedTime(&t, a, b));
  cudaEventDestroy(a), cudaEventDestroy(b);
  int code = 0;
  LB_CUDA(cudaMemcpy(&code, err, 4, cudaMemcpyDeviceToHost));
  if (code) {
    set_error("fp8_tensor_peak: device error word = " + std::to_string(code));
    return LING_B200_ERR_DEVICE_FLAG;
  }
  *tflops = float(2.0 * 128 * 256 * 128 * double(iters) * sms / (double(t) * 1e-3) / 1e12);
  if (ms) *ms = t;
  return LING_B200_OK;
}

// A bounded device wait made to run out on purpose (see wait_probe_kernel): returns LING_B200_ERR_DEVICE_FLAG with the
// recorded code in *code and the time the kernel waited in *waited_us; the device stays usable.
int ling_b200_wait_probe(int device, unsigned limit_us, int* code, unsigned* waited_us) {
  if (!code || !waited_us || limit_us < 1 || limit_us > 100000) {
    set_error("wait_probe: a limit of 1 .. 100000 microseconds expected");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(check_device(device));
  Scratch sc;
  int* err = sc.get<int>(1);
  unsigned long long* waited = sc.get<unsigned long long>(1);
  LB_PTR(err && waited);
  LB_TRY(wait_probe_launch(uint64_t(limit_us) * 1000ull, err, waited, 0));
  LB_CUDA(cudaDeviceSynchronize());
  unsigned long long w = 0;
  LB_CUDA(cudaMemcpy(code, err, 4, cudaMemcpyDeviceToHost));
  LB_CUDA(cudaMemcpy(&w, waited, 8, cudaMemcpyDeviceToHost));
  *waited_us = unsigned(w / 1000ull);
  if (*code != 0) {
    set_error("device error word = " + std::to_string(*code) + " (a bounded wait ran out)");
    return LING_B200_ERR_DEVICE_FLAG;
  }
  return LING_B200_OK;
}

namespace {
// A one-sequence StepBuffers for the DeltaNet kernels.
struct OneSeq {
  StepBuffers sb;
  ModelDims d{};
  int build(Scratch& sc, int Hk, int HV, int Dk, int Dv, int n_rows, int chain, const ling_b200_tree_desc* td,
            const ling_b200_seq_result* res) {
    d.Hk = Hk, d.HV = HV, d.Dk = Dk, d.Dv = Dv, d.C = 2 * Hk * Dk + HV * Dv, d.Vs = HV * Dv;
    d.max_seqs = 1, d.n_gdn = 1, d.rows_alloc = n_rows;
    const int one = 1;
    const SeqDev q{0, 0, 0, n_rows, chain, 0};
    const int row0[2] = {0, n_rows};
    sb.n_seqs = sc.put(&one, 1);
    sb.seqs = sc.put(&q, 1);
    sb.row0 = sc.put(row0, 2);
    sb.n_rows_total = sc.put(&n_rows, 1);
    int seq_of[kTreeRows] = {}, local[kTreeRows];
    for (int r = 0; r < kTreeRows; ++r) local[r] = r;
    sb.seq_of = sc.put(seq_of, kTreeRows);
    sb.local = sc.put(local, kTreeRows);
    sb.trees = td ? sc.put(td, 1) : sc.get<ling_b200_tree_desc>(1);
    sb.results = res ? sc.put(res, 1) : sc.get<ling_b200_seq_result>(1);
    sb.err = sc.get<int>(1);
    LB_PTR(sb.n_seqs && sb.seqs && sb.row0 && sb.n_rows_total && sb.trees && sb.results && sb.err && sb.seq_of && sb.local);
    return LING_B200_OK;
  }
};
bool gdn_dims_ok(int Hk, int HV, int Dk, int Dv) {
  return Hk > 0 && HV % Hk == 0 && (Dk == 64 || Dk == 128) && Dv % 32 == 0 && Dv <= 128;
}
}  // namespace

int ling_b200_gdn_tree_host(int device, int Hk, int HV, int Dk, int Dv, const ling_b200_tree_desc* td, const float* pre,
                            const float* convw, const float* g, const float* beta, const float* state, const float* conv,
                            float* post, float* core) {
  if (!td || !pre || !convw || !g || !beta || !state || !conv || !post || !core || !gdn_dims_ok(Hk, HV, Dk, Dv) || td->n < 1 ||
      td->n > kTreeRows) {
    set_error("gdn_tree_host: bad argument");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(check_device(device));
  Scratch sc;
  OneSeq o;
  LB_TRY(o.build(sc, Hk, HV, Dk, Dv, td->n, 0, td, nullptr));
  const int n = td->n, C = o.d.C, Vs = o.d.Vs;
  float* d_in = sc.put(pre, size_t(n) * C);
  float* d_w32 = sc.put(convw, size_t(C) * 4);
  __nv_bfloat16* d_w = sc.get<__nv_bfloat16>(size_t(C) * 4);
  float* d_g = sc.put(g, size_t(n) * HV);
  float* d_b = sc.put(beta, size_t(n) * HV);
  float* d_state = sc.put(state, size_t(HV) * Dk * Dv);
  float* d_conv = sc.put(conv, size_t(C) * 3);
  float* d_pre = sc.get<float>(size_t(n) * C);
  float* d_post = sc.get<float>(size_t(n) * C);
  float* d_core = sc.get<float>(size_t(n) * Vs);
  LB_PTR(d_in && d_w32 && d_w && d_g && d_b && d_state && d_conv && d_pre && d_post && d_core);
  LB_TRY(fill_bf16_launch(d_w32, 0, 0.f, 0.f, 0, d_w, size_t(C) * 4, 0));
  Planes in;
  in.p = d_in, in.n = 1, in.stride = 0, in.ld = C;
  LB_TRY(conv_tree_launch(in, o.sb, o.d, d_w, d_conv, 0, d_pre, d_post, n, 0));
  LB_TRY(gdn_tree_launch(d_post, d_g, d_b, o.sb, o.d, d_state, 0, d_core, 148 * 4, 0));
  LB_CUDA(cudaDeviceSynchronize());
  LB_CUDA(cudaMemcpy(post, d_post, size_t(n) * C * 4, cudaMemcpyDeviceToHost));
  LB_CUDA(cudaMemcpy(core, d_core, size_t(n) * Vs * 4, cudaMemcpyDeviceToHost));
  return LING_B200_OK;
}

namespace {
// Device-side description of a step of n_seqs sequences for the kernels that read StepBuffers, packed on the device by
// pack_kernel (tree descriptions, DeltaNet paths, conv taps) exactly as a context's step does.
struct PackedSeqs {
  StepBuffers sb;
  ModelDims d{};
  int rows = 0;
  int build(Scratch& sc, int n_seqs, const int* n_rows, const int* chain, const int* parent, int vocab) {
    if (n_seqs < 1 || n_seqs > LING_B200_MAX_SEQS) {
      set_error("sequence count out of range");
      return LING_B200_ERR_ARG;
    }
    std::vector<SeqDev> seqs(n_seqs);
    std::vector<int> par(size_t(n_seqs) * kTreeRows, 0), tok(size_t(n_seqs) * kTreeRows, 0);
    rows = 0;
    for (int s = 0; s < n_seqs; ++s) {
      if (n_rows[s] < 1 || n_rows[s] > kTreeRows) {
        set_error("a tree of 1 to 32 rows expected");
        return LING_B200_ERR_ARG;
      }
      seqs[s] = SeqDev{s, 0, 0, n_rows[s], chain[s], 0};
      for (int r = 0; r < n_rows[s]; ++r) par[size_t(s) * kTreeRows + r] = r == 0 ? -1 : parent[rows + r];
      rows += n_rows[s];
    }
    d.max_seqs = n_seqs, d.V = vocab, d.rows_alloc = round_up(rows, 128);
    sb.n_seqs = sc.put(&n_seqs, 1);
    sb.seqs = sc.put(seqs.data(), seqs.size());
    sb.in_parent = sc.put(par.data(), par.size());
    sb.in_token = sc.put(tok.data(), tok.size());
    sb.in_force = sc.get<int>(par.size());
    sb.row0 = sc.get<int>(n_seqs + 1);
    sb.n_rows_total = sc.get<int>(1);
    sb.token = sc.get<int>(d.rows_alloc), sb.seq_of = sc.get<int>(d.rows_alloc), sb.local = sc.get<int>(d.rows_alloc);
    sb.depth = sc.get<int>(d.rows_alloc), sb.rope_pos = sc.get<int>(d.rows_alloc), sb.cache_slot = sc.get<int>(d.rows_alloc);
    sb.anc = sc.get<uint32_t>(d.rows_alloc);
    sb.trees = sc.get<ling_b200_tree_desc>(n_seqs);
    sb.gdn_aux = sc.get<GdnAux>(n_seqs);
    sb.argmax_id = sc.get<int>(d.rows_alloc), sb.argmax_val = sc.get<float>(d.rows_alloc);
    sb.results = sc.get<ling_b200_seq_result>(n_seqs);
    sb.err = sc.get<int>(1);
    LB_PTR(sb.n_seqs && sb.seqs && sb.in_parent && sb.in_token && sb.in_force && sb.row0 && sb.n_rows_total && sb.token &&
           sb.seq_of && sb.local && sb.depth && sb.rope_pos && sb.cache_slot && sb.anc && sb.trees && sb.gdn_aux &&
           sb.argmax_id && sb.argmax_val && sb.results && sb.err);
    return LING_B200_OK;
  }
};
}  // namespace

// The step's DeltaNet mixer as the 27B-class step runs it (one launch: conv over the trees + SiLU, q/k normalization,
// the gated delta rule along every DeltaNet path, gated RMSNorm, FP8 copy), on host buffers; see include/ling_b200.h.
int ling_b200_gdn_fused_host(int device, int Hk, int HV, int Dk, int Dv, int n_seqs, const int* n_rows, const int* chain,
                             const int* parent, const float* in, const float* convw, const float* g, const float* beta,
                             const float* state, const float* conv, const float* norm_w, float eps, float* pre, float* post,
                             float* core, uint8_t* out_codes, float* out_scales) {
  if (!n_rows || !chain || !parent || !in || !convw || !g || !beta || !state || !conv || !norm_w || !pre || !post || !core ||
      !out_codes || !out_scales || !gdn_dims_ok(Hk, HV, Dk, Dv)) {
    set_error("gdn_fused_host: bad argument");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(check_device(device));
  Scratch sc;
  PackedSeqs ps;
  LB_TRY(ps.build(sc, n_seqs, n_rows, chain, parent, 1 << 30));
  ModelDims& d = ps.d;
  d.Hk = Hk, d.HV = HV, d.Dk = Dk, d.Dv = Dv, d.C = 2 * Hk * Dk + HV * Dv, d.Vs = HV * Dv, d.eps = eps, d.n_gdn = 1;
  if (!gdn_fused_supported(d)) {
    set_error("gdn_fused_host: the fused kernel covers key dim = value dim = 64 or 128 and value widths that are multiples of 128");
    return LING_B200_ERR_UNSUPPORTED;
  }
  const int n = ps.rows, C = d.C, Vs = d.Vs, W = C + Vs, KB = Vs / 128;
  float* d_in = sc.put(in, size_t(n) * W);
  float* d_w32 = sc.put(convw, size_t(C) * 4);
  float* d_n32 = sc.put(norm_w, size_t(Dv));
  __nv_bfloat16* d_w = sc.get<__nv_bfloat16>(size_t(C) * 4);
  __nv_bfloat16* d_nw = sc.get<__nv_bfloat16>(size_t(Dv));
  float* d_g = sc.put(g, size_t(n) * HV);
  float* d_b = sc.put(beta, size_t(n) * HV);
  float* d_state = sc.put(state, size_t(n_seqs) * HV * Dk * Dv);
  float* d_conv = sc.put(conv, size_t(n_seqs) * C * 3);
  float* d_pre = sc.get<float>(size_t(n) * C);
  float* d_post = sc.get<float>(size_t(n) * C);
  float* d_core = sc.get<float>(size_t(n) * Vs);
  uint8_t* d_codes = sc.get<uint8_t>(size_t(d.rows_alloc) * Vs);
  float* d_scales = sc.get<float>(size_t(KB) * d.rows_alloc);
  LB_PTR(d_in && d_w32 && d_n32 && d_w && d_nw && d_g && d_b && d_state && d_conv && d_pre && d_post && d_core && d_codes && d_scales);
  LB_TRY(fill_bf16_launch(d_w32, 0, 0.f, 0.f, 0, d_w, size_t(C) * 4, 0));
  LB_TRY(fill_bf16_launch(d_n32, 0, 0.f, 0.f, 0, d_nw, size_t(Dv), 0));
  LB_CUDA(cudaStreamSynchronize(0));
  Planes p_in;
  p_in.p = d_in, p_in.n = 1, p_in.stride = 0, p_in.ld = W;
  LB_TRY(pack_launch(ps.sb, d, 0));
  LB_TRY(gdn_fused_launch(p_in, ps.sb, d, d_w, d_conv, size_t(C) * 3, d_g, d_b, d_state, size_t(HV) * Dk * Dv, d_nw,
                          QuantOut{d_codes, d_scales, Vs, Vs, d.rows_alloc}, d_pre, d_post, d_core, n_seqs, 148, PrefetchPlan(), nullptr, 0));
  LB_CUDA(cudaDeviceSynchronize());
  int err = 0;
  LB_CUDA(cudaMemcpy(&err, ps.sb.err, 4, cudaMemcpyDeviceToHost));
  if (err) {
    set_error("gdn_fused_host: device error word = " + std::to_string(err));
    return LING_B200_ERR_DEVICE_FLAG;
  }
  LB_CUDA(cudaMemcpy(pre, d_pre, size_t(n) * C * 4, cudaMemcpyDeviceToHost));
  LB_CUDA(cudaMemcpy(post, d_post, size_t(n) * C * 4, cudaMemcpyDeviceToHost));
  LB_CUDA(cudaMemcpy(core, d_core, size_t(n) * Vs * 4, cudaMemcpyDeviceToHost));
  LB_CUDA(cudaMemcpy(out_codes, d_codes, size_t(n) * Vs, cudaMemcpyDeviceToHost));
  std::vector<float> sc_host(size_t(KB) * d.rows_alloc);
  LB_CUDA(cudaMemcpy(sc_host.data(), d_scales, sc_host.size() * 4, cudaMemcpyDeviceToHost));
  for (int m = 0; m < n; ++m)
    for (int b = 0; b < KB; ++b) out_scales[size_t(m) * KB + b] = sc_host[size_t(b) * d.rows_alloc + m];
  return LING_B200_OK;
}

int ling_b200_gdn_commit_host(int device, int Hk, int HV, int Dk, int Dv, const int* path, int n, int rows, const float* pre,
                              const float* post, const float* g, const float* beta, float* state, float* conv) {
  if (!path || !pre || !post || !g || !beta || !state || !conv || !gdn_dims_ok(Hk, HV, Dk, Dv) || n < 1 || n > kTreeRows ||
      rows < 1 || rows > kTreeRows) {
    set_error("gdn_commit_host: bad argument");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(check_device(device));
  Scratch sc;
  OneSeq o;
  ling_b200_seq_result res{};
  res.status = 0, res.n_path = n;
  for (int j = 0; j < n; ++j) res.path[j] = path[j];
  LB_TRY(o.build(sc, Hk, HV, Dk, Dv, rows, 0, nullptr, &res));
  const int C = o.d.C;
  float* d_pre = sc.put(pre, size_t(rows) * C);
  float* d_post = sc.put(post, size_t(rows) * C);
  float* d_g = sc.put(g, size_t(rows) * HV);
  float* d_b = sc.put(beta, size_t(rows) * HV);
  float* d_state = sc.put(state, size_t(HV) * Dk * Dv);
  float* d_conv = sc.put(conv, size_t(C) * 3);
  LB_PTR(d_pre && d_post && d_g && d_b && d_state && d_conv);
  LB_TRY(conv_commit_launch(o.sb, o.d, d_pre, 0, d_conv, 0, 0, 0));
  LB_TRY(gdn_commit_launch(o.sb, o.d, d_post, d_g, d_b, 0, 0, d_state, 0, 0, 148 * 4, 0));
  LB_CUDA(cudaDeviceSynchronize());
  LB_CUDA(cudaMemcpy(state, d_state, size_t(HV) * Dk * Dv * 4, cudaMemcpyDeviceToHost));
  LB_CUDA(cudaMemcpy(conv, d_conv, size_t(C) * 3 * 4, cudaMemcpyDeviceToHost));
  return LING_B200_OK;
}

int ling_b200_argmax_host(int device, const float* logits, int rows, int vocab, int* ids, float* vals) {
  if (!logits || !ids || !vals || rows < 1 || vocab < 1) {
    set_error("argmax_host: bad argument");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(check_device(device));
  Scratch sc;
  float* d_l = sc.put(logits, size_t(rows) * vocab);
  int* d_i = sc.get<int>(rows);
  float* d_v = sc.get<float>(rows);
  LB_PTR(d_l && d_i && d_v);
  LB_TRY(argmax_rows_launch(d_l, rows, vocab, d_i, d_v, 0));
  LB_CUDA(cudaDeviceSynchronize());
  LB_CUDA(cudaMemcpy(ids, d_i, size_t(rows) * 4, cudaMemcpyDeviceToHost));
  LB_CUDA(cudaMemcpy(vals, d_v, size_t(rows) * 4, cudaMemcpyDeviceToHost));
  return LING_B200_OK;
}

// topk_rows (src/core/topk.cu:83-129) over host rows.
int ling_b200_topk_rows_host(int device, const float* x, int rows, int vocab, int k, float* vals, int* ids) {
  if (!x || !ids || !vals || rows < 1 || vocab < 1 || k < 1 || k > kTopMaxK) {
    set_error("topk_rows_host: bad argument (1 <= k <= 64)");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(check_device(device));
  Scratch sc;
  float* d_x = sc.put(x, size_t(rows) * vocab);
  float* d_s = sc.get<float>(topk_scratch_floats(rows, vocab, k));
  int* d_i = sc.get<int>(size_t(rows) * k);
  float* d_v = sc.get<float>(size_t(rows) * k);
  LB_PTR(d_x && d_s && d_i && d_v);
  LB_TRY(topk_rows_launch(d_x, rows, vocab, k, d_s, d_v, d_i, 0));
  LB_CUDA(cudaDeviceSynchronize());
  LB_CUDA(cudaMemcpy(ids, d_i, size_t(rows) * k * 4, cudaMemcpyDeviceToHost));
  LB_CUDA(cudaMemcpy(vals, d_v, size_t(rows) * k * 4, cudaMemcpyDeviceToHost));
  return LING_B200_OK;
}

// The sparse head's selection over host buffers (sparse_head_select, src/core/kernels.cuh:296-306): p [M][256] fp32, us [N][256]
// BF16, n_masks masks of N bytes each (one after the other); rows [cap] and *nrows out; keys (may be NULL) [N]: the 32-bit keys
// the selection ranks (0 = marked).
int ling_b200_sparse_select_host(int device, const float* p, int M, const uint16_t* us_bf16, int N, const uint8_t* masks, int n_masks,
                                 int dynamic, int cap, int* rows, int* nrows, uint32_t* keys) {
  if (!p || !us_bf16 || !masks || !rows || !nrows || M < 1 || M > 32 || N < 1 || n_masks < 1 || n_masks > kSparseMasks || cap < 1 || dynamic < 0) {
    set_error("sparse_select_host: bad argument (1 <= M <= 32, 1 to 4 masks)");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(check_device(device));
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  Scratch sc;
  float* d_p = sc.put(p, size_t(M) * kSelRank);
  auto* d_us = reinterpret_cast<__nv_bfloat16*>(sc.put(us_bf16, size_t(N) * kSelRank));
  uint8_t* d_m = sc.put(masks, size_t(n_masks) * N);
  uint8_t* d_s = sc.get<uint8_t>(sparse_scratch_bytes(N));
  int* d_rows = sc.get<int>(size_t(cap));
  int* d_n = sc.get<int>(1);
  LB_PTR(d_p && d_us && d_m && d_s && d_rows && d_n);
  SparseMasks ms;
  ms.n = n_masks;
  for (int i = 0; i < kSparseMasks; ++i) ms.m[i] = d_m + size_t(i < n_masks ? i : 0) * N;
  int* d_err = sc.get<int>(1);
  LB_PTR(d_err);
  LB_TRY(sparse_select_launch(d_p, M, d_us, N, ms, dynamic, cap, d_s, sms, d_rows, d_n, d_err, 0));
  LB_CUDA(cudaDeviceSynchronize());
  {
    int code = 0;
    LB_CUDA(cudaMemcpy(&code, d_err, 4, cudaMemcpyDeviceToHost));
    if (code) {
      set_error("sparse_select: device error word = " + std::to_string(code));
      return LING_B200_ERR_DEVICE_FLAG;
    }
  }
  LB_CUDA(cudaMemcpy(nrows, d_n, 4, cudaMemcpyDeviceToHost));
  if (*nrows > 0) LB_CUDA(cudaMemcpy(rows, d_rows, size_t(*nrows) * 4, cudaMemcpyDeviceToHost));
  if (keys) LB_CUDA(cudaMemcpy(keys, d_s, size_t(N) * 4, cudaMemcpyDeviceToHost));
  return LING_B200_OK;
}

// Timing aid: the selection on synthetic factors resident in HBM (N rows, M step rows, 2 % of the rows marked), `iters` times
// after a warm-up: ms[0] the scores kernel alone (it reads us once: N x 512 bytes), ms[1] the whole selection (scores, three
// radix levels, count / scan / scatter).
int ling_b200_sparse_select_bench(int device, int N, int M, int dynamic, int cap, int iters, float ms[2]) {
  if (!ms || N < 1 || M < 1 || M > 32 || iters < 1 || cap < 1 || dynamic < 0) {
    set_error("sparse_select_bench: bad argument");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(check_device(device));
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  const size_t n_us = size_t(N) * kSelRank, n_p = size_t(M) * kSelRank, n_mask = size_t(N);
  std::vector<uint16_t> us(n_us);
  std::vector<float> p(n_p);
  std::vector<uint8_t> mask(n_mask);
  uint64_t r = 0x9E3779B97F4A7C15ull;
  auto next = [&]() { return r = r * 6364136223846793005ull + 1442695040888963407ull; };
  for (auto& v : us) v = uint16_t(0x3c00 + ((next() >> 40) & 0x83ff));  // BF16 values of magnitude ~0.01, both signs
  for (auto& v : p) v = float(int((next() >> 40) & 0xffff) - 32768) / 32768.f;
  for (auto& v : mask) v = (next() >> 40) % 50 == 0;
  Scratch sc;
  float* d_p = sc.put(p.data(), p.size());
  // three copies of the factor, read in turn: the working set (3 x 127 MB at the 27B vocabulary) is then larger than L2, so a
  // launch finds little of its copy there
  __nv_bfloat16* d_us[3];
  for (auto& u : d_us) u = reinterpret_cast<__nv_bfloat16*>(sc.put(us.data(), us.size()));
  uint8_t* d_m = sc.put(mask.data(), mask.size());
  uint8_t* d_s = sc.get<uint8_t>(sparse_scratch_bytes(N));
  int* d_rows = sc.get<int>(size_t(cap));
  int* d_n = sc.get<int>(1);
  LB_PTR(d_p && d_us[0] && d_us[1] && d_us[2] && d_m && d_s && d_rows && d_n);
  SparseMasks msk;
  msk.n = 1;
  for (int i = 0; i < kSparseMasks; ++i) msk.m[i] = d_m;
  cudaEvent_t a, b;
  LB_CUDA(cudaEventCreate(&a));
  LB_CUDA(cudaEventCreate(&b));
  for (int part = 0; part < 2; ++part) {
    LB_TRY(sparse_select_launch(d_p, M, d_us[0], N, msk, dynamic, cap, d_s, sms, d_rows, d_n, nullptr, 0, part == 0));
    LB_CUDA(cudaEventRecord(a, 0));
    for (int i = 0; i < iters; ++i) LB_TRY(sparse_select_launch(d_p, M, d_us[(i + 1) % 3], N, msk, dynamic, cap, d_s, sms, d_rows, d_n, nullptr, 0, part == 0));
    LB_CUDA(cudaEventRecord(b, 0));
    LB_CUDA(cudaEventSynchronize(b));
    LB_CUDA(cudaEventElapsedTime(&ms[part], a, b));
    ms[part] /= iters;
  }
  cudaEventDestroy(a), cudaEventDestroy(b);
  return LING_B200_OK;
}

// The candidate selector over host buffers: its projection (x [E][hidden] . W^T, W [256][hidden] BF16) when x and W are
// given (else hp is an input), then selector_lattice (src/core/draft_kernels.cu:328-351).
int ling_b200_selector_lattice_host(int device, const float* x, const uint16_t* proj_bf16, int hidden, float* hp, const int* cand,
                                    const float* unary, const uint16_t* pred_bf16, const uint16_t* succ_bf16, int vocab, int anchor,
                                    int E, float* scores) {
  if (!hp || !cand || !unary || !pred_bf16 || !succ_bf16 || !scores || E < 1 || vocab < 1 || (x && (!proj_bf16 || hidden % 256 != 0))) {
    set_error("selector_lattice_host: bad argument");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(check_device(device));
  Scratch sc;
  float* d_hp = x ? sc.get<float>(size_t(E) * kSelRank) : sc.put(hp, size_t(E) * kSelRank);
  const int* d_c = sc.put(cand, size_t(E) * kSelTop);
  const float* d_u = sc.put(unary, size_t(E) * kSelTop);
  const auto* d_p = reinterpret_cast<const __nv_bfloat16*>(sc.put(pred_bf16, size_t(vocab) * kSelRank));
  const auto* d_s = reinterpret_cast<const __nv_bfloat16*>(sc.put(succ_bf16, size_t(vocab) * kSelRank));
  float* d_o = sc.get<float>(size_t(E) * kSelTop * kSelTop);
  int* d_err = sc.get<int>(1);
  LB_PTR(d_hp && d_c && d_u && d_p && d_s && d_o && d_err);
  if (x) {
    const float* d_x = sc.put(x, size_t(E) * hidden);
    const auto* d_w = reinterpret_cast<const __nv_bfloat16*>(sc.put(proj_bf16, size_t(kSelRank) * hidden));
    LB_PTR(d_x && d_w);
    LB_TRY(selector_project_launch(d_x, d_w, E, hidden, d_hp, 0));
  }
  LB_TRY(selector_lattice_launch(d_hp, d_c, d_u, d_p, d_s, vocab, anchor, nullptr, E, d_o, d_err, 0));
  LB_CUDA(cudaDeviceSynchronize());
  int err = 0;
  LB_CUDA(cudaMemcpy(&err, d_err, 4, cudaMemcpyDeviceToHost));
  LB_CUDA(cudaMemcpy(scores, d_o, size_t(E) * kSelTop * kSelTop * 4, cudaMemcpyDeviceToHost));
  if (x) LB_CUDA(cudaMemcpy(hp, d_hp, size_t(E) * kSelRank * 4, cudaMemcpyDeviceToHost));
  if (err) {
    set_error("selector_lattice_host: a candidate or the anchor is not a token id (device error word = " + std::to_string(err) + ")");
    return LING_B200_ERR_DEVICE_FLAG;
  }
  return LING_B200_OK;
}

// The prefill path's DeltaNet mixer core over host buffers: conv over the rows, then the chunked delta rule.
int ling_b200_gdn_prefill_host(int device, int Hk, int HV, int Dk, int Dv, int M, const float* pre, const uint16_t* convw_bf16,
                               const float* g, const float* beta, float* state, float* conv, float* post, float* core) {
  if (!pre || !convw_bf16 || !g || !beta || !state || !conv || !core || M < 1 || Hk < 1 || HV < 1 || HV % Hk != 0 || Dk != 128 || Dv != 128) {
    set_error("gdn_prefill_host: bad argument (key dim = value dim = 128)");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(check_device(device));
  LB_TRY(gdn_chunk_init());
  const int C = 2 * Hk * Dk + HV * Dv;
  Scratch sc;
  const float* d_pre = sc.put(pre, size_t(M) * C);
  const auto* d_w = reinterpret_cast<const __nv_bfloat16*>(sc.put(convw_bf16, size_t(C) * 4));
  const float* d_g = sc.put(g, size_t(M) * HV);
  const float* d_b = sc.put(beta, size_t(M) * HV);
  float* d_state = sc.put(state, size_t(HV) * Dk * Dv);
  float* d_conv = sc.put(conv, size_t(C) * 3);
  float* d_post = sc.get<float>(size_t(M) * C);
  float* d_core = sc.get<float>(size_t(M) * HV * Dv);
  uint8_t* d_scr = sc.get<uint8_t>(gdn_chunk_scratch_bytes(M, HV), false);
  LB_PTR(d_pre && d_w && d_g && d_b && d_state && d_conv && d_post && d_core && d_scr);
  LB_TRY(conv_rows_launch(d_pre, d_w, d_conv, M, C, d_post, 0));
  LB_TRY(gdn_chunk_launch(d_post, d_g, d_b, M, Hk, HV, Dk, Dv, d_state, d_core, d_scr, 0));
  LB_CUDA(cudaDeviceSynchronize());
  LB_CUDA(cudaMemcpy(state, d_state, size_t(HV) * Dk * Dv * 4, cudaMemcpyDeviceToHost));
  LB_CUDA(cudaMemcpy(conv, d_conv, size_t(C) * 3 * 4, cudaMemcpyDeviceToHost));
  LB_CUDA(cudaMemcpy(core, d_core, size_t(M) * HV * Dv * 4, cudaMemcpyDeviceToHost));
  if (post) LB_CUDA(cudaMemcpy(post, d_post, size_t(M) * C * 4, cudaMemcpyDeviceToHost));
  return LING_B200_OK;
}

// Device time of the chunked delta rule alone over M rows of synthetic inputs (ms per launch).
int ling_b200_gdn_chunk_bench(int device, int Hk, int HV, int M, int iters, float* ms) {
  if (M < 1 || Hk < 1 || HV % Hk != 0 || iters < 1 || !ms) {
    set_error("gdn_chunk_bench: bad argument");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(check_device(device));
  LB_TRY(gdn_chunk_init());
  const int C = 2 * Hk * 128 + HV * 128;
  Scratch sc;
  float* d_post = sc.get<float>(size_t(M) * C, false);
  float* d_g = sc.get<float>(size_t(M) * HV, false);
  float* d_b = sc.get<float>(size_t(M) * HV, false);
  float* d_state = sc.get<float>(size_t(HV) * 128 * 128);
  float* d_core = sc.get<float>(size_t(M) * HV * 128, false);
  uint8_t* d_scr = sc.get<uint8_t>(gdn_chunk_scratch_bytes(M, HV), false);
  LB_PTR(d_post && d_g && d_b && d_state && d_core && d_scr);
  LB_TRY(fill_f32_launch(stream_key(1, 1), 1.f, d_post, size_t(M) * C, 0));
  LB_TRY(fill_f32_launch(stream_key(1, 2), 0.05f, d_g, size_t(M) * HV, 0));  // log-decays near 0 (|g| small), signs mixed
  LB_TRY(fill_f32_launch(stream_key(1, 3), 0.2f, d_b, size_t(M) * HV, 0));
  cudaEvent_t a, b;
  LB_CUDA(cudaEventCreate(&a));
  LB_CUDA(cudaEventCreate(&b));
  LB_TRY(gdn_chunk_launch(d_post, d_g, d_b, M, Hk, HV, 128, 128, d_state, d_core, d_scr, 0));
  LB_CUDA(cudaMemsetAsync(d_state, 0, size_t(HV) * 128 * 128 * 4, 0));
  LB_CUDA(cudaEventRecord(a, 0));
  for (int i = 0; i < iters; ++i) LB_TRY(gdn_chunk_launch(d_post, d_g, d_b, M, Hk, HV, 128, 128, d_state, d_core, d_scr, 0));
  LB_CUDA(cudaEventRecord(b, 0));
  LB_CUDA(cudaEventSynchronize(b));
  float t = 0;
  LB_CUDA(cudaEventElapsedTime(&t, a, b));
  cudaEventDestroy(a), cudaEventDestroy(b);
  *ms = t / iters;
  return LING_B200_OK;
}

}  // extern "C"
