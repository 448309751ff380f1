// ling_oracle.cpp -- CPU oracle of the ragged speculative verify step.  TEST INFRASTRUCTURE ONLY: the product
// never links, loads or calls it (see ling_oracle.h for what it is pinned against and what stays unpinned).
//
// Each function names the reference (dreamference/ling-engine) file:line whose arithmetic it restates.  The
// numerics that the reference does not have (FP8 E4M3 KV with one fp32 scale per (position, head), FP8 weights
// and activations with one fp32 scale per 1x128 block) are defined here:
//   scale = amax / 448 (1 when the block is all zero), code = E4M3(x / scale) round-to-nearest-even, saturating;
//   a GEMM output is the sum over 128-wide K blocks of (dot of the codes) * act_scale * weight_scale.
// Dot products are accumulated in double so that the oracle is the accurate side of every tolerance check.
#include "ling_oracle.h"

#include <algorithm>
#include <cfloat>
#include <cmath>
#include <cstring>
#include <vector>
#include <functional>
#include <thread>

namespace {

int g_threads = 1;

// A static split of [0, n) over g_threads std::threads (no OpenMP runtime is assumed on the host).
void parallel_for(int n, const std::function<void(int, int)>& body) {
  const int t = std::max(1, std::min(g_threads, n));
  if (t == 1) return body(0, n);
  std::vector<std::thread> pool;
  for (int i = 0; i < t; ++i) {
    const int lo = int(int64_t(n) * i / t), hi = int(int64_t(n) * (i + 1) / t);
    pool.emplace_back([=, &body] { body(lo, hi); });
  }
  for (std::thread& th : pool) th.join();
}

// ---------------------------------------------------------------------------------------------- formats
float g_dec[256];
bool g_dec_ready = false;
void init_dec() {
  if (g_dec_ready) return;
  for (int c = 0; c < 256; ++c) {
    const int s = c >> 7, e = (c >> 3) & 15, m = c & 7;
    float v;
    if (e == 15 && m == 7) v = NAN;
    else if (e == 0) v = std::ldexp(float(m), -9);
    else v = std::ldexp(1.f + m / 8.f, e - 7);
    g_dec[c] = s ? -v : v;
  }
  g_dec_ready = true;
}

// E4M3 (4 exponent bits, bias 7, 3 mantissa bits, no inf, max 448), round to nearest even, saturating:
// the conversion __nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3) performs
// (reference use: src/core/prefill_gemm.cu:396-402).
uint8_t e4m3(float x) {
  const uint8_t sign = std::signbit(x) ? 0x80 : 0;
  if (std::isnan(x)) return sign | 0x7f;
  const float a = std::fabs(x);
  if (a >= 448.f) return sign | 0x7e;
  if (a < 0.015625f) {  // below 2^-6: subnormal, spacing 2^-9
    const int q = int(std::nearbyint(a * 512.f));
    return sign | uint8_t(q);  // q == 8 is the smallest normal's code
  }
  int e;
  const float fr = std::frexp(a, &e);  // a = fr * 2^e, fr in [0.5, 1)
  int q = int(std::nearbyint((fr * 2.f - 1.f) * 8.f));
  int ex = e - 1;
  if (q == 8) {
    q = 0;
    ++ex;
  }
  int code = ((ex + 7) << 3) | q;
  if (code > 0x7e) code = 0x7e;
  return sign | uint8_t(code);
}

float bf16r(float x) {  // round to nearest even to BF16 (__float2bfloat16)
  uint32_t u;
  std::memcpy(&u, &x, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return x;
  u += 0x7fffu + ((u >> 16) & 1u);
  u &= 0xffff0000u;
  float r;
  std::memcpy(&r, &u, 4);
  return r;
}

// One fp32 scale per row per 128 columns; the last block may be short.
void quant_rows(const float* x, int rows, int cols, bool bf16_first, uint8_t* codes, float* scales) {
  const int KB = (cols + 127) / 128;
  parallel_for(rows, [&](int r_lo, int r_hi) {
  for (int r = r_lo; r < r_hi; ++r)
    for (int b = 0; b < KB; ++b) {
      const int k0 = b * 128, k1 = std::min(cols, k0 + 128);
      float amax = 0.f;
      for (int k = k0; k < k1; ++k) {
        const float v = bf16_first ? bf16r(x[size_t(r) * cols + k]) : x[size_t(r) * cols + k];
        amax = std::max(amax, std::fabs(v));
      }
      const float sc = amax > 0.f ? amax / 448.f : 1.f;
      scales[size_t(r) * KB + b] = sc;
      for (int k = k0; k < k1; ++k) {
        const float v = bf16_first ? bf16r(x[size_t(r) * cols + k]) : x[size_t(r) * cols + k];
        codes[size_t(r) * cols + k] = e4m3(v / sc);
      }
    }
  });
}

// ---------------------------------------------------------------------------------------------- generator
// Counter based: element i of stream s under seed is a function of (seed, s, i) alone, so any slice can be
// regenerated.  z ~ N(0,1) as the centred sum of twelve 16-bit uniforms (integer arithmetic: exact everywhere).
inline uint64_t mix(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}
inline float synth_z(uint64_t key, uint64_t i) {
  int s = 0;
  for (int j = 0; j < 3; ++j) {
    const uint64_t h = mix(key + 3 * i + j);
    s += int(h & 0xffff) + int((h >> 16) & 0xffff) + int((h >> 32) & 0xffff) + int((h >> 48) & 0xffff);
  }
  return float(2 * s - 786420) * (1.0f / 131072.0f);
}
inline uint64_t stream_key(uint64_t seed, uint64_t stream) { return mix(seed ^ mix(stream)); }

enum : uint64_t { kStreamKv = 1ull << 32, kStreamState = 2ull << 32, kStreamConv = 3ull << 32 };

// ---------------------------------------------------------------------------------------------- tensors
enum {
  T_EMBED = 0, T_FINAL_NORM, T_LM_HEAD, T_INPUT_NORM, T_POST_NORM, T_GATE, T_UP, T_DOWN, T_IN_QKV, T_IN_Z, T_OUT,
  T_IN_A, T_IN_B, T_CONV, T_A_LOG, T_DT_BIAS, T_LIN_NORM, T_Q, T_K, T_V, T_O, T_Q_NORM, T_K_NORM, T_COUNT
};

struct Mat {
  int N = 0, K = 0, KB = 0;
  std::vector<uint8_t> codes;  // [N][K]
  std::vector<float> scales;   // [N][KB]
  void set(const float* w, int n, int k) {
    N = n, K = k, KB = (k + 127) / 128;
    codes.resize(size_t(n) * k);
    scales.resize(size_t(n) * KB);
    quant_rows(w, n, k, true, codes.data(), scales.data());
  }
};

struct Layer {
  bool full = false;
  std::vector<float> input_norm, post_norm;
  Mat gate, up, down, in_qkv, in_z, out, q, k, v, o;
  std::vector<float> in_a, in_b, conv, A_log, dt_bias, lin_norm, q_norm, k_norm;
};

struct QAct {  // activations quantized per row per 128 columns, decoded to float for the dot products
  int M = 0, K = 0, KB = 0;
  std::vector<float> val;  // decoded codes
  std::vector<float> scales;
  void set(const float* x, int m, int k) {
    M = m, K = k, KB = (k + 127) / 128;
    std::vector<uint8_t> codes(size_t(m) * k);
    scales.resize(size_t(m) * KB);
    quant_rows(x, m, k, false, codes.data(), scales.data());
    val.resize(codes.size());
    for (size_t i = 0; i < codes.size(); ++i) val[i] = g_dec[codes[i]];
  }
};

// y[m][off + n] (row stride ldy) = sum over K blocks of dot(codes) * act_scale * weight_scale
// (the reference's rows-path GEMM, src/core/stream_gemm.cu:181-349, at this build's block-scaled numerics).
// n_limit: only the first n_limit weight rows (the CPU-baseline sample of the LM head).
void gemm(const QAct& a, const Mat& w, float* y, size_t ldy, int off, int n_limit = -1) {
  const int N = n_limit >= 0 ? std::min(n_limit, w.N) : w.N, K = w.K, KB = w.KB, M = a.M;
  parallel_for(N, [&](int n_lo, int n_hi) {
    std::vector<float> wrow(K);
    for (int n = n_lo; n < n_hi; ++n) {
      const uint8_t* wc = w.codes.data() + size_t(n) * K;
      for (int k = 0; k < K; ++k) wrow[k] = g_dec[wc[k]];
      for (int m = 0; m < M; ++m) {
        const float* av = a.val.data() + size_t(m) * K;
        double acc = 0;
        for (int b = 0; b < KB; ++b) {
          const int k0 = b * 128, k1 = std::min(K, k0 + 128);
          float s = 0.f;  // products of two E4M3 values are exact in fp32
#pragma omp simd reduction(+ : s)
          for (int k = k0; k < k1; ++k) s += av[k] * wrow[k];
          acc += double(s) * double(a.scales[size_t(m) * KB + b] * w.scales[size_t(n) * KB + b]);
        }
        y[size_t(m) * ldy + off + n] = float(acc);
      }
    }
  });
}

inline float silu(float x) { return x / (1.f + std::exp(-x)); }      // src/core/kernels.cu:38
inline float sigmoid(float x) { return 1.f / (1.f + std::exp(-x)); }  // src/core/kernels.cu:314-318

// Gemma RMSNorm x * rsqrt(mean(x^2) + eps) * (1 + w)  (src/core/kernels.cu:289-301, gemma = true); plain = * w.
void rmsnorm(const float* x, const float* w, float* out, int H, float eps, bool gemma) {
  double ss = 0;
  for (int h = 0; h < H; ++h) ss += double(x[h]) * x[h];
  const float rstd = float(1.0 / std::sqrt(ss / H + double(eps)));
  for (int h = 0; h < H; ++h) out[h] = x[h] * rstd * (gemma ? 1.f + w[h] : w[h]);
}

}  // namespace

struct lo_model {
  lo_model_config cfg{};
  lo_options opt{};
  int n_attn = 0, n_gdn = 0;
  std::vector<int> attn_index, gdn_index;  // per layer: index among its kind
  std::vector<Layer> layers;
  std::vector<float> embed, final_norm;  // embed as BF16 values
  Mat head;
  // sessions
  std::vector<std::vector<int>> tables;       // [slot][max_pages]
  std::vector<uint8_t> kv_codes;              // [attn][K|V][head][page][tok][D]
  std::vector<float> kv_scales;               // [attn][K|V][head][page][tok]
  std::vector<std::vector<float>> gdn_state;  // [slot * n_gdn + l] -> [HV][Dk][Dv]
  std::vector<std::vector<float>> conv_state; // [slot * n_gdn + l] -> [C][3]
  // last step
  int n_seqs = 0, rows = 0;
  std::vector<int> row0, token, seq_of, depth, rope_pos, cache_slot, argmax_id;
  std::vector<uint32_t> anc;
  std::vector<float> argmax_val, logits;
  std::vector<lo_tree_desc> trees;
  std::vector<std::vector<float>> taps;

  int C() const { return 2 * cfg.lin_k_heads * cfg.lin_k_dim + cfg.lin_v_heads * cfg.lin_v_dim; }
  int Vs() const { return cfg.lin_v_heads * cfg.lin_v_dim; }
  int max_pages() const { return (opt.max_context + opt.page_tokens - 1) / opt.page_tokens; }
  // [layer][K|V][kv head][page][token][D]: the reference's head-major pool (src/core/engine.cpp:175-207).
  size_t kv_index(int al, int kv, int h, int page, int tok) const {
    return ((((size_t(al) * 2 + kv) * cfg.kv_heads + h) * (opt.pool_pages + 1) + page) * opt.page_tokens + tok);
  }
};

extern "C" {

void lo_set_threads(int n) { g_threads = std::max(1, n); }
int lo_threads(void) { return g_threads; }
uint8_t lo_e4m3_encode(float x) { return e4m3(x); }
float lo_e4m3_decode(uint8_t c) {
  init_dec();
  return g_dec[c];
}
float lo_bf16_round(float x) { return bf16r(x); }
void lo_quant_rows(const float* x, int rows, int cols, int bf16_first, uint8_t* codes, float* scales) {
  quant_rows(x, rows, cols, bf16_first != 0, codes, scales);
}
void lo_synth(uint64_t seed, uint64_t stream, size_t offset, size_t n, float std_, float bias, int bf16, float* out) {
  const uint64_t key = stream_key(seed, stream);
  const int chunks = int(std::min<size_t>(n / 4096 + 1, 1 << 20));
  parallel_for(chunks, [&](int c_lo, int c_hi) {
    const size_t lo = n * size_t(c_lo) / chunks, hi = n * size_t(c_hi) / chunks;
    for (size_t i = lo; i < hi; ++i) {
      const float v = synth_z(key, offset + i) * std_ + bias;
      out[i] = bf16 ? bf16r(v) : v;
    }
  });
}
uint64_t lo_weight_stream(int layer, int tensor) { return uint64_t(layer + 1) * 64 + uint64_t(tensor); }

// ---------------------------------------------------------------------------------------------- host logic

// describe_tree (src/core/tree.cpp:81-146).  Variants: one per leaf in row order, path[v][d] = the leaf's ancestor
// at depth d; a row's variant is the leaf reached through first children.  DeltaNet paths: the chain first, then
// one per internal row no earlier path covered (root .. that row, continued through first internal children);
// along a path a node advances the state and is followed by its leaf children (computed from its state without
// advancing it); a row carries the write flag the first time any path emits it.
int lo_describe_tree(const int* parent, int n, int chain, lo_tree_desc* out) {
  if (n < 1 || n > LO_MAX_TREE_ROWS) return 1;
  lo_tree_desc& d = *out;
  std::memset(&d, 0, sizeof d);
  d.n = n;
  std::vector<std::vector<int>> kids(n);
  std::vector<int> dep(n, 0);
  for (int r = 1; r < n; ++r) {
    if (parent[r] < 0 || parent[r] >= r) return 1;
    kids[parent[r]].push_back(r);
    dep[r] = dep[parent[r]] + 1;
  }
  std::vector<int> leaf_variant(n, -1);
  for (int r = 0; r < n; ++r) {
    d.depth[r] = dep[r];
    if (!kids[r].empty()) continue;
    if (d.nvar >= LO_MAX_TREE_VARIANTS) return 1;
    leaf_variant[r] = d.nvar;
    for (int a = r; a >= 0; a = (a == 0 ? -1 : parent[a])) d.path[d.nvar][dep[a]] = a;
    ++d.nvar;
  }
  for (int r = 0; r < n; ++r) {
    int a = r;
    while (!kids[a].empty()) a = kids[a].front();
    d.var[r] = leaf_variant[a];
  }
  std::vector<char> written(n, 0), covered(n, 0);
  auto emit = [&](const std::vector<int>& nodes) {
    int* steps = d.gdn_step[d.ngdn];
    int len = 0;
    for (int w : nodes) {
      steps[len++] = w | (written[w] ? 0 : (1 << 9));
      written[w] = covered[w] = 1;
      for (int c : kids[w])
        if (kids[c].empty() && !written[c]) {
          steps[len++] = c | (1 << 8) | (1 << 9);
          written[c] = covered[c] = 1;
        }
    }
    d.gdn_len[d.ngdn++] = len;
  };
  std::vector<int> nodes;
  for (int r = 0; r <= chain && r < n; ++r) nodes.push_back(r);
  emit(nodes);
  for (int r = 0; r < n; ++r) {
    if (covered[r] || kids[r].empty()) continue;
    nodes.clear();
    for (int a = r; a >= 0; a = (a == 0 ? -1 : parent[a])) nodes.push_back(a);
    std::reverse(nodes.begin(), nodes.end());
    for (int a = r;;) {
      int nxt = -1;
      for (int c : kids[a])
        if (!kids[c].empty()) {
          nxt = c;
          break;
        }
      if (nxt < 0) break;
      nodes.push_back(nxt);
      a = nxt;
    }
    if (d.ngdn >= LO_MAX_TREE_VARIANTS) return 1;
    emit(nodes);
  }
  for (int r = 0; r < n; ++r)
    if (!written[r]) return 1;
  return 0;
}

// accept_tree_greedy (src/core/tree.cpp:148-166): from the root, take the first child (row order) whose token is
// the current row's argmax; stop when there is none, `next` is that argmax.
int lo_accept_tree_greedy(const int* parent, const int* token, int n, const int* argmax, int* path, int* next) {
  int len = 0, u = 0;
  path[len++] = 0;
  for (;;) {
    const int x = argmax[u];
    int child = -1;
    for (int c = u + 1; c < n; ++c)
      if (parent[c] == u && token[c] == x) {
        child = c;
        break;
      }
    if (child < 0) {
      *next = x;
      return len;
    }
    path[len++] = child;
    u = child;
  }
}

// lookup_propose (src/core/lookup.cpp:7-24): the continuation of the most recent earlier occurrence of the last
// `ngram` tokens (the occurrence must leave a token after it), at most `max` tokens; match = how far back the
// agreement reaches, capped at 64.
int lo_lookup_propose(const int* s, int L, int max, int ngram, int* out, int* match) {
  *match = 0;
  if (L <= ngram || max <= 0) return 0;
  for (int i = L - ngram - 1; i >= 0; --i) {
    bool same = true;
    for (int j = 0; j < ngram && same; ++j) same = s[i + j] == s[L - ngram + j];
    if (!same) continue;
    int m = ngram;
    while (m < 64) {
      const int a = i - (m - ngram) - 1, b = L - m - 1;
      if (a < 0 || s[a] != s[b]) break;
      ++m;
    }
    const int start = i + ngram, n = std::min(max, L - start);
    for (int j = 0; j < n; ++j) out[j] = s[start + j];
    *match = m;
    return n;
  }
  return 0;
}

// ---------------------------------------------------------------------------------------------- kernels

void lo_gemm_fp8(const float* x, const float* w, float* y, int M, int N, int K) {
  init_dec();
  Mat wm;
  wm.set(w, N, K);
  QAct a;
  a.set(x, M, K);
  gemm(a, wm, y, N, 0);
}

namespace {
// One token of the gated delta rule on one head's state S[Dk][Dv] (k-major), src/core/kernels.cu:402-453:
// q, k L2-normalized (eps 1e-6), q also scaled by 1/sqrt(Dk); S *= decay; kv = S^T k; d = (v - kv) * beta;
// S += k d^T; o = S^T q.  advance = false: the leaf rule (src/core/attention_body.cuh:575-603), S untouched.
void delta_step(float* S, int Dk, int Dv, const float* q, const float* k, const float* v, float g, float beta,
                float* o, bool advance) {
  double qn = 0, kn = 0;
  for (int i = 0; i < Dk; ++i) qn += double(q[i]) * q[i], kn += double(k[i]) * k[i];
  const float qr = float(1.0 / std::sqrt(qn + 1e-6)) / std::sqrt(float(Dk)), kr = float(1.0 / std::sqrt(kn + 1e-6));
  const float decay = std::exp(g);
  std::vector<float> Sd;
  float* T = S;
  if (!advance) {
    Sd.assign(S, S + size_t(Dk) * Dv);
    T = Sd.data();
  }
  for (size_t i = 0; i < size_t(Dk) * Dv; ++i) T[i] *= decay;
  for (int c = 0; c < Dv; ++c) {
    double kv = 0;
    for (int i = 0; i < Dk; ++i) kv += double(T[size_t(i) * Dv + c]) * double(k[i] * kr);
    const float d = (v[c] - float(kv)) * beta;
    double oo = 0;
    for (int i = 0; i < Dk; ++i) {
      float& s = T[size_t(i) * Dv + c];
      s = std::fma(d, k[i] * kr, s);
      oo += double(s) * double(q[i] * qr);
    }
    o[c] = float(oo);
  }
}

// gdn_conv_tree (src/core/kernels.cu:365-383): taps = raw inputs of the ancestors at depths d-3..d-1 (the variant's
// path) or the window [c][0..2] (oldest first) before depth 0; tap 3 multiplies the row itself; then SiLU.
void conv_tree(const lo_tree_desc& td, const float* pre, const float* convw, const float* win, float* post, int C) {
  for (int t = 0; t < td.n; ++t) {
    const int d = td.depth[t];
    const int* path = td.path[td.var[t]];
    for (int c = 0; c < C; ++c) {
      float tap[3];
      for (int j = 0; j < 3; ++j) {
        const int dj = d - 3 + j;
        tap[j] = dj >= 0 ? pre[size_t(path[dj]) * C + c] : win[c * 3 + 3 + dj];
      }
      const float* w = convw + size_t(c) * 4;
      const float o = w[0] * tap[0] + w[1] * tap[1] + w[2] * tap[2] + w[3] * pre[size_t(t) * C + c];
      post[size_t(t) * C + c] = silu(o);
    }
  }
}

// gdn_recurrent_tree (src/core/kernels.cu:455-477; body src/core/attention_body.cuh:535-606): every DeltaNet path
// walked from the session's state (unwritten), rows written where flagged.
void recurrent_tree(const lo_tree_desc& td, const float* post, const float* g, const float* beta, const float* state,
                    float* core, int Hk, int HV, int Dk, int Dv) {
  const int C = 2 * Hk * Dk + HV * Dv;
  parallel_for(HV, [&](int hv_lo, int hv_hi) {
  for (int hv = hv_lo; hv < hv_hi; ++hv) {
    const int h = hv / (HV / Hk);
    std::vector<float> S(size_t(Dk) * Dv), o(Dv);
    for (int p = 0; p < td.ngdn; ++p) {
      std::copy(state + size_t(hv) * Dk * Dv, state + size_t(hv + 1) * Dk * Dv, S.begin());
      for (int i = 0; i < td.gdn_len[p]; ++i) {
        const int st = td.gdn_step[p][i], t = st & 0xff;
        const bool leaf = st & (1 << 8), write = st & (1 << 9);
        const float* row = post + size_t(t) * C;
        delta_step(S.data(), Dk, Dv, row + h * Dk, row + Hk * Dk + h * Dk, row + 2 * Hk * Dk + hv * Dv,
                   g[t * HV + hv], beta[t * HV + hv], o.data(), !leaf);
        if (write) std::copy(o.begin(), o.end(), core + size_t(t) * HV * Dv + size_t(hv) * Dv);
      }
    }
  }
  });
}
}  // namespace

void lo_gdn_tree(int Hk, int HV, int Dk, int Dv, const lo_tree_desc* td, const float* pre, const float* convw,
                 const float* g, const float* beta, const float* state, const float* conv, float* post, float* core) {
  const int C = 2 * Hk * Dk + HV * Dv;
  conv_tree(*td, pre, convw, conv, post, C);
  recurrent_tree(*td, post, g, beta, state, core, Hk, HV, Dk, Dv);
}

// gdn_conv_prefill + gdn_recurrent_prefill (src/core/kernels.cuh:445-456): the conv over M rows in order (taps before row 0
// from the window, which then holds the last three raw inputs) and the delta rule token by token from the session's state,
// which advances.  The reference's prefill kernel computes the same recurrence chunk-wise in FP16 products; this is the
// exact token form it is unrolled from (src/core/prefill_gdn.cu:75-88), in the oracle's fp32/double arithmetic.
void lo_gdn_prefill(int Hk, int HV, int Dk, int Dv, int M, const float* pre, const float* convw, const float* g, const float* beta,
                    float* state, float* conv, float* post, float* core) {
  const int C = 2 * Hk * Dk + HV * Dv;
  for (int t = 0; t < M; ++t)
    for (int c = 0; c < C; ++c) {
      float x[4];
      for (int j = 0; j < 4; ++j) {
        const int tt = t - 3 + j;
        x[j] = tt >= 0 ? pre[size_t(tt) * C + c] : conv[c * 3 + 3 + tt];
      }
      const float* w = convw + size_t(c) * 4;
      post[size_t(t) * C + c] = silu(w[0] * x[0] + w[1] * x[1] + w[2] * x[2] + w[3] * x[3]);
    }
  for (int c = 0; c < C; ++c) {
    float s[3];
    for (int j = 0; j < 3; ++j) {
      const int tt = M - 3 + j;
      s[j] = tt >= 0 ? pre[size_t(tt) * C + c] : conv[c * 3 + 3 + tt];
    }
    for (int j = 0; j < 3; ++j) conv[c * 3 + j] = s[j];
  }
  parallel_for(HV, [&](int hv_lo, int hv_hi) {
    for (int hv = hv_lo; hv < hv_hi; ++hv) {
      const int h = hv / (HV / Hk);
      float* S = state + size_t(hv) * Dk * Dv;
      for (int t = 0; t < M; ++t) {
        const float* row = post + size_t(t) * C;
        delta_step(S, Dk, Dv, row + h * Dk, row + Hk * Dk + h * Dk, row + 2 * Hk * Dk + hv * Dv, g[size_t(t) * HV + hv],
                   beta[size_t(t) * HV + hv], core + size_t(t) * HV * Dv + size_t(hv) * Dv, true);
      }
    }
  });
}

// Engine::commit (src/core/speculate.cpp:516-529): the accepted rows path[0..n) replayed in order; the conv window
// advances over their raw inputs (src/core/kernels.cu:320-338), the recurrence over their conv outputs, both written.
void lo_gdn_commit(int Hk, int HV, int Dk, int Dv, const int* path, int n, int rows, const float* pre,
                   const float* post, const float* g, const float* beta, float* state, float* conv) {
  (void)rows;
  const int C = 2 * Hk * Dk + HV * Dv;
  for (int j = 0; j < n; ++j) {
    const int t = path[j];
    for (int c = 0; c < C; ++c) {
      conv[c * 3] = conv[c * 3 + 1];
      conv[c * 3 + 1] = conv[c * 3 + 2];
      conv[c * 3 + 2] = pre[size_t(t) * C + c];
    }
  }
  parallel_for(HV, [&](int hv_lo, int hv_hi) {
  for (int hv = hv_lo; hv < hv_hi; ++hv) {
    const int h = hv / (HV / Hk);
    std::vector<float> o(Dv);
    for (int j = 0; j < n; ++j) {
      const int t = path[j];
      const float* row = post + size_t(t) * C;
      delta_step(state + size_t(hv) * Dk * Dv, Dk, Dv, row + h * Dk, row + Hk * Dk + h * Dk,
                 row + 2 * Hk * Dk + hv * Dv, g[t * HV + hv], beta[t * HV + hv], o.data(), true);
    }
  }
  });
}

// topk_rows with K = 1 (src/core/topk.cu:19,58,83-129): larger value first, equal values to the lower index, NaN
// skipped; a row with no candidate comes back as (-FLT_MAX, 0x7fffffff).
void lo_argmax(const float* logits, int rows, int vocab, int* ids, float* vals) {
  for (int r = 0; r < rows; ++r) {
    float bv = -FLT_MAX;
    int bi = 0x7fffffff;
    for (int i = 0; i < vocab; ++i) {
      const float v = logits[size_t(r) * vocab + i];
      if (v != v) continue;
      if (v > bv || (v == bv && i < bi)) bv = v, bi = i;
    }
    ids[r] = bi;
    vals[r] = bv;
  }
}

// topk_rows for K <= 64 (src/core/topk.cu:83-129; kernels.cuh:400-410): per row the K largest values, descending, equal
// values to the lower index, NaN skipped; past the rankable values (-FLT_MAX, 0x7fffffff).
void lo_topk_rows(const float* x, int rows, int vocab, int k, float* vals, int* ids) {
  for (int r = 0; r < rows; ++r) {
    std::vector<std::pair<float, int>> best;  // kept in rank order
    for (int i = 0; i < vocab; ++i) {
      const float v = x[size_t(r) * vocab + i];
      if (v != v || !(v > -FLT_MAX)) continue;
      if (int(best.size()) == k && !(v > best.back().first)) continue;  // equal to the last: the earlier index stays
      size_t at = best.size();
      while (at > 0 && v > best[at - 1].first) --at;
      best.insert(best.begin() + long(at), {v, i});
      if (int(best.size()) > k) best.pop_back();
    }
    for (int j = 0; j < k; ++j) {
      vals[size_t(r) * k + j] = j < int(best.size()) ? best[size_t(j)].first : -FLT_MAX;
      ids[size_t(r) * k + j] = j < int(best.size()) ? best[size_t(j)].second : 0x7fffffff;
    }
  }
}

// The candidate selector (src/core/draft_kernels.cu:328-351): score[e][p][c] = unary[e][c] + sum_r P[pred(e, p)][r] *
// hp[e][r] * S[cand[e][c]][r], pred(0, p) = the anchor, pred(e, p) = cand[e - 1][p]; 16 candidates, rank 256, the codebooks
// rounded to BF16 as the reference keeps them, the sum in double.
void lo_selector_lattice(const float* hp, const int* cand, const float* unary, const float* P, const float* S, int anchor, int E,
                         float* scores) {
  for (int e = 0; e < E; ++e)
    for (int p = 0; p < 16; ++p)
      for (int c = 0; c < 16; ++c) {
        const int pid = e == 0 ? anchor : cand[(e - 1) * 16 + p], cid = cand[e * 16 + c];
        double acc = 0;
        for (int r = 0; r < 256; ++r)
          acc += double(bf16r(P[size_t(pid) * 256 + r])) * double(hp[size_t(e) * 256 + r]) * double(bf16r(S[size_t(cid) * 256 + r]));
        scores[(size_t(e) * 16 + p) * 16 + c] = float(double(unary[e * 16 + c]) + acc);
      }
}
// hp[e][j] = x[e] . W[j] with W [256][H] rounded to BF16 (linear_bf16_drafter over the selector's projection,
// src/core/speculate.cpp:610), the sum in double.
void lo_selector_project(const float* x, const float* W, int E, int H, float* hp) {
  for (int e = 0; e < E; ++e)
    for (int j = 0; j < 256; ++j) {
      double acc = 0;
      for (int h = 0; h < H; ++h) acc += double(x[size_t(e) * H + h]) * double(bf16r(W[size_t(j) * H + h]));
      hp[size_t(e) * 256 + j] = float(acc);
    }
}

// ---------------------------------------------------------------------------------------------- model

lo_model* lo_create(const lo_model_config* cfg, const lo_options* opt) {
  init_dec();
  lo_model* m = new lo_model;
  m->cfg = *cfg;
  m->opt = *opt;
  m->layers.resize(cfg->layers);
  m->attn_index.assign(cfg->layers, -1);
  m->gdn_index.assign(cfg->layers, -1);
  for (int l = 0; l < cfg->layers; ++l) {
    m->layers[l].full = cfg->full_attention[l] != 0;
    if (m->layers[l].full) m->attn_index[l] = m->n_attn++;
    else m->gdn_index[l] = m->n_gdn++;
  }
  m->tables.assign(opt->sessions, std::vector<int>(m->max_pages(), 0));
  const size_t slots = size_t(m->n_attn) * 2 * cfg->kv_heads * (opt->pool_pages + 1) * opt->page_tokens;
  m->kv_codes.assign(slots * cfg->head_dim, 0);
  m->kv_scales.assign(slots, 0.f);
  m->gdn_state.assign(size_t(opt->sessions) * m->n_gdn,
                      std::vector<float>(size_t(cfg->lin_v_heads) * cfg->lin_k_dim * cfg->lin_v_dim, 0.f));
  m->conv_state.assign(size_t(opt->sessions) * m->n_gdn, std::vector<float>(size_t(m->C()) * 3, 0.f));
  return m;
}
void lo_destroy(lo_model* m) { delete m; }

static void set_vec(std::vector<float>& v, const float* h, size_t n) {
  v.resize(n);
  for (size_t i = 0; i < n; ++i) v[i] = bf16r(h[i]);
}

int lo_set_tensor(lo_model* m, int layer, int tensor, const float* host, int rows, int cols) {
  const lo_model_config& c = m->cfg;
  const size_t n = size_t(rows) * cols;
  if (tensor == T_EMBED) return set_vec(m->embed, host, n), 0;
  if (tensor == T_FINAL_NORM) return set_vec(m->final_norm, host, n), 0;
  if (tensor == T_LM_HEAD) return m->head.set(host, rows, cols), 0;
  if (layer < 0 || layer >= c.layers) return 1;
  Layer& L = m->layers[layer];
  switch (tensor) {
    case T_INPUT_NORM: set_vec(L.input_norm, host, n); break;
    case T_POST_NORM: set_vec(L.post_norm, host, n); break;
    case T_GATE: L.gate.set(host, rows, cols); break;
    case T_UP: L.up.set(host, rows, cols); break;
    case T_DOWN: L.down.set(host, rows, cols); break;
    case T_IN_QKV: L.in_qkv.set(host, rows, cols); break;
    case T_IN_Z: L.in_z.set(host, rows, cols); break;
    case T_OUT: L.out.set(host, rows, cols); break;
    case T_IN_A: set_vec(L.in_a, host, n); break;
    case T_IN_B: set_vec(L.in_b, host, n); break;
    case T_CONV: set_vec(L.conv, host, n); break;
    case T_A_LOG: set_vec(L.A_log, host, n); break;
    case T_DT_BIAS: set_vec(L.dt_bias, host, n); break;
    case T_LIN_NORM: set_vec(L.lin_norm, host, n); break;
    case T_Q: L.q.set(host, rows, cols); break;
    case T_K: L.k.set(host, rows, cols); break;
    case T_V: L.v.set(host, rows, cols); break;
    case T_O: L.o.set(host, rows, cols); break;
    case T_Q_NORM: set_vec(L.q_norm, host, n); break;
    case T_K_NORM: set_vec(L.k_norm, host, n); break;
    default: return 1;
  }
  return 0;
}

namespace {
struct SynthSpec {
  int tensor, rows, cols;
  float std_, bias;
};
std::vector<SynthSpec> layer_specs(const lo_model& m, bool full) {
  const lo_model_config& c = m.cfg;
  const int H = c.hidden, I = c.intermediate, D = c.head_dim;
  std::vector<SynthSpec> s = {{T_INPUT_NORM, 1, H, 0.02f, 0}, {T_POST_NORM, 1, H, 0.02f, 0},
                              {T_GATE, I, H, 0.02f, 0},       {T_UP, I, H, 0.02f, 0},
                              {T_DOWN, H, I, 0.02f, 0}};
  if (full) {
    s.push_back({T_Q, c.heads * 2 * D, H, 0.02f, 0});
    s.push_back({T_K, c.kv_heads * D, H, 0.02f, 0});
    s.push_back({T_V, c.kv_heads * D, H, 0.02f, 0});
    s.push_back({T_O, H, c.heads * D, 0.02f, 0});
    s.push_back({T_Q_NORM, 1, D, 0.02f, 0});
    s.push_back({T_K_NORM, 1, D, 0.02f, 0});
  } else {
    s.push_back({T_IN_QKV, m.C(), H, 0.02f, 0});
    s.push_back({T_IN_Z, m.Vs(), H, 0.02f, 0});
    s.push_back({T_OUT, H, m.Vs(), 0.02f, 0});
    s.push_back({T_IN_A, c.lin_v_heads, H, 0.02f, 0});
    s.push_back({T_IN_B, c.lin_v_heads, H, 0.02f, 0});
    s.push_back({T_CONV, m.C(), 4, 0.3f, 0});
    s.push_back({T_A_LOG, 1, c.lin_v_heads, 0.5f, 0});
    s.push_back({T_DT_BIAS, 1, c.lin_v_heads, 0.5f, 0});
    s.push_back({T_LIN_NORM, 1, c.lin_v_dim, 0.02f, 1.f});
  }
  return s;
}
void synth_one(lo_model* m, uint64_t seed, int layer, const SynthSpec& sp, int rows_limit = -1) {
  const int rows = rows_limit >= 0 ? std::min(rows_limit, sp.rows) : sp.rows;
  std::vector<float> buf(size_t(rows) * sp.cols);
  lo_synth(seed, lo_weight_stream(layer, sp.tensor), 0, buf.size(), sp.std_, sp.bias, 1, buf.data());
  lo_set_tensor(m, layer, sp.tensor, buf.data(), rows, sp.cols);
}
}  // namespace

int lo_synth_weights_layers(lo_model* m, uint64_t seed, const int* layers, int n_layers, int head_rows) {
  const lo_model_config& c = m->cfg;
  // The embedding is materialized only as far as head_rows asks (token ids of a sample stay below it).
  const int vrows = head_rows >= 0 ? std::min(head_rows, c.vocab) : c.vocab;
  synth_one(m, seed, -1, {T_EMBED, c.vocab, c.hidden, 0.02f, 0}, vrows);
  synth_one(m, seed, -1, {T_FINAL_NORM, 1, c.hidden, 0.02f, 0});
  synth_one(m, seed, -1, {T_LM_HEAD, c.vocab, c.hidden, 0.02f, 0}, vrows);
  for (int i = 0; i < n_layers; ++i) {
    const int l = layers[i];
    if (l < 0 || l >= c.layers) continue;
    for (const SynthSpec& sp : layer_specs(*m, m->layers[l].full)) synth_one(m, seed, l, sp);
  }
  return 0;
}
int lo_synth_weights(lo_model* m, uint64_t seed) {
  std::vector<int> all(m->cfg.layers);
  for (int l = 0; l < m->cfg.layers; ++l) all[l] = l;
  return lo_synth_weights_layers(m, seed, all.data(), m->cfg.layers, -1);
}

int lo_get_matrix(lo_model* m, int layer, int tensor, uint8_t* codes, float* scales, int rows, int cols) {
  const Mat* w = nullptr;
  if (tensor == T_LM_HEAD) w = &m->head;
  else {
    if (layer < 0 || layer >= m->cfg.layers) return 1;
    Layer& L = m->layers[layer];
    switch (tensor) {
      case T_GATE: w = &L.gate; break;
      case T_UP: w = &L.up; break;
      case T_DOWN: w = &L.down; break;
      case T_IN_QKV: w = &L.in_qkv; break;
      case T_IN_Z: w = &L.in_z; break;
      case T_OUT: w = &L.out; break;
      case T_Q: w = &L.q; break;
      case T_K: w = &L.k; break;
      case T_V: w = &L.v; break;
      case T_O: w = &L.o; break;
      default: return 1;
    }
  }
  if (w->N != rows || w->K != cols) return 1;
  if (codes) std::memcpy(codes, w->codes.data(), w->codes.size());
  if (scales) std::memcpy(scales, w->scales.data(), w->scales.size() * 4);
  return 0;
}

int lo_kv_table_set(lo_model* m, int slot, const int* idx, const int* page, int n) {
  if (slot < 0 || slot >= m->opt.sessions) return 1;
  for (int i = 0; i < n; ++i) {
    if (idx[i] < 0 || idx[i] >= m->max_pages() || page[i] < 0 || page[i] > m->opt.pool_pages) return 1;
    m->tables[slot][idx[i]] = page[i];
  }
  return 0;
}

namespace {
// One (position, head) vector into the cache: scale = amax/448, codes E4M3 (this build's KV format; the reference
// stores BF16, src/core/attention_body.cuh:67-70,97).
void kv_store(lo_model* m, int slot, int al, int kv, int h, int pos, const float* x) {
  const int D = m->cfg.head_dim, pt = m->opt.page_tokens;
  const int page = m->tables[slot][pos / pt];
  const size_t at = m->kv_index(al, kv, h, page, pos % pt);
  float amax = 0.f;
  for (int d = 0; d < D; ++d) amax = std::max(amax, std::fabs(x[d]));
  const float sc = amax > 0.f ? amax / 448.f : 1.f;
  m->kv_scales[at] = sc;
  for (int d = 0; d < D; ++d) m->kv_codes[at * D + d] = e4m3(x[d] / sc);
}
}  // namespace

int lo_kv_write(lo_model* m, int slot, int al, int from, int n, const float* k, const float* v) {
  const int Hkv = m->cfg.kv_heads, D = m->cfg.head_dim;
  for (int i = 0; i < n; ++i)
    for (int h = 0; h < Hkv; ++h) {
      kv_store(m, slot, al, 0, h, from + i, k + (size_t(i) * Hkv + h) * D);
      kv_store(m, slot, al, 1, h, from + i, v + (size_t(i) * Hkv + h) * D);
    }
  return 0;
}

int lo_kv_read(lo_model* m, int slot, int al, int from, int n, float* k, float* v, uint8_t* kc, float* ks,
               uint8_t* vc, float* vs) {
  const int Hkv = m->cfg.kv_heads, D = m->cfg.head_dim, pt = m->opt.page_tokens;
  for (int i = 0; i < n; ++i)
    for (int h = 0; h < Hkv; ++h)
      for (int kv = 0; kv < 2; ++kv) {
        const int pos = from + i;
        const size_t at = m->kv_index(al, kv, h, m->tables[slot][pos / pt], pos % pt);
        const size_t o = size_t(i) * Hkv + h;
        float* f = kv ? v : k;
        uint8_t* c = kv ? vc : kc;
        float* s = kv ? vs : ks;
        if (s) s[o] = m->kv_scales[at];
        for (int d = 0; d < D; ++d) {
          if (c) c[o * D + d] = m->kv_codes[at * D + d];
          if (f) f[o * D + d] = g_dec[m->kv_codes[at * D + d]] * m->kv_scales[at];
        }
      }
  return 0;
}

int lo_synth_kv(lo_model* m, int slot, int n, uint64_t seed) {
  const int Hkv = m->cfg.kv_heads, D = m->cfg.head_dim;
  for (int al = 0; al < m->n_attn; ++al)
    for (int kv = 0; kv < 2; ++kv) {
      const uint64_t key = stream_key(seed, kStreamKv + (uint64_t(slot) * m->n_attn + al) * 2 + kv);
      parallel_for(n, [&](int p_lo, int p_hi) {
        std::vector<float> x(D);
        for (int p = p_lo; p < p_hi; ++p)
          for (int h = 0; h < Hkv; ++h) {
            for (int d = 0; d < D; ++d) x[d] = synth_z(key, (size_t(p) * Hkv + h) * D + d);
            kv_store(m, slot, al, kv, h, p, x.data());
          }
      });
    }
  return 0;
}

int lo_state_write(lo_model* m, int slot, int gl, const float* state, const float* conv) {
  if (slot < 0 || slot >= m->opt.sessions || gl < 0 || gl >= m->n_gdn) return 1;
  auto& S = m->gdn_state[size_t(slot) * m->n_gdn + gl];
  auto& W = m->conv_state[size_t(slot) * m->n_gdn + gl];
  if (state) std::copy(state, state + S.size(), S.begin());
  if (conv) std::copy(conv, conv + W.size(), W.begin());
  return 0;
}
int lo_state_read(lo_model* m, int slot, int gl, float* state, float* conv) {
  if (slot < 0 || slot >= m->opt.sessions || gl < 0 || gl >= m->n_gdn) return 1;
  const auto& S = m->gdn_state[size_t(slot) * m->n_gdn + gl];
  const auto& W = m->conv_state[size_t(slot) * m->n_gdn + gl];
  if (state) std::copy(S.begin(), S.end(), state);
  if (conv) std::copy(W.begin(), W.end(), conv);
  return 0;
}
int lo_synth_state(lo_model* m, int slot, uint64_t seed) {
  for (int gl = 0; gl < m->n_gdn; ++gl) {
    auto& S = m->gdn_state[size_t(slot) * m->n_gdn + gl];
    auto& W = m->conv_state[size_t(slot) * m->n_gdn + gl];
    lo_synth(seed, kStreamState + uint64_t(slot) * m->n_gdn + gl, 0, S.size(), 0.1f, 0.f, 0, S.data());
    lo_synth(seed, kStreamConv + uint64_t(slot) * m->n_gdn + gl, 0, W.size(), 1.f, 0.f, 0, W.data());
  }
  return 0;
}
// Engine::state_hash (src/core/engine.cpp:954-971): FNV-1a, byte by byte, every DeltaNet layer's state then window.
int lo_state_hash(lo_model* m, int slot, uint64_t* hash) {
  uint64_t h = 1469598103934665603ull;
  auto eat = [&](const std::vector<float>& v) {
    const unsigned char* b = reinterpret_cast<const unsigned char*>(v.data());
    for (size_t i = 0; i < v.size() * 4; ++i) h = (h ^ b[i]) * 1099511628211ull;
  };
  for (int gl = 0; gl < m->n_gdn; ++gl) {
    eat(m->gdn_state[size_t(slot) * m->n_gdn + gl]);
    eat(m->conv_state[size_t(slot) * m->n_gdn + gl]);
  }
  *hash = h;
  return 0;
}

// ---------------------------------------------------------------------------------------------- the step

namespace {

struct StepScope {
  const int* layers = nullptr;  // nullptr: every layer
  int n_layers = 0;
  int head_rows = -1;           // -1: the whole vocabulary
  bool run(int l) const {
    if (!layers) return true;
    for (int i = 0; i < n_layers; ++i)
      if (layers[i] == l) return true;
    return false;
  }
};

// attn_prepare for one row of one head (src/core/attention_body.cuh:54-99): RMSNorm with (1 + w), rotation of the
// first `rot` dims as two halves, inv_freq = theta^(-2i/rot), angle = position * inv_freq.
void norm_rope(const float* x, const float* w, float* out, int D, int rot, float theta, float eps, int position) {
  double ss = 0;
  for (int d = 0; d < D; ++d) ss += double(x[d]) * x[d];
  const float rstd = float(1.0 / std::sqrt(ss / D + double(eps)));
  std::vector<float> xn(D);
  for (int d = 0; d < D; ++d) xn[d] = x[d] * rstd * (1.f + w[d]);
  const int half = rot / 2;
  for (int d = 0; d < D; ++d) {
    if (d >= rot) {
      out[d] = xn[d];
      continue;
    }
    const int i = d % half;
    const float inv_freq = std::pow(theta, -2.f * i / rot);
    const float ang = float(position) * inv_freq;
    const float sn = std::sin(ang), cs = std::cos(ang);
    out[d] = d < half ? xn[d] * cs - xn[d + half] * sn : xn[d] * cs + xn[d - half] * sn;
  }
}

// Packing (src/core/speculate.cpp:1190-1201, src/core/kernels.cuh:58-78): rows concatenated sequence by sequence; a
// row's RoPE position is pos + depth (+ rope delta), its cache slot pos + row index (src/core/kernels.cuh:109-118).
int pack_step(lo_model* m, const lo_seq_step* seqs, int n_seqs) {
  if (n_seqs < 1 || n_seqs > m->opt.max_seqs) return 1;
  m->n_seqs = n_seqs;
  m->row0.assign(n_seqs + 1, 0);
  m->trees.assign(n_seqs, lo_tree_desc{});
  for (int s = 0; s < n_seqs; ++s) {
    if (seqs[s].n_rows < 1 || seqs[s].n_rows > LO_MAX_TREE_ROWS) return 1;
    if (lo_describe_tree(seqs[s].parent, seqs[s].n_rows, seqs[s].chain, &m->trees[s])) return 1;
    m->row0[s + 1] = m->row0[s] + seqs[s].n_rows;
  }
  const int M = m->rows = m->row0[n_seqs];
  if (M > m->opt.max_rows) return 1;
  m->token.resize(M), m->seq_of.resize(M), m->depth.resize(M), m->rope_pos.resize(M), m->cache_slot.resize(M);
  m->anc.assign(M, 0);
  for (int s = 0; s < n_seqs; ++s)
    for (int r = 0; r < seqs[s].n_rows; ++r) {
      const int row = m->row0[s] + r;
      m->token[row] = seqs[s].tokens[r];
      m->seq_of[row] = s;
      m->depth[row] = m->trees[s].depth[r];
      m->rope_pos[row] = seqs[s].pos + m->trees[s].depth[r] + seqs[s].rope_delta;
      m->cache_slot[row] = seqs[s].pos + r;
      for (int a = r; a >= 0; a = (a == 0 ? -1 : seqs[s].parent[a])) m->anc[row] |= 1u << a;
    }
  return 0;
}

// Row r sees the context [0, pos) and the rows of its own root-to-row path (src/core/attention_body.cuh:175-195,289-294);
// scores q.k / sqrt(D), softmax and the value sum in double; K and V as the cache holds them (E4M3 codes x the
// position's scale).  out [M][Hq][D], before the output gate.  Per (sequence, kv head) the codes of every position the
// sequence can see are decoded once and shared by its rows and the q heads of the group (the arithmetic per row is the
// same as decoding them on the fly).
void attend(lo_model* m, const lo_seq_step* seqs, int al, const float* q, float* out) {
  const lo_model_config& c = m->cfg;
  const int Hq = c.heads, Hkv = c.kv_heads, D = c.head_dim, G = Hq / Hkv, pt = m->opt.page_tokens;
  const float inv_sqrt_d = 1.f / std::sqrt(float(D));
  for (int s = 0; s < m->n_seqs; ++s) {
    const int slot = seqs[s].slot, pos0 = seqs[s].pos, n = seqs[s].n_rows, nk = pos0 + n, r0 = m->row0[s];
    std::vector<float> kd(size_t(nk) * D), vd(size_t(nk) * D), ksc(nk), vsc(nk);
    for (int hk = 0; hk < Hkv; ++hk) {
      parallel_for(nk, [&](int lo, int hi) {
        for (int p = lo; p < hi; ++p) {
          const size_t ak = m->kv_index(al, 0, hk, m->tables[slot][p / pt], p % pt);
          const size_t av = m->kv_index(al, 1, hk, m->tables[slot][p / pt], p % pt);
          ksc[p] = m->kv_scales[ak], vsc[p] = m->kv_scales[av];
          for (int d = 0; d < D; ++d) kd[size_t(p) * D + d] = g_dec[m->kv_codes[ak * D + d]];
          for (int d = 0; d < D; ++d) vd[size_t(p) * D + d] = g_dec[m->kv_codes[av * D + d]];
        }
      });
      parallel_for(n * G, [&](int lo, int hi) {
        std::vector<float> sc(nk);
        std::vector<double> acc(D);
        for (int u = lo; u < hi; ++u) {
          const int r = r0 + u / G, hq = hk * G + u % G;
          const float* qv = &q[(size_t(r) * Hq + hq) * D];
          auto visible = [&](int p) { return p < pos0 || ((m->anc[r] >> (p - pos0)) & 1u); };
          float mx = -INFINITY;
          for (int p = 0; p < nk; ++p) {
            if (!visible(p)) continue;
            const float* kr = &kd[size_t(p) * D];
            double dot = 0;
            for (int d = 0; d < D; ++d) dot += double(qv[d]) * kr[d];
            sc[p] = float(dot) * ksc[p] * inv_sqrt_d;
            mx = std::max(mx, sc[p]);
          }
          double den = 0;
          std::fill(acc.begin(), acc.end(), 0.0);
          for (int p = 0; p < nk; ++p) {
            if (!visible(p)) continue;
            const double pr = std::exp(double(sc[p] - mx));
            den += pr;
            const double pv = pr * vsc[p];
            const float* vr = &vd[size_t(p) * D];
            for (int d = 0; d < D; ++d) acc[d] += pv * vr[d];
          }
          for (int d = 0; d < D; ++d) out[(size_t(r) * Hq + hq) * D + d] = float(acc[d] / den);
        }
      });
    }
  }
}

// What a DeltaNet layer keeps for the commit (src/core/engine.hpp:846-848): raw and convolved inputs, gates.
struct Saved {
  std::vector<std::vector<float>> pre, post, g, beta;
  explicit Saved(int n_gdn) : pre(n_gdn), post(n_gdn), g(n_gdn), beta(n_gdn) {}
};

// One layer of the forward pass over the packed rows (src/core/engine.cpp:1361-1725): h [M][H] is the residual stream
// before the layer on entry and after it on return.  pack_step() has run.
void layer_forward(lo_model* m, const lo_seq_step* seqs, int n_seqs, int l, std::vector<float>& h, Saved& saved, bool ffn = true) {
  const lo_model_config& c = m->cfg;
  const int H = c.hidden, I = c.intermediate, Hq = c.heads, Hkv = c.kv_heads, D = c.head_dim;
  const int Hk = c.lin_k_heads, HV = c.lin_v_heads, Dk = c.lin_k_dim, Dv = c.lin_v_dim, C = m->C(), Vs = m->Vs();
  const int M = m->rows;
  std::vector<float> xn(size_t(M) * H);
  {
    const Layer& L = m->layers[l];
    for (int r = 0; r < M; ++r) rmsnorm(&h[size_t(r) * H], L.input_norm.data(), &xn[size_t(r) * H], H, c.eps, true);
    QAct xq;
    xq.set(xn.data(), M, H);
    if (L.full) {
      // B.3 gated GQA attention (src/core/engine.cpp:1424-1469)
      const int al = m->attn_index[l];
      std::vector<float> qg(size_t(M) * Hq * 2 * D), kk(size_t(M) * Hkv * D), vv(size_t(M) * Hkv * D);
      gemm(xq, L.q, qg.data(), size_t(Hq) * 2 * D, 0);
      gemm(xq, L.k, kk.data(), size_t(Hkv) * D, 0);
      gemm(xq, L.v, vv.data(), size_t(Hkv) * D, 0);
      std::vector<float> q(size_t(M) * Hq * D), kr(D);
      for (int r = 0; r < M; ++r) {
        const int s = m->seq_of[r];
        for (int hq = 0; hq < Hq; ++hq)
          norm_rope(&qg[(size_t(r) * Hq + hq) * 2 * D], L.q_norm.data(), &q[(size_t(r) * Hq + hq) * D], D,
                    c.rotary_dim, c.rope_theta, c.eps, m->rope_pos[r]);
        for (int hk = 0; hk < Hkv; ++hk) {
          norm_rope(&kk[(size_t(r) * Hkv + hk) * D], L.k_norm.data(), kr.data(), D, c.rotary_dim, c.rope_theta, c.eps,
                    m->rope_pos[r]);
          kv_store(m, seqs[s].slot, al, 0, hk, m->cache_slot[r], kr.data());
          kv_store(m, seqs[s].slot, al, 1, hk, m->cache_slot[r], &vv[(size_t(r) * Hkv + hk) * D]);
        }
      }
      std::vector<float> att(size_t(M) * Hq * D);
      attend(m, seqs, al, q.data(), att.data());
      // out * sigmoid(gate) (src/core/kernels.cu:314-318); the gate is the head's second D values
      for (int r = 0; r < M; ++r)
        for (int hq = 0; hq < Hq; ++hq)
          for (int d = 0; d < D; ++d)
            att[(size_t(r) * Hq + hq) * D + d] *= sigmoid(qg[(size_t(r) * Hq + hq) * 2 * D + D + d]);
      QAct aq;
      aq.set(att.data(), M, Hq * D);
      std::vector<float> o(size_t(M) * H);
      gemm(aq, L.o, o.data(), H, 0);
      for (size_t i = 0; i < h.size(); ++i) h[i] += o[i];
    } else {
      // B.4 gated DeltaNet (src/core/engine.cpp:1612-1677)
      const int gl = m->gdn_index[l];
      std::vector<float> pre(size_t(M) * C), z(size_t(M) * Vs), post(size_t(M) * C), core(size_t(M) * Vs);
      gemm(xq, L.in_qkv, pre.data(), C, 0);
      gemm(xq, L.in_z, z.data(), Vs, 0);
      // a, b: fp32 rows against BF16 weights (src/core/kernels.cu:200-253), then the gating
      // (src/core/kernels.cu:385-395): g = -exp(A_log) * softplus(a + dt_bias), beta = sigmoid(b).
      std::vector<float> g(size_t(M) * HV), beta(size_t(M) * HV);
      for (int r = 0; r < M; ++r)
        for (int hv = 0; hv < HV; ++hv) {
          double a = 0, b = 0;
          for (int i = 0; i < H; ++i) {
            a += double(xn[size_t(r) * H + i]) * L.in_a[size_t(hv) * H + i];
            b += double(xn[size_t(r) * H + i]) * L.in_b[size_t(hv) * H + i];
          }
          const float x = float(a) + L.dt_bias[hv];
          const float sp = x <= 20.f ? std::log1p(std::exp(x)) : x;
          g[size_t(r) * HV + hv] = -std::exp(L.A_log[hv]) * sp;
          beta[size_t(r) * HV + hv] = sigmoid(float(b));
        }
      for (int s = 0; s < n_seqs; ++s) {
        const size_t r0 = m->row0[s];
        const size_t st = size_t(seqs[s].slot) * m->n_gdn + gl;
        lo_gdn_tree(Hk, HV, Dk, Dv, &m->trees[s], &pre[r0 * C], L.conv.data(), &g[r0 * HV], &beta[r0 * HV],
                    m->gdn_state[st].data(), m->conv_state[st].data(), &post[r0 * C], &core[r0 * Vs]);
      }
      // gated RMSNorm over Dv with the plain weight, times silu(z) (src/core/kernels.cu:543-554)
      std::vector<float> normed(size_t(M) * Vs);
      for (int r = 0; r < M; ++r)
        for (int hv = 0; hv < HV; ++hv) {
          const size_t at = size_t(r) * Vs + size_t(hv) * Dv;
          rmsnorm(&core[at], L.lin_norm.data(), &normed[at], Dv, c.eps, false);
          for (int d = 0; d < Dv; ++d) normed[at + d] *= silu(z[at + d]);
        }
      QAct nq;
      nq.set(normed.data(), M, Vs);
      std::vector<float> o(size_t(M) * H);
      gemm(nq, L.out, o.data(), H, 0);
      for (size_t i = 0; i < h.size(); ++i) h[i] += o[i];
      saved.pre[gl] = std::move(pre), saved.post[gl] = std::move(post), saved.g[gl] = std::move(g), saved.beta[gl] = std::move(beta);
    }
    if (!ffn) return;  // the mixer alone
    // B.5 SwiGLU FFN (src/core/engine.cpp:1698-1703, src/core/kernels.cu:308-312)
    for (int r = 0; r < M; ++r) rmsnorm(&h[size_t(r) * H], L.post_norm.data(), &xn[size_t(r) * H], H, c.eps, true);
    QAct fq;
    fq.set(xn.data(), M, H);
    std::vector<float> gu(size_t(M) * 2 * I), t(size_t(M) * I), dn(size_t(M) * H);
    gemm(fq, L.gate, gu.data(), size_t(2) * I, 0);
    gemm(fq, L.up, gu.data(), size_t(2) * I, I);
    for (int r = 0; r < M; ++r)
      for (int i = 0; i < I; ++i) t[size_t(r) * I + i] = silu(gu[size_t(r) * 2 * I + i]) * gu[size_t(r) * 2 * I + I + i];
    QAct tq;
    tq.set(t.data(), M, I);
    gemm(tq, L.down, dn.data(), H, 0);
    for (size_t i = 0; i < h.size(); ++i) h[i] += dn[i];
  }
}

// B.6 final norm and head over every row, argmax (src/core/engine.cpp:1726-1733, src/core/topk.cu): xn = the normed
// rows, logits and argmax kept in the model for the read-backs.
void head_forward(lo_model* m, const std::vector<float>& h, std::vector<float>& xn, int head_rows) {
  const lo_model_config& c = m->cfg;
  const int H = c.hidden, M = m->rows;
  xn.resize(size_t(M) * H);
  for (int r = 0; r < M; ++r) rmsnorm(&h[size_t(r) * H], m->final_norm.data(), &xn[size_t(r) * H], H, c.eps, true);
  QAct hq8;
  hq8.set(xn.data(), M, H);
  const int Vn = head_rows >= 0 ? std::min(head_rows, c.vocab) : c.vocab;
  m->logits.assign(size_t(M) * Vn, 0.f);
  gemm(hq8, m->head, m->logits.data(), Vn, 0, Vn);
  m->argmax_id.resize(M), m->argmax_val.resize(M);
  lo_argmax(m->logits.data(), M, Vn, m->argmax_id.data(), m->argmax_val.data());
}

int step_impl(lo_model* m, const lo_seq_step* seqs, int n_seqs, int flags, lo_seq_result* results,
              const StepScope& scope) {
  const lo_model_config& c = m->cfg;
  const int H = c.hidden, Hkv = c.kv_heads, D = c.head_dim;
  const int Hk = c.lin_k_heads, HV = c.lin_v_heads, Dk = c.lin_k_dim, Dv = c.lin_v_dim, C = m->C();
  const int pt = m->opt.page_tokens;
  if (const int rc = pack_step(m, seqs, n_seqs)) return rc;
  const int M = m->rows;

  // B.1 embedding (src/core/kernels.cu:280-286)
  std::vector<float> h(size_t(M) * H), xn;
  for (int r = 0; r < M; ++r)
    for (int i = 0; i < H; ++i) h[size_t(r) * H + i] = m->embed[size_t(m->token[r]) * H + i];

  const bool taps = flags & 4;
  if (taps) m->taps.assign(c.layers + 1, {});
  Saved saved(m->n_gdn);
  std::vector<std::vector<float>>&s_pre = saved.pre, &s_post = saved.post, &s_g = saved.g, &s_beta = saved.beta;

  for (int l = 0; l < c.layers; ++l) {
    if (!scope.run(l)) continue;
    layer_forward(m, seqs, n_seqs, l, h, saved);
    if (taps) m->taps[l] = h;
  }

  head_forward(m, h, xn, scope.head_rows);
  if (taps) m->taps[c.layers] = xn;
  if (!results) return 0;

  // B.7 accept, compaction, commit
  for (int s = 0; s < n_seqs; ++s) {
    lo_seq_result& R = results[s];
    std::memset(&R, 0, sizeof R);
    const int r0 = m->row0[s], n = seqs[s].n_rows;
    // require_finite_topk (src/core/sampling.cpp:20-23) over the sequence's rows
    for (int r = 0; r < n; ++r) {
      const float v = m->argmax_val[r0 + r];
      const int id = m->argmax_id[r0 + r];
      if (!std::isfinite(v) || v == -FLT_MAX || id < 0 || id >= c.vocab) R.status = 1;
    }
    std::vector<int> am(n);
    for (int r = 0; r < n; ++r) am[r] = (seqs[s].force_argmax && seqs[s].force_argmax[r] >= 0) ? seqs[s].force_argmax[r] : m->argmax_id[r0 + r];
    if (R.status) continue;  // nothing committed (src/core/speculate.cpp:1214-1219)
    R.n_path = lo_accept_tree_greedy(seqs[s].parent, seqs[s].tokens, n, am.data(), R.path, &R.next_token);
    // SeqStep::out: the accepted drafts, then the next token (src/core/speculate.cpp:1066-1067)
    for (int j = 1; j < R.n_path; ++j) R.out[R.n_out++] = seqs[s].tokens[R.path[j]];
    R.out[R.n_out++] = R.next_token;
    if (!(flags & 1)) continue;
    // tree_gather (src/core/kernels.cu:481-498): cache slot pos + path[j] -> pos + j, j ascending
    for (int al = 0; al < m->n_attn; ++al)
      for (int kv = 0; kv < 2; ++kv)
        for (int hk = 0; hk < Hkv; ++hk)
          for (int j = 1; j < R.n_path; ++j) {
            if (R.path[j] == j) continue;
            const int ps = seqs[s].pos + R.path[j], pd = seqs[s].pos + j;
            const size_t a = m->kv_index(al, kv, hk, m->tables[seqs[s].slot][ps / pt], ps % pt);
            const size_t b = m->kv_index(al, kv, hk, m->tables[seqs[s].slot][pd / pt], pd % pt);
            m->kv_scales[b] = m->kv_scales[a];
            std::memcpy(&m->kv_codes[b * D], &m->kv_codes[a * D], D);
          }
    for (int gl = 0; gl < m->n_gdn; ++gl) {
      if (s_pre[gl].empty()) continue;
      const size_t st = size_t(seqs[s].slot) * m->n_gdn + gl;
      lo_gdn_commit(Hk, HV, Dk, Dv, R.path, R.n_path, n, &s_pre[gl][size_t(r0) * C], &s_post[gl][size_t(r0) * C],
                    &s_g[gl][size_t(r0) * HV], &s_beta[gl][size_t(r0) * HV], m->gdn_state[st].data(),
                    m->conv_state[st].data());
    }
  }
  return 0;
}
}  // namespace

int lo_verify_step(lo_model* m, const lo_seq_step* seqs, int n_seqs, int flags, lo_seq_result* results) {
  return step_impl(m, seqs, n_seqs, flags, results, StepScope{});
}
int lo_verify_step_sample(lo_model* m, const lo_seq_step* seqs, int n_seqs, const int* layers, int n_layers,
                          int head_rows) {
  StepScope sc;
  sc.layers = layers, sc.n_layers = n_layers, sc.head_rows = head_rows;
  return step_impl(m, seqs, n_seqs, 0, nullptr, sc);
}

// The attention of one layer alone: packing of `seqs`, then every row over its context and its path's in-flight rows as
// the cache holds them; q and out are [rows][heads][head_dim], out before the output gate.
int lo_attention(lo_model* m, const lo_seq_step* seqs, int n_seqs, int attn_layer, const float* q, float* out) {
  if (attn_layer < 0 || attn_layer >= m->n_attn) return 1;
  if (const int rc = pack_step(m, seqs, n_seqs)) return rc;
  attend(m, seqs, attn_layer, q, out);
  return 0;
}

// One layer alone on a given residual stream (teacher forcing): h_in [rows][hidden] is what stands before layer `layer`,
// h_out what stands after it; the layer's weights, the sessions' KV and DeltaNet state must be in place.  layer ==
// cfg.layers: the final norm and the head instead (h_out = the normed rows; logits and argmax for the read-backs;
// head_rows < 0: the whole vocabulary).
int lo_layer_forward(lo_model* m, const lo_seq_step* seqs, int n_seqs, int layer, const float* h_in, float* h_out,
                     int head_rows) {
  if (layer < 0 || layer > m->cfg.layers) return 1;
  if (const int rc = pack_step(m, seqs, n_seqs)) return rc;
  const size_t n = size_t(m->rows) * m->cfg.hidden;
  std::vector<float> h(h_in, h_in + n), xn;
  if (layer == m->cfg.layers) {
    head_forward(m, h, xn, head_rows);
    std::copy(xn.begin(), xn.end(), h_out);
    return 0;
  }
  Saved saved(m->n_gdn);
  layer_forward(m, seqs, n_seqs, layer, h, saved);
  std::copy(h.begin(), h.end(), h_out);
  return 0;
}
// The layer's mixer alone (attention or DeltaNet with its projections and the residual add), without the feed-forward block.
int lo_mixer_forward(lo_model* m, const lo_seq_step* seqs, int n_seqs, int layer, const float* h_in, float* h_out) {
  if (layer < 0 || layer >= m->cfg.layers) return 1;
  if (const int rc = pack_step(m, seqs, n_seqs)) return rc;
  const size_t n = size_t(m->rows) * m->cfg.hidden;
  std::vector<float> h(h_in, h_in + n);
  Saved saved(m->n_gdn);
  layer_forward(m, seqs, n_seqs, layer, h, saved, false);
  std::copy(h.begin(), h.end(), h_out);
  return 0;
}

// attn_prepare alone (src/core/kernels.cu:558-596, src/core/attention_body.cuh:54-99) for one full-attention layer:
// qkv [rows][Hq*2*D + 2*Hkv*D] is the q|k|v projection's output (per q head: D query values then D gate values);
// q_out [rows][Hq][D] the normed, rotated queries; k_out [rows][Hkv][D] (may be NULL) the normed, rotated keys BEFORE
// the cache rounding; K (rotated) and V (raw) go to cache slot pos + row index as the step stores them.
int lo_attn_prepare(lo_model* m, const lo_seq_step* seqs, int n_seqs, int attn_layer, const float* qkv, float* q_out,
                    float* k_out) {
  if (attn_layer < 0 || attn_layer >= m->n_attn) return 1;
  if (const int rc = pack_step(m, seqs, n_seqs)) return rc;
  const lo_model_config& c = m->cfg;
  const int Hq = c.heads, Hkv = c.kv_heads, D = c.head_dim, W = Hq * 2 * D + 2 * Hkv * D;
  int layer = -1;
  for (int l = 0; l < c.layers; ++l)
    if (m->attn_index[l] == attn_layer) layer = l;
  const Layer& L = m->layers[layer];
  if (int(L.q_norm.size()) != D || int(L.k_norm.size()) != D) return 1;
  std::vector<float> kr(D);
  for (int r = 0; r < m->rows; ++r) {
    const int s = m->seq_of[r];
    const float* row = qkv + size_t(r) * W;
    for (int hq = 0; hq < Hq; ++hq)
      norm_rope(row + size_t(hq) * 2 * D, L.q_norm.data(), &q_out[(size_t(r) * Hq + hq) * D], D, c.rotary_dim, c.rope_theta,
                c.eps, m->rope_pos[r]);
    for (int hk = 0; hk < Hkv; ++hk) {
      norm_rope(row + size_t(Hq) * 2 * D + size_t(hk) * D, L.k_norm.data(), kr.data(), D, c.rotary_dim, c.rope_theta, c.eps,
                m->rope_pos[r]);
      if (k_out) std::copy(kr.begin(), kr.end(), &k_out[(size_t(r) * Hkv + hk) * D]);
      kv_store(m, seqs[s].slot, attn_layer, 0, hk, m->cache_slot[r], kr.data());
      kv_store(m, seqs[s].slot, attn_layer, 1, hk, m->cache_slot[r], row + size_t(Hq) * 2 * D + size_t(Hkv) * D + size_t(hk) * D);
    }
  }
  return 0;
}

int lo_read_tree_desc(lo_model* m, int seq, lo_tree_desc* out) {
  if (seq < 0 || seq >= m->n_seqs) return 1;
  *out = m->trees[seq];
  return 0;
}
int lo_read_packing(lo_model* m, int* row0, int* token, int* seq_of, int* depth, int* rope_pos, int* cache_slot,
                    uint32_t* anc) {
  auto cp = [](auto* dst, const auto& src) {
    if (dst) std::copy(src.begin(), src.end(), dst);
  };
  cp(row0, m->row0), cp(token, m->token), cp(seq_of, m->seq_of), cp(depth, m->depth), cp(rope_pos, m->rope_pos);
  cp(cache_slot, m->cache_slot), cp(anc, m->anc);
  return 0;
}
int lo_read_argmax(lo_model* m, int* ids, float* vals) {
  if (ids) std::copy(m->argmax_id.begin(), m->argmax_id.end(), ids);
  if (vals) std::copy(m->argmax_val.begin(), m->argmax_val.end(), vals);
  return 0;
}
int lo_read_logits(lo_model* m, float* out) {
  std::copy(m->logits.begin(), m->logits.end(), out);
  return 0;
}
int lo_read_tap(lo_model* m, int layer, float* out) {
  if (layer < 0 || layer >= int(m->taps.size()) || m->taps[layer].empty()) return 1;
  std::copy(m->taps[layer].begin(), m->taps[layer].end(), out);
  return 0;
}

// ---------------------------------------------------------------------------------------------- NVFP4 (prefill chunk)
// E2M1 values, two a byte with the first in the low nibble, one E4M3 scale per 16 values, one fp32 scale per tensor.
static const float kE2M1[16] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f, -0.f, -0.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};

// E2M1 to nearest with ties to the even code and saturation at 6 (cvt.rn.satfinite.e2m1x2.f32); a negative value that
// rounds to zero keeps its sign bit (tests/prefill_tests.cu:44-55 of the reference project writes out the same rule).
static uint8_t e2m1_rne(float x) {
  static const float mid[7] = {0.25f, 0.75f, 1.25f, 1.75f, 2.5f, 3.5f, 5.f};  // mid[i] lies between codes i and i + 1
  if (std::isnan(x)) return 7;  // satfinite turns NaN into the largest positive magnitude
  const float a = std::fabs(x);
  int c = 0;
  for (int i = 0; i < 7; ++i)
    if (a > mid[i] || (a == mid[i] && (i & 1))) c = i + 1;  // on a midpoint: the even code of the two
  return uint8_t(c | (std::signbit(x) ? 8 : 0));
}

// Weights to NVFP4 in the checkpoints' rounding (src/core/model.cu:188-249): g = amax / (448 * 6) (1 for an all-zero
// matrix); per block of 16 the E4M3 scale of max(amax16 / 6 / g, 2^-9); each value's code is the first of the codes'
// midpoints {0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5} that is not below |x / (scale * g)|, so a value on a midpoint takes
// the smaller magnitude; zero magnitudes carry no sign.  w: BF16 bit patterns [N][K]; q [N][K/2]; sf [N][K/16].
int lo_nvfp4_quantize_weight(const uint16_t* w, int N, int K, uint8_t* q, uint8_t* sf, float* scale2) {
  if (N <= 0 || K <= 0 || K % 16) return 1;
  init_dec();
  auto val = [&](size_t i) {
    const uint32_t u = uint32_t(w[i]) << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
  };
  float mx = 0.f;
  for (size_t i = 0; i < size_t(N) * K; ++i) mx = std::max(mx, std::fabs(val(i)));
  const float g = mx > 0.f ? mx / (448.f * 6.f) : 1.f;
  *scale2 = g;
  static const float mid[7] = {0.25f, 0.75f, 1.25f, 1.75f, 2.5f, 3.5f, 5.f};
  parallel_for(N, [&](int lo, int hi) {
    for (int r = lo; r < hi; ++r)
      for (int b = 0; b < K / 16; ++b) {
        const size_t base = size_t(r) * K + size_t(b) * 16;
        float bm = 0.f;
        for (int j = 0; j < 16; ++j) bm = std::max(bm, std::fabs(val(base + j)));
        const uint8_t sc = e4m3(std::max(bm / 6.f / g, 0x1p-9f));
        sf[size_t(r) * (K / 16) + b] = sc;
        const float s = g_dec[sc] * g;
        for (int j = 0; j < 16; j += 2) {
          uint8_t byte = 0;
          for (int h = 0; h < 2; ++h) {
            const float x = val(base + j + h), a = std::fabs(x / s);
            int c = 0;
            while (c < 7 && mid[c] < a) ++c;
            if (x < 0.f && c > 0) c |= 8;
            byte |= uint8_t(c << (4 * h));
          }
          q[(base + j) / 2] = byte;
        }
      }
  });
  return 0;
}

// Activations to NVFP4 under the global scale 1 / input_scale (src/core/prefill_gemm.cu:383-394,408-420; the host recipe
// the reference's own test checks it against byte for byte: tests/prefill_tests.cu:72-85): values rounded to BF16, block
// scale E4M3(gs * (amax * (1/6))), codes E2M1(v * os) with os = 1 / (scale * (1 / gs)) (0 for a zero scale).  With `up`
// the value quantized is silu(x) * up.  q [M][K/2], sf [M][K/16].
int lo_nvfp4_quant_act(const float* x, const float* up, int M, int K, float input_scale, uint8_t* q, uint8_t* sf) {
  if (M <= 0 || K <= 0 || K % 16) return 1;
  init_dec();
  const float gs = 1.f / input_scale;
  parallel_for(M, [&](int lo, int hi) {
    for (size_t b = size_t(lo) * (K / 16); b < size_t(hi) * (K / 16); ++b) {
      float v[16], amax = 0.f;
      for (int j = 0; j < 16; ++j) {
        float f = x[b * 16 + j];
        if (up) f = (f / (1.f + std::exp(-f))) * up[b * 16 + j];
        v[j] = bf16r(f);
        amax = std::max(amax, std::fabs(v[j]));
      }
      const uint8_t sc = e4m3(gs * (amax * (1.f / 6.f)));
      sf[b] = sc;
      const float sv = g_dec[sc], os = sv != 0.f ? 1.f / (sv * (1.f / gs)) : 0.f;
      for (int j = 0; j < 16; j += 2) q[b * 8 + j / 2] = uint8_t(e2m1_rne(v[j] * os) | (e2m1_rne(v[j + 1] * os) << 4));
    }
  });
  return 0;
}

// NVFP4 codes and block scales back to fp32 (without the tensor scale).
int lo_nvfp4_dequant(const uint8_t* q, const uint8_t* sf, int rows, int K, float* out) {
  init_dec();
  for (size_t i = 0; i < size_t(rows) * K; ++i) out[i] = kE2M1[(q[i / 2] >> (4 * (i & 1))) & 15] * g_dec[sf[i / 16]];
  return 0;
}

// y[m][n] = alpha * sum_k x[m][k] * w[n][k] (+ y with accumulate) over the dequantized operands, the sum in double: the
// check the reference's own test applies to prefill_gemm_nvfp4 (tests/prefill_tests.cu:176-205; the kernel:
// src/core/prefill_gemm.cu:344-380,685-690).
int lo_nvfp4_gemm(const uint8_t* xq, const uint8_t* xs, int M, const uint8_t* wq, const uint8_t* ws, int N, int K, float alpha,
                  float* y, int ldy, int accumulate) {
  if (K % 16) return 1;
  std::vector<float> xa(size_t(M) * K), wa(size_t(N) * K);
  lo_nvfp4_dequant(xq, xs, M, K, xa.data());
  lo_nvfp4_dequant(wq, ws, N, K, wa.data());
  parallel_for(M, [&](int lo, int hi) {
    for (int m = lo; m < hi; ++m)
      for (int n = 0; n < N; ++n) {
        double acc = 0;
        const float *a = &xa[size_t(m) * K], *b = &wa[size_t(n) * K];
        for (int k = 0; k < K; ++k) acc += double(a[k]) * double(b[k]);
        float& o = y[size_t(m) * ldy + n];
        o = float(acc * double(alpha) + (accumulate ? double(o) : 0.0));
      }
  });
  return 0;
}

// Gemma RMSNorm rows in fp32 with the sum of squares in double: x * rstd * (1 + w) (src/core/prefill_gemm.cu:426-459; the
// quantization that follows it there is lo_nvfp4_quant_act of this output).  w: BF16 bit patterns [H].
int lo_rmsnorm_rows(const float* x, const uint16_t* w, int M, int H, float eps, float* out) {
  for (int r = 0; r < M; ++r) {
    double ss = 0;
    for (int i = 0; i < H; ++i) ss += double(x[size_t(r) * H + i]) * x[size_t(r) * H + i];
    const float rstd = 1.f / std::sqrt(float(ss / H) + eps);
    for (int i = 0; i < H; ++i) {
      const uint32_t u = uint32_t(w[i]) << 16;
      float wf;
      std::memcpy(&wf, &u, 4);
      out[size_t(r) * H + i] = x[size_t(r) * H + i] * rstd * (1.f + wf);
    }
  }
  return 0;
}

}  // extern "C"
