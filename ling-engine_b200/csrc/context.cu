// context.cu -- the engine context behind the C ABI: every device buffer allocated at creation (the reference allocates
// nothing while serving, src/core/engine.cpp:169 in the reference project), weights, the paged FP8 KV pool and the
// DeltaNet state slots, and the verify step as one enqueue function that is captured into a CUDA graph per
// capacity class (the reference replays three graphs per step with two host syncs, src/core/speculate.cpp:473-514;
// here packing, forward pass, argmax, acceptance, compaction and commit are one graph and one sync).
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <map>
#include <vector>

#include "chain.h"
#include "draft_head.h"
#include "gemm.h"
#include "kernels.h"

namespace lb {

thread_local std::string g_error;
void set_error(const std::string& what) { g_error = what; }
// Programmatic dependent launch is a property of the launching host thread (one thread drives one context): a context's
// step sets it for its own launches and puts the caller's setting back, so contexts on different threads (one per GPU) do
// not see each other's choice.
static thread_local bool g_pdl = false;
void set_pdl(bool on) { g_pdl = on; }
bool pdl_enabled() { return g_pdl; }

namespace {

template <typename T>
int dev_alloc(T** p, size_t n, bool zero = true) {
  *p = nullptr;
  if (n == 0) n = 1;
  if (!cuda_ok(cudaMalloc(reinterpret_cast<void**>(p), n * sizeof(T)), "cudaMalloc")) return LING_B200_ERR_CUDA;
  if (zero && !cuda_ok(cudaMemset(*p, 0, n * sizeof(T)), "cudaMemset")) return LING_B200_ERR_CUDA;
  return LING_B200_OK;
}
#define LB_TRY(call)                      \
  do {                                    \
    const int rc__ = (call);              \
    if (rc__ != LING_B200_OK) return rc__; \
  } while (0)

struct LayerW {
  bool full = false;
  __nv_bfloat16 *input_norm = nullptr, *post_norm = nullptr;
  Fp8Matrix gu, down;       // gate|up fused along N, down
  Fp8Matrix in, out;        // DeltaNet: in_qkv|in_z fused, out
  __nv_bfloat16 *in_a = nullptr, *in_b = nullptr, *conv = nullptr, *A_log = nullptr, *dt_bias = nullptr, *lin_norm = nullptr;
  Fp8Matrix qkv, o;         // attention: q|k|v fused, o
  __nv_bfloat16 *q_norm = nullptr, *k_norm = nullptr;
};

enum Family { kFamGemm = 0, kFamAttn, kFamGdn, kFamElem, kFamHead, kFamStep, kFamCount };

}  // namespace
}  // namespace lb

using namespace lb;

struct ling_b200_ctx {
  ling_b200_model_config cfg{};
  ling_b200_options opt{};
  ModelDims d{};
  int sm_count = 148;
  cudaStream_t stream = nullptr;
  std::vector<void*> owned;  // every device allocation, freed at destroy
  std::vector<int> attn_index, gdn_index;

  // weights
  std::vector<LayerW> layers;
  __nv_bfloat16 *embed = nullptr, *final_norm = nullptr;
  Fp8Matrix head;
  float* upload = nullptr;  // staging for ling_b200_set_tensor (largest tensor)
  size_t upload_floats = 0;

  // activations
  float *h = nullptr, *xn = nullptr, *core = nullptr;
  __half* qh = nullptr;
  Fp8Acts xq_h, xq_v, xq_a, xq_i;
  float* planes[2] = {nullptr, nullptr};
  size_t plane_floats = 0;
  float *pre = nullptr, *post = nullptr, *g = nullptr, *beta = nullptr;  // [n_gdn][rows][..], saved for the commit
  float *part_o = nullptr, *part_ml = nullptr;
  int chunk_slots = 0;
  bool sibling = false;  // weights, KV pool, page tables and state slots belong to another context
  HeadEpilogue head_ep;
  float* logits = nullptr;
  float* taps = nullptr;
  float* flush = nullptr;
  size_t flush_floats = 0;

  // sessions
  KvPoolDev kv;
  float *gdn_state = nullptr, *conv_state = nullptr;  // [slot][gdn layer][...]
  unsigned* swiglu_tickets = nullptr;  // [token tiles][gate tiles], zero between launches (GemmCall::swiglu)
  uint8_t* state_arena = nullptr;  // saved states of the prefix KV store (ling_b200_state_arena_reserve)
  size_t state_arena_bytes = 0;
  size_t state_layer = 0, conv_layer = 0;             // floats per layer

  // the step
  StepBuffers sb;
  uint8_t* stage_dev = nullptr;   // host-written block: n_seqs, seqs, parent, token, force
  uint8_t* stage_host = nullptr;  // pinned mirror
  size_t stage_bytes = 0;
  ling_b200_seq_result* results_host = nullptr;  // pinned
  int* err_host = nullptr;                       // pinned
  int staged_seqs = 0, staged_rows = 0, staged_flags = 0, last_rows = 0, last_seqs = 0, last_flags = 0;
  long staged_slots = 0;  // attention partial slots the staged sequences' contexts take
  std::map<std::pair<int, int>, cudaGraphExec_t> graphs;  // (row class, flags)
  int launches_per_step = 0;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  cudaStream_t side = nullptr;               // the gating projections run here beside the in projection (options.gating_stream)
  cudaEvent_t ev_fork = nullptr, ev_join = nullptr;

  // persistent layer segments (options.chain): dependency counters of every chain of a step, partial sums of squares
  unsigned* chain_counters = nullptr;
  size_t chain_words = 0;
  float* chain_ssq = nullptr;
  int chain_next = 0;  // chains enqueued so far in the step being built
  int chain_ahead = 0;  // K blocks of L2 prefetch ahead of the loads (measured on the 27B single-stream step: 0 -> 10.1 ms, 8 -> 11.4, 32 -> 13.2)

  // GEMM timeline (LING_B200_TIMELINE=1 at creation): four %globaltimer stamps per GEMM launch of the last step
  unsigned long long* timeline = nullptr;
  int timeline_next = 0;

  static constexpr int kTimelineLaunches = 1024;

  // profiling of one eager replay
  bool profiling = false;
  std::vector<std::pair<int, std::pair<cudaEvent_t, cudaEvent_t>>> prof;

  template <typename T>
  int alloc(T** p, size_t n, bool zero = true) {
    const int rc = dev_alloc(p, n, zero);
    if (rc == LING_B200_OK) owned.push_back(*p);
    return rc;
  }
  int alloc_matrix(Fp8Matrix& w, int N, int K) {
    w.N = N, w.K = K, w.N_pad = round_up(N, kTileN), w.K_pad = round_up(K, kBlockK), w.KB = w.K_pad / kBlockK;
    w.splits = opt.gemm_impl == 1 ? 1 : choose_splits(w.N_pad, w.KB, sm_count);  // the CUDA-core GEMM never splits K
    LB_TRY(alloc(&w.codes, size_t(w.N_pad) * w.K_pad));
    LB_TRY(alloc(&w.scales, size_t(w.KB) * w.N_pad));
    return make_weight_map(w);
  }
  int alloc_acts(Fp8Acts& x, int K) {
    x.K = K, x.K_pad = round_up(K, kBlockK), x.KB = x.K_pad / kBlockK, x.rows_alloc = d.rows_alloc;
    LB_TRY(alloc(&x.codes, size_t(x.rows_alloc) * x.K_pad));
    LB_TRY(alloc(&x.scales, size_t(x.KB) * x.rows_alloc));
    return make_acts_maps(x);
  }
  QuantOut qout(const Fp8Acts& x) const { return QuantOut{x.codes, x.scales, x.K, x.K_pad, x.rows_alloc}; }
};

namespace {

// The capacity class a step of M packed rows runs in (one graph per class and flag set; grids and the GEMMs' token tiles are
// sized for it): the token tile up to 128 rows, multiples of 32 beyond -- fine enough for the GEMM to pick the tile size with
// the least padding (token_tile), at most 64 classes in all.
int row_class(int M) { return M <= 128 ? token_tile(M) : round_up(M, 32); }

struct Timed {
  ling_b200_ctx* c;
  bool on;
  cudaEvent_t a = nullptr, b = nullptr;
  Timed(ling_b200_ctx* ctx, int fam) : c(ctx), on(ctx->profiling) {
    ++c->launches_per_step;
    if (!on) return;
    cudaEventCreate(&a), cudaEventCreate(&b);
    cudaEventRecord(a, c->stream);
    c->prof.push_back({fam, {a, b}});
  }
  ~Timed() {
    if (on) cudaEventRecord(b, c->stream);
  }
};

Planes planes_of(const ling_b200_ctx* c, int which, const Fp8Matrix& w, bool head = false) {
  Planes p;
  p.p = c->planes[which];
  p.n = head ? 1 : w.splits;
  p.ld = w.N_pad;
  p.stride = size_t(c->d.rows_alloc) * w.N_pad;
  return p;
}

int run_gemm(ling_b200_ctx* c, const Fp8Matrix& w, const Fp8Acts& x, int which, int rows, const HeadEpilogue* head = nullptr,
             const SwigluEpilogue* swiglu = nullptr) {
  Timed t(c, head ? kFamHead : kFamGemm);
  GemmCall g;
  g.W = &w, g.X = &x, g.M = rows;
  g.out = head ? c->logits : c->planes[which];
  g.ld = head ? w.N : w.N_pad;
  g.split_stride = size_t(c->d.rows_alloc) * w.N_pad;
  g.head = head;
  g.swiglu = swiglu;
  g.impl = c->opt.gemm_impl;
  g.err_flag = c->sb.err;
  if (c->timeline && c->timeline_next < ling_b200_ctx::kTimelineLaunches) g.timeline = c->timeline + 4 * size_t(c->timeline_next++);
  return gemm_launch(g, c->stream);
}

ChainGemm chain_gemm(const ling_b200_ctx* c, const Fp8Matrix& w, const Fp8Acts& x, int which) {
  ChainGemm g;
  g.mapW = w.map, g.mapX = x.map[0];
  g.ws = w.scales, g.xs = x.scales;
  g.out = c->planes[which];
  g.split_stride = size_t(c->d.rows_alloc) * w.N_pad;
  g.N = w.N, g.N_pad = w.N_pad, g.KB = w.KB, g.splits = w.splits, g.xrows = x.rows_alloc;
  return g;
}
ChainProgram chain_base(ling_b200_ctx* c, int rows) {
  ChainProgram P;
  P.n_rows = c->sb.n_rows_total, P.rows_grid = rows;
  P.counters = c->chain_counters + size_t(c->chain_next) * kChainCounterWords;
  P.ssq = c->chain_ssq, P.err_flag = c->sb.err, P.l2_ahead = c->chain_ahead;
  // with the timeline on, chain k's stamps take the slots of GEMM launches 4 (k + 1) .. 4 (k + 1) + 3 (16 words)
  if (c->timeline && 4 * (c->chain_next + 2) <= ling_b200_ctx::kTimelineLaunches - 32) P.stamps = c->timeline + 16 * size_t(c->chain_next + 1);
  return P;
}
// The head of a layer as one persistent kernel: residual add + input norm (+ the DeltaNet gating projections) and the in /
// q|k|v projection.
ChainProgram chain_front(ling_b200_ctx* c, int l, int rows, const Planes& carry) {
  const ModelDims& d = c->d;
  const LayerW& L = c->layers[l];
  ChainProgram P = chain_base(c, rows);
  P.n_gemm = 1, P.norm_gemm = 0;
  P.norm = ChainNorm{c->h, carry, l == 0 ? c->sb.token : nullptr, c->embed, L.input_norm, L.full ? nullptr : c->xn, c->qout(c->xq_h), d.H, d.eps};
  if (!L.full) {
    const int gl = c->gdn_index[l];
    P.has_ab = 1;
    P.ab = ChainAb{c->xn, L.in_a, L.in_b, L.A_log, L.dt_bias, c->g + size_t(gl) * d.rows_alloc * d.HV, c->beta + size_t(gl) * d.rows_alloc * d.HV,
                   d.H, d.HV};
  }
  P.g[0] = chain_gemm(c, L.full ? L.qkv : L.in, c->xq_h, 0);
  return P;
}
// The rest of a layer behind its mixer as one persistent kernel: out / o projection, residual add + post norm, gate|up,
// SiLU(gate) * up, down.
ChainProgram chain_back(ling_b200_ctx* c, int l, int rows) {
  const ModelDims& d = c->d;
  const LayerW& L = c->layers[l];
  ChainProgram P = chain_base(c, rows);
  P.n_gemm = 3, P.norm_gemm = 1, P.has_silu = 1;
  P.g[0] = chain_gemm(c, L.full ? L.o : L.out, L.full ? c->xq_a : c->xq_v, 1);
  P.norm = ChainNorm{c->h, planes_of(c, 1, L.full ? L.o : L.out), nullptr, nullptr, L.post_norm, nullptr, c->qout(c->xq_h), d.H, d.eps};
  P.g[1] = chain_gemm(c, L.gu, c->xq_h, 0);
  P.silu = ChainSilu{d.I, round_up(d.I, kTileN), c->qout(c->xq_i)};
  P.g[2] = chain_gemm(c, L.down, c->xq_i, 1);
  return P;
}
int run_chain(ling_b200_ctx* c, const ChainProgram& P) {
  Timed t(c, kFamGemm);
  ++c->chain_next;
  return chain_launch(P, c->sm_count, c->stream);
}
// Whether the step of this row class runs its layers' segments as persistent kernels: asked for, the tensor-core path,
// one 32-row token tile, and shapes the chain kernel covers.
bool use_chains(ling_b200_ctx* c, int rows) {
  if (!c->opt.chain || c->opt.gemm_impl != 0 || rows > kChainRows) return false;
  const int saved = c->chain_next;
  bool ok = true;
  Planes none;
  none.p = nullptr;
  for (int l = 0; l < c->cfg.layers && ok; ++l)
    ok = chain_supported(chain_front(c, l, rows, none), c->sm_count) && chain_supported(chain_back(c, l, rows), c->sm_count);
  c->chain_next = saved;
  return ok;
}

// The whole step on the context's stream.  rows = the capacity class (grids and GEMM extents); the kernels read the
// real extents from device memory.  Order of the forward pass: src/core/engine.cpp:1288-1745 (verify branch).
// Sets the calling thread's dependent-launch switch for a scope and restores what the caller had set.
struct PdlScope {
  bool before;
  explicit PdlScope(bool on) : before(pdl_enabled()) { set_pdl(on); }
  ~PdlScope() { set_pdl(before); }
};
// Weights that the long glue kernels' idle CTAs ask into L2 for the GEMMs behind them, in MB (measured on the 27B
// single-stream step: the DeltaNet kernel 48 MB of gate|up, 7.97 -> 7.59 ms per step; the attention kernel the whole o
// projection and 48 MB of gate|up; more than ~64 MB per kernel, the down projection or the next layer's in projection were
// slower), requested 3 us after the kernel's dependency wait.
constexpr int kPfAttnOMb = 32, kPfAttnGuMb = 48, kPfGdnGuMb = 48, kPfDelayNs = 3000;
int enqueue_step_body(ling_b200_ctx* c, int rows, int flags);
int enqueue_step(ling_b200_ctx* c, int rows, int flags) {
  PdlScope pdl(c->opt.pdl != 0);
  return enqueue_step_body(c, rows, flags);
}
int enqueue_step_body(ling_b200_ctx* c, int rows, int flags) {
  const ModelDims& d = c->d;
  cudaStream_t s = c->stream;
  const int* n_rows = c->sb.n_rows_total;
  const bool taps = (flags & LING_B200_STEP_KEEP_TAPS) != 0;
  const bool keep_logits = (flags & LING_B200_STEP_KEEP_LOGITS) != 0;
  c->launches_per_step = 0;
  c->timeline_next = 0;
  c->chain_next = 0;
  const bool chains = use_chains(c, rows);
  if (chains) LB_CUDA(cudaMemsetAsync(c->chain_counters, 0, c->chain_words * sizeof(unsigned), s));  // every chain starts from zero counters
  {
    Timed t(c, kFamStep);
    LB_TRY(pack_launch(c->sb, d, s));
  }
  Planes none;
  none.p = nullptr;
  Planes carry = none;  // the previous layer's down projection, still to be added to the residual
  for (int l = 0; l < c->cfg.layers; ++l) {
    const LayerW& L = c->layers[l];
    if (chains) {
      LB_TRY(run_chain(c, chain_front(c, l, rows, carry)));
    } else {
      Timed t(c, kFamElem);
      LB_TRY(norm_quant_launch(c->h, carry, l == 0 ? c->sb.token : nullptr, c->embed, L.input_norm, L.full ? nullptr : c->xn,
                               c->qout(c->xq_h), n_rows, rows, d.H, d.eps, s));
    }
    if (L.full) {
      const int al = c->attn_index[l];
      const bool tc = c->opt.gemm_impl == 0 && attention_tc_supported(d);
      if (!chains) LB_TRY(run_gemm(c, L.qkv, c->xq_h, 0, rows));
      const Planes p0 = planes_of(c, 0, L.qkv);
      {
        Timed t(c, kFamAttn);
        LB_TRY(attn_prepare_launch(p0, c->sb, d, al, L.q_norm, L.k_norm, c->qh, c->kv, rows, s));
      }
      {
        Timed t(c, kFamAttn);
        // tcgen05/TMEM attention; the mma.sync form stays as the cross-check implementation (gemm_impl = 1)
        PrefetchPlan plan;
        if (tc && c->opt.pdl) {
          auto range = [&](int i, const Fp8Matrix& w, int mb) {
            plan.p[i] = w.codes, plan.bytes[i] = std::min<size_t>(size_t(mb) << 20, size_t(w.N_pad) * w.K_pad);
          };
          range(0, L.o, kPfAttnOMb), range(1, L.gu, kPfAttnGuMb);
          plan.delay_ns = kPfDelayNs;
        }
        if (tc)
          LB_TRY(attention_tc_launch(c->qh, c->sb, d, al, c->kv, c->part_o, c->part_ml, c->chunk_slots, c->sm_count, plan,
                                     c->timeline && al == 0 ? c->timeline + 4 * size_t(ling_b200_ctx::kTimelineLaunches - 16) : nullptr, s));
        else
          LB_TRY(attention_launch(c->qh, c->sb, d, al, c->kv, c->part_o, c->part_ml, c->chunk_slots, c->sm_count * 2, s));
      }
      {
        Timed t(c, kFamAttn);
        LB_TRY(attn_combine_launch(c->part_o, c->part_ml, p0, c->sb, d, c->qout(c->xq_a), nullptr, rows,
                                   c->opt.max_context / kAttnChunkShort + 2, tc ? kAttnTcRows : kAttnRowTile,
                                   tc ? c->sm_count : c->sm_count * 2, c->chunk_slots, s));
      }
      if (!chains) LB_TRY(run_gemm(c, L.o, c->xq_a, 1, rows));
      carry = planes_of(c, 1, L.o);
    } else {
      const int gl = c->gdn_index[l];
      float* pre = c->pre + size_t(gl) * d.rows_alloc * d.C;
      float* post = c->post + size_t(gl) * d.rows_alloc * d.C;
      float* g = c->g + size_t(gl) * d.rows_alloc * d.HV;
      float* beta = c->beta + size_t(gl) * d.rows_alloc * d.HV;
      const bool side_gating = !chains && c->opt.gating_stream >= 0 && !c->profiling;
      if (side_gating) {
        // the gating needs only the normalized row and only the DeltaNet kernel needs the gating: it runs on a second stream
        // beside the in projection (fork after the norm, join before the DeltaNet kernel)
        ++c->launches_per_step;
        LB_CUDA(cudaEventRecord(c->ev_fork, s));
        LB_CUDA(cudaStreamWaitEvent(c->side, c->ev_fork, 0));
        LB_TRY(ab_gating_launch(c->xn, L.in_a, L.in_b, L.A_log, L.dt_bias, g, beta, n_rows, rows, d.H, d.HV, c->side));
        LB_CUDA(cudaEventRecord(c->ev_join, c->side));
      } else if (!chains) {
        // the gating needs only the normalized row, so it runs before the in projection: with dependent launch the
        // GEMM's CTAs are already resident and stream their first weight tiles while it executes
        Timed t(c, kFamGdn);
        LB_TRY(ab_gating_launch(c->xn, L.in_a, L.in_b, L.A_log, L.dt_bias, g, beta, n_rows, rows, d.H, d.HV, s));
      }
      if (!chains) LB_TRY(run_gemm(c, L.in, c->xq_h, 0, rows));
      if (side_gating) LB_CUDA(cudaStreamWaitEvent(s, c->ev_join, 0));
      const Planes p0 = planes_of(c, 0, L.in);
      if (gdn_fused_supported(d)) {
        Timed t(c, kFamGdn);
        PrefetchPlan plan;
        if (c->opt.pdl) {
          plan.p[0] = L.gu.codes;
          plan.bytes[0] = std::min<size_t>(size_t(kPfGdnGuMb) << 20, size_t(L.gu.N_pad) * L.gu.K_pad);
          plan.delay_ns = kPfDelayNs;
        }
        LB_TRY(gdn_fused_launch(p0, c->sb, d, L.conv, c->conv_state + size_t(gl) * c->conv_layer, c->conv_layer * d.n_gdn, g, beta,
                                c->gdn_state + size_t(gl) * c->state_layer, c->state_layer * d.n_gdn, L.lin_norm, c->qout(c->xq_v),
                                pre, post, nullptr, c->opt.sessions, c->sm_count, plan,
                                c->timeline && gl == 0 ? c->timeline + 4 * size_t(ling_b200_ctx::kTimelineLaunches - 4) : nullptr, s));
      } else {
        {
          Timed t(c, kFamGdn);
          LB_TRY(conv_tree_launch(p0, c->sb, d, L.conv, c->conv_state + size_t(gl) * c->conv_layer, c->conv_layer * d.n_gdn, pre,
                                  post, rows, s));
        }
        {
          Timed t(c, kFamGdn);
          LB_TRY(gdn_tree_launch(post, g, beta, c->sb, d, c->gdn_state + size_t(gl) * c->state_layer, c->state_layer * d.n_gdn,
                                 c->core, c->sm_count * 4, s));
        }
        {
          Timed t(c, kFamGdn);
          LB_TRY(gated_norm_quant_launch(c->core, p0, d.C, L.lin_norm, c->qout(c->xq_v), n_rows, rows, d.HV, d.Dv, d.eps, s));
        }
      }
      if (!chains) LB_TRY(run_gemm(c, L.out, c->xq_v, 1, rows));
      carry = planes_of(c, 1, L.out);
    }
    if (chains) {
      LB_TRY(run_chain(c, chain_back(c, l, rows)));
    } else {
      {
        Timed t(c, kFamElem);
        LB_TRY(norm_quant_launch(c->h, carry, nullptr, nullptr, L.post_norm, nullptr, c->qout(c->xq_h), n_rows, rows, d.H, d.eps, s));
      }
      if (c->opt.fuse_swiglu > 0 && c->opt.gemm_impl == 0) {
        // the activation and its FP8 copy inside the GEMM: the CTA that completes a (gate tile, up tile) pair writes them
        // (measured slower than the kernel of its own on the 27B single-stream step: 7.96 against 7.49 ms; off by default)
        const QuantOut q = c->qout(c->xq_i);
        const SwigluEpilogue sw{c->swiglu_tickets, d.I, round_up(d.I, kTileN), q.codes, q.scales, q.K_pad, q.rows_alloc};
        LB_TRY(run_gemm(c, L.gu, c->xq_h, 0, rows, nullptr, &sw));
      } else {
        LB_TRY(run_gemm(c, L.gu, c->xq_h, 0, rows));
        Timed t(c, kFamElem);
        LB_TRY(silu_mul_quant_launch(planes_of(c, 0, L.gu), d.I, round_up(d.I, kTileN), c->qout(c->xq_i), n_rows, rows, s));
      }
      LB_TRY(run_gemm(c, L.down, c->xq_i, 1, rows));
    }
    carry = planes_of(c, 1, L.down);
    if (taps) {
      Timed t(c, kFamElem);
      LB_TRY(tap_launch(c->h, carry, c->taps + size_t(l) * c->opt.debug_rows * d.H, n_rows, std::min(rows, c->opt.debug_rows),
                        d.H, s));
    }
  }
  {
    Timed t(c, kFamElem);
    LB_TRY(norm_quant_launch(c->h, carry, nullptr, nullptr, c->final_norm, c->xn, c->qout(c->xq_h), n_rows, rows, d.H, d.eps, s));
  }
  if (taps) {
    Timed t(c, kFamElem);
    LB_TRY(copy_rows_launch(c->xn, c->taps + size_t(c->cfg.layers) * c->opt.debug_rows * d.H, n_rows,
                            std::min(rows, c->opt.debug_rows), d.H, s));
  }
  HeadEpilogue ep = c->head_ep;
  ep.store_logits = keep_logits;
  LB_TRY(run_gemm(c, c->head, c->xq_h, 0, keep_logits ? std::min(rows, c->opt.debug_rows) : rows, &ep));
  {
    Timed t(c, kFamHead);
    LB_TRY(argmax_reduce_launch(ep.tile_val, ep.tile_idx, c->head.N_pad / kTileN, ep.rows_alloc, c->sb.argmax_id,
                                c->sb.argmax_val, n_rows, rows, s));
  }
  {
    Timed t(c, kFamStep);
    LB_TRY(accept_launch(c->sb, d, 0, s));
  }
  if (flags & LING_B200_STEP_COMMIT) {
    {
      Timed t(c, kFamStep);
      LB_TRY(kv_compact_launch(c->sb, d, c->kv, s));
    }
    {
      Timed t(c, kFamStep);
      LB_TRY(conv_commit_launch(c->sb, d, c->pre, size_t(d.rows_alloc) * d.C, c->conv_state, c->conv_layer * d.n_gdn,
                                c->conv_layer, s));
    }
    {
      Timed t(c, kFamStep);
      LB_TRY(gdn_commit_launch(c->sb, d, c->post, c->g, c->beta, size_t(d.rows_alloc) * d.C, size_t(d.rows_alloc) * d.HV,
                               c->gdn_state, c->state_layer * d.n_gdn, c->state_layer, c->sm_count * 64, s));
    }
  }
  return LING_B200_OK;
}

int check_ctx(const ling_b200_ctx* c) {
  if (!c) {
    set_error("null context");
    return LING_B200_ERR_ARG;
  }
  return LING_B200_OK;
}

// A tensor's place in the fused matrices: destination matrix, first row.
struct MatSlot {
  Fp8Matrix* w = nullptr;
  int row_off = 0, rows = 0, cols = 0;
};
MatSlot mat_slot(ling_b200_ctx* c, int layer, int tensor) {
  const ModelDims& d = c->d;
  MatSlot m;
  if (tensor == LING_B200_T_LM_HEAD) return MatSlot{&c->head, 0, d.V, d.H};
  if (layer < 0 || layer >= c->cfg.layers) return m;
  LayerW& L = c->layers[layer];
  switch (tensor) {
    case LING_B200_T_GATE: return MatSlot{&L.gu, 0, d.I, d.H};
    case LING_B200_T_UP: return MatSlot{&L.gu, round_up(d.I, kTileN), d.I, d.H};  // on a tile boundary
    case LING_B200_T_DOWN: return MatSlot{&L.down, 0, d.H, d.I};
  }
  if (L.full) {
    switch (tensor) {
      case LING_B200_T_Q: return MatSlot{&L.qkv, 0, d.Hq * 2 * d.D, d.H};
      case LING_B200_T_K: return MatSlot{&L.qkv, d.Hq * 2 * d.D, d.Hkv * d.D, d.H};
      case LING_B200_T_V: return MatSlot{&L.qkv, d.Hq * 2 * d.D + d.Hkv * d.D, d.Hkv * d.D, d.H};
      case LING_B200_T_O: return MatSlot{&L.o, 0, d.H, d.Hq * d.D};
    }
  } else {
    switch (tensor) {
      case LING_B200_T_IN_QKV: return MatSlot{&L.in, 0, d.C, d.H};
      case LING_B200_T_IN_Z: return MatSlot{&L.in, d.C, d.Vs, d.H};
      case LING_B200_T_OUT: return MatSlot{&L.out, 0, d.H, d.Vs};
    }
  }
  return m;
}
struct VecSlot {
  __nv_bfloat16* p = nullptr;
  size_t n = 0;
  float std_ = 0.02f, bias = 0.f;
};
VecSlot vec_slot(ling_b200_ctx* c, int layer, int tensor) {
  const ModelDims& d = c->d;
  if (tensor == LING_B200_T_EMBED) return VecSlot{c->embed, size_t(d.V) * d.H};
  if (tensor == LING_B200_T_FINAL_NORM) return VecSlot{c->final_norm, size_t(d.H)};
  if (layer < 0 || layer >= c->cfg.layers) return VecSlot{};
  LayerW& L = c->layers[layer];
  switch (tensor) {
    case LING_B200_T_INPUT_NORM: return VecSlot{L.input_norm, size_t(d.H)};
    case LING_B200_T_POST_NORM: return VecSlot{L.post_norm, size_t(d.H)};
  }
  if (L.full) {
    switch (tensor) {
      case LING_B200_T_Q_NORM: return VecSlot{L.q_norm, size_t(d.D)};
      case LING_B200_T_K_NORM: return VecSlot{L.k_norm, size_t(d.D)};
    }
  } else {
    switch (tensor) {
      case LING_B200_T_IN_A: return VecSlot{L.in_a, size_t(d.HV) * d.H};
      case LING_B200_T_IN_B: return VecSlot{L.in_b, size_t(d.HV) * d.H};
      case LING_B200_T_CONV: return VecSlot{L.conv, size_t(d.C) * 4, 0.3f};
      case LING_B200_T_A_LOG: return VecSlot{L.A_log, size_t(d.HV), 0.5f};
      case LING_B200_T_DT_BIAS: return VecSlot{L.dt_bias, size_t(d.HV), 0.5f};
      case LING_B200_T_LIN_NORM: return VecSlot{L.lin_norm, size_t(d.Dv), 0.02f, 1.f};
    }
  }
  return VecSlot{};
}

const int kLayerTensorsFull[] = {LING_B200_T_INPUT_NORM, LING_B200_T_POST_NORM, LING_B200_T_GATE, LING_B200_T_UP,
                                 LING_B200_T_DOWN,       LING_B200_T_Q,         LING_B200_T_K,    LING_B200_T_V,
                                 LING_B200_T_O,          LING_B200_T_Q_NORM,    LING_B200_T_K_NORM};
const int kLayerTensorsGdn[] = {LING_B200_T_INPUT_NORM, LING_B200_T_POST_NORM, LING_B200_T_GATE,   LING_B200_T_UP,
                                LING_B200_T_DOWN,       LING_B200_T_IN_QKV,    LING_B200_T_IN_Z,   LING_B200_T_OUT,
                                LING_B200_T_IN_A,       LING_B200_T_IN_B,      LING_B200_T_CONV,   LING_B200_T_A_LOG,
                                LING_B200_T_DT_BIAS,    LING_B200_T_LIN_NORM};

int synth_tensor(ling_b200_ctx* c, uint64_t seed, int layer, int tensor) {
  const uint64_t key = stream_key(seed, weight_stream(layer, tensor));
  const MatSlot m = mat_slot(c, layer, tensor);
  if (m.w) return quant_weight_launch(nullptr, key, 0.02f, 1, m.w->codes, m.w->scales, m.row_off, m.rows, m.cols, m.w->N_pad,
                                      m.w->K_pad, c->stream);
  const VecSlot v = vec_slot(c, layer, tensor);
  if (v.p) return fill_bf16_launch(nullptr, key, v.std_, v.bias, 1, v.p, v.n, c->stream);
  set_error("synth: unknown tensor");
  return LING_B200_ERR_ARG;
}

int finish(ling_b200_ctx* c) {
  LB_CUDA(cudaStreamSynchronize(c->stream));
  return LING_B200_OK;
}

}  // namespace

// ================================================================================================ C ABI
extern "C" {

const char* ling_b200_last_error(void) { return g_error.c_str(); }
void ling_b200_set_pdl(int on) { set_pdl(on != 0); }
int ling_b200_pdl_enabled(void) { return pdl_enabled() ? 1 : 0; }
int ling_b200_abi_version(void) { return 1; }
int ling_b200_token_tile(int rows) { return rows < 1 ? 0 : token_tile(rows); }
int ling_b200_row_class(int rows) { return rows < 1 ? 0 : row_class(rows); }

int ling_b200_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) return 0;
  return n;
}
int ling_b200_device_name(int device, char* buf, int len) {
  cudaDeviceProp p;
  LB_CUDA(cudaGetDeviceProperties(&p, device));
  std::snprintf(buf, size_t(len), "%s (sm_%d%d, %d SMs)", p.name, p.major, p.minor, p.multiProcessorCount);
  return LING_B200_OK;
}

// share != nullptr: a sibling context -- the weights, the KV pool, the page tables and the DeltaNet state slots are `share`'s (not
// owned, not freed here); the activations, step buffers, streams and graphs are its own.
static int create_impl(const ling_b200_model_config* cfg, const ling_b200_options* opt, const ling_b200_ctx* share, ling_b200_ctx** out) {
  if (!cfg || !opt || !out) {
    set_error("create: null argument");
    return LING_B200_ERR_ARG;
  }
  *out = nullptr;
  const int G = cfg->kv_heads > 0 ? cfg->heads / cfg->kv_heads : 0;
  const bool ok = cfg->layers >= 1 && cfg->layers <= LING_B200_MAX_LAYERS && cfg->hidden % 4 == 0 && cfg->hidden <= 8192 &&
                  cfg->intermediate % 4 == 0 && cfg->conv_kernel == 4 && cfg->kv_heads > 0 && cfg->heads % cfg->kv_heads == 0 &&
                  (cfg->head_dim == 64 || cfg->head_dim == 128 || cfg->head_dim == 256) && cfg->rotary_dim % 2 == 0 &&
                  cfg->rotary_dim <= cfg->head_dim && (cfg->lin_k_dim == 64 || cfg->lin_k_dim == 128) &&
                  cfg->lin_v_dim % 32 == 0 && cfg->lin_v_dim <= 128 && cfg->lin_k_heads > 0 &&
                  cfg->lin_v_heads % cfg->lin_k_heads == 0 && G >= 1 && opt->sessions >= 1 &&
                  (opt->page_tokens == 16 || opt->page_tokens == 32 || opt->page_tokens == 64) && opt->pool_pages >= 1 &&
                  opt->max_seqs >= 1 && opt->max_seqs <= LING_B200_MAX_SEQS && opt->max_rows >= 1 &&
                  opt->max_rows <= LING_B200_MAX_ROWS && opt->max_context >= 1 && opt->debug_rows >= 0;
  if (!ok) {
    set_error("create: unsupported model configuration or options");
    return LING_B200_ERR_ARG;
  }
  LB_CUDA(cudaSetDevice(opt->device));
  cudaDeviceProp prop;
  LB_CUDA(cudaGetDeviceProperties(&prop, opt->device));
  if (prop.major != 10) {
    set_error(std::string("this library is built for sm_100a (B200) only; device is ") + prop.name);
    return LING_B200_ERR_UNSUPPORTED;
  }
  ling_b200_ctx* c = new ling_b200_ctx;
  *out = c;  // the caller destroys it also after a failed creation
  c->cfg = *cfg, c->opt = *opt;
  c->sibling = share != nullptr;
  c->sm_count = prop.multiProcessorCount;
  ModelDims& d = c->d;
  d.H = cfg->hidden, d.I = cfg->intermediate, d.V = cfg->vocab, d.Hq = cfg->heads, d.Hkv = cfg->kv_heads, d.D = cfg->head_dim;
  d.rot = cfg->rotary_dim, d.Hk = cfg->lin_k_heads, d.HV = cfg->lin_v_heads, d.Dk = cfg->lin_k_dim, d.Dv = cfg->lin_v_dim;
  d.C = 2 * d.Hk * d.Dk + d.HV * d.Dv, d.Vs = d.HV * d.Dv;
  d.theta = cfg->rope_theta, d.eps = cfg->eps;
  d.page_tokens = opt->page_tokens, d.pool_pages = opt->pool_pages;
  d.max_pages = ceil_div(opt->max_context, opt->page_tokens);
  d.rows_alloc = round_up(opt->max_rows, 128);
  d.max_seqs = opt->max_seqs;
  c->layers.resize(cfg->layers);
  c->attn_index.assign(cfg->layers, -1), c->gdn_index.assign(cfg->layers, -1);
  d.n_attn = d.n_gdn = 0;
  for (int l = 0; l < cfg->layers; ++l) {
    c->layers[l].full = cfg->full_attention[l] != 0;
    if (c->layers[l].full) c->attn_index[l] = d.n_attn++;
    else c->gdn_index[l] = d.n_gdn++;
  }
  LB_TRY(gemm_init());
  LB_TRY(kernels_init());
  LB_CUDA(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
  LB_CUDA(cudaStreamCreateWithFlags(&c->side, cudaStreamNonBlocking));
  LB_CUDA(cudaEventCreateWithFlags(&c->ev_fork, cudaEventDisableTiming));
  LB_CUDA(cudaEventCreateWithFlags(&c->ev_join, cudaEventDisableTiming));
  LB_CUDA(cudaEventCreate(&c->ev0));
  LB_CUDA(cudaEventCreate(&c->ev1));

  // ---- weights
  size_t biggest = size_t(d.V) * d.H;
  if (share) {
    c->embed = share->embed, c->final_norm = share->final_norm, c->head = share->head;
    for (int l = 0; l < cfg->layers; ++l) c->layers[l] = share->layers[l];
  } else {
    LB_TRY(c->alloc(&c->embed, size_t(d.V) * d.H));
    LB_TRY(c->alloc(&c->final_norm, size_t(d.H)));
    LB_TRY(c->alloc_matrix(c->head, d.V, d.H));
    c->head.splits = 1;
  }
  size_t max_plane = 0;  // floats of the largest GEMM output (all K splits); the head writes no planes
  for (int l = 0; l < cfg->layers; ++l) {
    LayerW& L = c->layers[l];
    std::vector<Fp8Matrix*> mats = {&L.gu, &L.down};
    if (!share) {
      LB_TRY(c->alloc(&L.input_norm, size_t(d.H)));
      LB_TRY(c->alloc(&L.post_norm, size_t(d.H)));
      LB_TRY(c->alloc_matrix(L.gu, round_up(d.I, kTileN) + d.I, d.H));
      LB_TRY(c->alloc_matrix(L.down, d.H, d.I));
    }
    if (L.full) {
      if (!share) {
        LB_TRY(c->alloc_matrix(L.qkv, d.Hq * 2 * d.D + 2 * d.Hkv * d.D, d.H));
        LB_TRY(c->alloc_matrix(L.o, d.H, d.Hq * d.D));
        LB_TRY(c->alloc(&L.q_norm, size_t(d.D)));
        LB_TRY(c->alloc(&L.k_norm, size_t(d.D)));
      }
      mats.push_back(&L.qkv), mats.push_back(&L.o);
    } else {
      if (!share) {
        LB_TRY(c->alloc_matrix(L.in, d.C + d.Vs, d.H));
        LB_TRY(c->alloc_matrix(L.out, d.H, d.Vs));
        LB_TRY(c->alloc(&L.in_a, size_t(d.HV) * d.H));
        LB_TRY(c->alloc(&L.in_b, size_t(d.HV) * d.H));
        LB_TRY(c->alloc(&L.conv, size_t(d.C) * 4));
        LB_TRY(c->alloc(&L.A_log, size_t(d.HV)));
        LB_TRY(c->alloc(&L.dt_bias, size_t(d.HV)));
        LB_TRY(c->alloc(&L.lin_norm, size_t(d.Dv)));
      }
      mats.push_back(&L.in), mats.push_back(&L.out);
    }
    for (Fp8Matrix* w : mats) max_plane = std::max(max_plane, size_t(w->splits) * d.rows_alloc * w->N_pad);
  }
  biggest = std::max(biggest, size_t(2) * d.I * d.H);
  c->upload_floats = share ? 0 : std::min(biggest, size_t(64) << 20);  // 256 MB of staging; larger tensors go in row bands (a sibling takes no uploads)
  if (!share) LB_TRY(c->alloc(&c->upload, c->upload_floats, false));

  // ---- activations
  LB_TRY(c->alloc(&c->h, size_t(d.rows_alloc) * d.H));
  LB_TRY(c->alloc(&c->xn, size_t(d.rows_alloc) * d.H));
  LB_TRY(c->alloc(&c->core, size_t(d.rows_alloc) * d.Vs));
  LB_TRY(c->alloc(&c->qh, size_t(d.rows_alloc) * d.Hq * d.D));
  LB_TRY(c->alloc_acts(c->xq_h, d.H));
  LB_TRY(c->alloc_acts(c->xq_v, d.Vs));
  LB_TRY(c->alloc_acts(c->xq_a, d.Hq * d.D));
  LB_TRY(c->alloc_acts(c->xq_i, d.I));
  c->plane_floats = max_plane;
  LB_TRY(c->alloc(&c->planes[0], max_plane));
  LB_TRY(c->alloc(&c->planes[1], max_plane));
  LB_TRY(c->alloc(&c->pre, size_t(d.n_gdn) * d.rows_alloc * d.C));
  LB_TRY(c->alloc(&c->post, size_t(d.n_gdn) * d.rows_alloc * d.C));
  LB_TRY(c->alloc(&c->g, size_t(d.n_gdn) * d.rows_alloc * d.HV));
  LB_TRY(c->alloc(&c->beta, size_t(d.n_gdn) * d.rows_alloc * d.HV));
  // Chunk slots of the flash-decoding partials: every mapped position in chunks of kAttnChunk plus, per sequence, one
  // partly filled chunk and the in-flight chunk; per kv head.  A step on the short chunks (attn_chunk_keys) has at most
  // one slot per CTA of the attention grid.
  // (pages shared between sessions let a batch's contexts add up to more than the pool holds: options.attn_positions)
  const size_t pool_positions = std::max(size_t(d.pool_pages) * d.page_tokens, size_t(std::max(opt->attn_positions, 0)));
  c->chunk_slots = std::max(int((pool_positions / kAttnChunk + size_t(2) * d.max_seqs) * d.Hkv), 2 * c->sm_count);
  const size_t rmax = size_t(kTreeRows) * (d.Hq / d.Hkv);
  LB_TRY(c->alloc(&c->part_o, size_t(c->chunk_slots) * rmax * d.D, false));
  LB_TRY(c->alloc(&c->part_ml, size_t(c->chunk_slots) * rmax * 2, false));
  c->head_ep.rows_alloc = d.rows_alloc;
  LB_TRY(c->alloc(&c->head_ep.tile_val, size_t(c->head.N_pad / kTileN) * d.rows_alloc));
  LB_TRY(c->alloc(&c->head_ep.tile_idx, size_t(c->head.N_pad / kTileN) * d.rows_alloc));
  if (opt->debug_rows > 0) {
    LB_TRY(c->alloc(&c->logits, size_t(opt->debug_rows) * d.V));
    LB_TRY(c->alloc(&c->taps, size_t(cfg->layers + 1) * opt->debug_rows * d.H));
  }
  if (const char* tl = std::getenv("LING_B200_TIMELINE"); tl && tl[0] == '1') {
    LB_TRY(c->alloc(&c->timeline, size_t(4) * ling_b200_ctx::kTimelineLaunches));
    LB_TRY(kernels_norm_stamps(c->timeline + 4 * size_t(ling_b200_ctx::kTimelineLaunches - 24)));
  }
  c->flush_floats = size_t(192) << 18;  // 192 MiB: more than the 126 MB L2
  LB_TRY(c->alloc(&c->flush, c->flush_floats, false));
  if (opt->chain) {
    LB_TRY(chain_init());
    c->chain_words = size_t(2 * cfg->layers + 2) * kChainCounterWords;
    LB_TRY(c->alloc(&c->chain_counters, c->chain_words));
    LB_TRY(c->alloc(&c->chain_ssq, size_t(kChainRows) * 8 * 8));
  }

  // ---- sessions
  const size_t kv_slots = size_t(d.n_attn) * 2 * d.Hkv * (d.pool_pages + 1) * d.page_tokens;
  c->state_layer = size_t(d.HV) * d.Dk * d.Dv;
  c->conv_layer = size_t(d.C) * 3;
  LB_TRY(c->alloc(&c->swiglu_tickets, size_t(d.rows_alloc / 32 + 1) * (round_up(d.I, kTileN) / kTileN)));
  if (share) {
    c->kv = share->kv, c->gdn_state = share->gdn_state, c->conv_state = share->conv_state;
  } else {
    LB_TRY(c->alloc(&c->kv.codes, kv_slots * d.D));
    LB_TRY(c->alloc(&c->kv.scales, kv_slots));
    LB_TRY(c->alloc(&c->kv.tables, size_t(opt->sessions) * d.max_pages));
    LB_TRY(c->alloc(&c->gdn_state, size_t(opt->sessions) * d.n_gdn * c->state_layer));
    LB_TRY(c->alloc(&c->conv_state, size_t(opt->sessions) * d.n_gdn * c->conv_layer));
  }

  // ---- the step's descriptors: one host-written block
  const size_t ms = size_t(d.max_seqs);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t at = off;
    off += (bytes + 15) / 16 * 16;
    return at;
  };
  const size_t o_n = take(sizeof(int)), o_seqs = take(ms * sizeof(SeqDev)), o_par = take(ms * kTreeRows * 4);
  const size_t o_tok = take(ms * kTreeRows * 4), o_force = take(ms * kTreeRows * 4);
  c->stage_bytes = off;
  LB_TRY(c->alloc(&c->stage_dev, c->stage_bytes));
  LB_CUDA(cudaMallocHost(reinterpret_cast<void**>(&c->stage_host), c->stage_bytes));
  std::memset(c->stage_host, 0, c->stage_bytes);
  LB_CUDA(cudaMallocHost(reinterpret_cast<void**>(&c->results_host), ms * sizeof(ling_b200_seq_result)));
  LB_CUDA(cudaMallocHost(reinterpret_cast<void**>(&c->err_host), sizeof(int)));
  StepBuffers& sb = c->sb;
  sb.n_seqs = reinterpret_cast<int*>(c->stage_dev + o_n);
  sb.seqs = reinterpret_cast<SeqDev*>(c->stage_dev + o_seqs);
  sb.in_parent = reinterpret_cast<int*>(c->stage_dev + o_par);
  sb.in_token = reinterpret_cast<int*>(c->stage_dev + o_tok);
  sb.in_force = reinterpret_cast<int*>(c->stage_dev + o_force);
  LB_TRY(c->alloc(&sb.row0, ms + 1));
  LB_TRY(c->alloc(&sb.n_rows_total, 1));
  LB_TRY(c->alloc(&sb.token, size_t(d.rows_alloc)));
  LB_TRY(c->alloc(&sb.seq_of, size_t(d.rows_alloc)));
  LB_TRY(c->alloc(&sb.local, size_t(d.rows_alloc)));
  LB_TRY(c->alloc(&sb.depth, size_t(d.rows_alloc)));
  LB_TRY(c->alloc(&sb.rope_pos, size_t(d.rows_alloc)));
  LB_TRY(c->alloc(&sb.cache_slot, size_t(d.rows_alloc)));
  LB_TRY(c->alloc(&sb.anc, size_t(d.rows_alloc)));
  LB_TRY(c->alloc(&sb.trees, ms));
  LB_TRY(c->alloc(&sb.gdn_aux, ms));
  LB_TRY(c->alloc(&sb.argmax_id, size_t(d.rows_alloc)));
  LB_TRY(c->alloc(&sb.argmax_val, size_t(d.rows_alloc)));
  LB_TRY(c->alloc(&sb.results, ms));
  LB_TRY(c->alloc(&sb.err, 1));
  LB_CUDA(cudaDeviceSynchronize());
  return LING_B200_OK;
}

int ling_b200_create(const ling_b200_model_config* cfg, const ling_b200_options* opt, ling_b200_ctx** out) {
  return create_impl(cfg, opt, nullptr, out);
}

// A second set of step buffers on a context's model and sessions: what runs beside that context's verify steps on the same
// GPU (a prefill chunk's attention layers) without touching its staged step.  The sibling shares the parent's weights, KV
// pool, page tables and state slots -- it must be destroyed before the parent, and takes no weight uploads.
int ling_b200_create_sibling(const ling_b200_ctx* parent, int max_seqs, int max_rows, ling_b200_ctx** out) {
  if (!parent || !out) {
    set_error("create_sibling: null argument");
    return LING_B200_ERR_ARG;
  }
  ling_b200_options opt = parent->opt;
  opt.max_seqs = max_seqs, opt.max_rows = max_rows, opt.debug_rows = 0;
  return create_impl(&parent->cfg, &opt, parent, out);
}

void ling_b200_destroy(ling_b200_ctx* c) {
  if (!c) return;
  cudaSetDevice(c->opt.device);
  if (c->stream) cudaStreamSynchronize(c->stream);
  if (c->timeline) kernels_norm_stamps(nullptr);
  for (auto& kvp : c->graphs) cudaGraphExecDestroy(kvp.second);
  for (void* p : c->owned) cudaFree(p);
  if (c->stage_host) cudaFreeHost(c->stage_host);
  if (c->results_host) cudaFreeHost(c->results_host);
  if (c->err_host) cudaFreeHost(c->err_host);
  if (c->ev0) cudaEventDestroy(c->ev0);
  if (c->ev1) cudaEventDestroy(c->ev1);
  if (c->side) cudaStreamDestroy(c->side);
  if (c->ev_fork) cudaEventDestroy(c->ev_fork);
  if (c->ev_join) cudaEventDestroy(c->ev_join);
  if (c->stream) cudaStreamDestroy(c->stream);
  delete c;
}

size_t ling_b200_weight_bytes(const ling_b200_ctx* c) {
  if (!c) return 0;
  const ModelDims& d = c->d;
  size_t b = c->head.bytes() + size_t(d.H) * 2;
  for (const LayerW& L : c->layers) {
    b += L.gu.bytes() + L.down.bytes() + size_t(2) * d.H * 2;
    if (L.full) b += L.qkv.bytes() + L.o.bytes() + size_t(2) * d.D * 2;
    else b += L.in.bytes() + L.out.bytes() + (size_t(2) * d.HV * d.H + size_t(d.C) * 4 + 2 * d.HV + d.Dv) * 2;
  }
  return b;
}

int ling_b200_set_tensor(ling_b200_ctx* c, int layer, int tensor, const float* host, int rows, int cols) {
  LB_TRY(check_ctx(c));
  if (c->sibling) {
    set_error("a sibling context takes no weights and owns no state arena: use its parent");
    return LING_B200_ERR_ARG;
  }
  if (!host || rows < 1 || cols < 1) {
    set_error("set_tensor: bad argument");
    return LING_B200_ERR_ARG;
  }
  const MatSlot m = mat_slot(c, layer, tensor);
  if (m.w) {
    if (rows != m.rows || cols != m.cols) {
      set_error("set_tensor: shape mismatch");
      return LING_B200_ERR_ARG;
    }
    const int band = int(std::max<size_t>(1, c->upload_floats / size_t(cols)));
    for (int r = 0; r < rows; r += band) {
      const int nr = std::min(band, rows - r);
      LB_CUDA(cudaMemcpyAsync(c->upload, host + size_t(r) * cols, size_t(nr) * cols * 4, cudaMemcpyHostToDevice, c->stream));
      LB_TRY(quant_weight_launch(c->upload, 0, 0.f, 0, m.w->codes, m.w->scales, m.row_off + r, nr, cols, m.w->N_pad, m.w->K_pad,
                                 c->stream));
      LB_TRY(finish(c));
    }
    return LING_B200_OK;
  }
  const VecSlot v = vec_slot(c, layer, tensor);
  if (!v.p || size_t(rows) * cols != v.n) {
    set_error("set_tensor: unknown tensor or shape mismatch");
    return LING_B200_ERR_ARG;
  }
  for (size_t at = 0; at < v.n; at += c->upload_floats) {
    const size_t n = std::min(c->upload_floats, v.n - at);
    LB_CUDA(cudaMemcpyAsync(c->upload, host + at, n * 4, cudaMemcpyHostToDevice, c->stream));
    LB_TRY(fill_bf16_launch(c->upload, 0, 0.f, 0.f, 0, v.p + at, n, c->stream));
    LB_TRY(finish(c));
  }
  return LING_B200_OK;
}

int ling_b200_synth_weights(ling_b200_ctx* c, uint64_t seed) {
  LB_TRY(check_ctx(c));
  if (c->sibling) {
    set_error("a sibling context takes no weights and owns no state arena: use its parent");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(synth_tensor(c, seed, -1, LING_B200_T_EMBED));
  LB_TRY(synth_tensor(c, seed, -1, LING_B200_T_FINAL_NORM));
  LB_TRY(synth_tensor(c, seed, -1, LING_B200_T_LM_HEAD));
  for (int l = 0; l < c->cfg.layers; ++l) {
    if (c->layers[l].full) {
      for (int t : kLayerTensorsFull) LB_TRY(synth_tensor(c, seed, l, t));
    } else {
      for (int t : kLayerTensorsGdn) LB_TRY(synth_tensor(c, seed, l, t));
    }
  }
  return finish(c);
}

int ling_b200_get_matrix(ling_b200_ctx* c, int layer, int tensor, uint8_t* codes, float* scales, int rows, int cols) {
  LB_TRY(check_ctx(c));
  const MatSlot m = mat_slot(c, layer, tensor);
  if (!m.w || rows != m.rows || cols != m.cols) {
    set_error("get_matrix: unknown matrix or shape mismatch");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(finish(c));
  const Fp8Matrix& w = *m.w;
  if (codes)
    LB_CUDA(cudaMemcpy2D(codes, size_t(cols), w.codes + size_t(m.row_off) * w.K_pad, size_t(w.K_pad), size_t(cols), size_t(rows),
                         cudaMemcpyDeviceToHost));
  if (scales) {
    const int KB = ceil_div(cols, 128);
    std::vector<float> tmp(size_t(KB) * rows);
    LB_CUDA(cudaMemcpy2D(tmp.data(), size_t(rows) * 4, w.scales + m.row_off, size_t(w.N_pad) * 4, size_t(rows) * 4, size_t(KB),
                         cudaMemcpyDeviceToHost));
    for (int r = 0; r < rows; ++r)
      for (int b = 0; b < KB; ++b) scales[size_t(r) * KB + b] = tmp[size_t(b) * rows + r];
  }
  return LING_B200_OK;
}

// ------------------------------------------------------------------------------------------------ sessions
int ling_b200_kv_table_set(ling_b200_ctx* c, int slot, const int* idx, const int* page, int n) {
  LB_TRY(check_ctx(c));
  if (slot < 0 || slot >= c->opt.sessions || n < 0) {
    set_error("kv_table_set: bad slot");
    return LING_B200_ERR_ARG;
  }
  for (int i = 0; i < n; ++i)
    if (idx[i] < 0 || idx[i] >= c->d.max_pages || page[i] < 0 || page[i] > c->d.pool_pages) {
      set_error("kv_table_set: entry out of range");
      return LING_B200_ERR_ARG;
    }
  // Ordered on the step stream before the next step reads the table; runs of consecutive indices go as one copy.
  for (int i = 0; i < n;) {
    int j = i + 1;
    while (j < n && idx[j] == idx[j - 1] + 1) ++j;
    LB_CUDA(cudaMemcpyAsync(c->kv.tables + size_t(slot) * c->d.max_pages + idx[i], page + i, size_t(j - i) * 4,
                            cudaMemcpyHostToDevice, c->stream));
    i = j;
  }
  return finish(c);  // the caller's arrays may be reused at once
}

int ling_b200_kv_pages_copy(ling_b200_ctx* c, const int* src, const int* dst, int n) {
  LB_TRY(check_ctx(c));
  for (int i = 0; i < n; ++i) {
    if (src[i] < 1 || src[i] > c->d.pool_pages || dst[i] < 1 || dst[i] > c->d.pool_pages) {
      set_error("kv_pages_copy: page out of range");
      return LING_B200_ERR_ARG;
    }
    LB_TRY(kv_page_copy_launch(c->d, c->kv, src[i], dst[i], c->stream));
  }
  return LING_B200_OK;
}

static int check_positions(ling_b200_ctx* c, int slot, int al, int from, int n) {
  if (slot < 0 || slot >= c->opt.sessions || al < 0 || al >= c->d.n_attn || from < 0 || n < 0 ||
      from + n > c->d.max_pages * c->d.page_tokens) {
    set_error("kv: slot, layer or positions out of range");
    return LING_B200_ERR_ARG;
  }
  return LING_B200_OK;
}

static int read_err(ling_b200_ctx* c) {
  LB_CUDA(cudaMemcpyAsync(c->err_host, c->sb.err, sizeof(int), cudaMemcpyDeviceToHost, c->stream));
  LB_TRY(finish(c));
  if (*c->err_host != 0) {
    set_error("device error word = " + std::to_string(*c->err_host) +
              " (1-4: a GEMM wait ran out; 5: unmapped page; 6: bad tree; 7: token out of range)");
    LB_CUDA(cudaMemsetAsync(c->sb.err, 0, sizeof(int), c->stream));
    return LING_B200_ERR_DEVICE_FLAG;
  }
  return LING_B200_OK;
}

int ling_b200_kv_write(ling_b200_ctx* c, int slot, int al, int from, int n, const float* k, const float* v) {
  LB_TRY(check_ctx(c));
  LB_TRY(check_positions(c, slot, al, from, n));
  const ModelDims& d = c->d;
  const size_t per = size_t(d.Hkv) * d.D;
  const int band = int(std::max<size_t>(1, c->upload_floats / (2 * per)));
  for (int i = 0; i < n; i += band) {
    const int nb = std::min(band, n - i);
    float* dk = c->upload;
    float* dv = c->upload + size_t(nb) * per;
    LB_CUDA(cudaMemcpyAsync(dk, k + size_t(i) * per, size_t(nb) * per * 4, cudaMemcpyHostToDevice, c->stream));
    LB_CUDA(cudaMemcpyAsync(dv, v + size_t(i) * per, size_t(nb) * per * 4, cudaMemcpyHostToDevice, c->stream));
    LB_TRY(kv_write_launch(dk, dv, 0, 0, 0, d, al, slot, from + i, nb, c->kv, c->sb.err, c->stream));
    LB_TRY(finish(c));
  }
  return read_err(c);
}

int ling_b200_synth_kv_range(ling_b200_ctx* c, int slot, int from, int n, uint64_t seed) {
  LB_TRY(check_ctx(c));
  const ModelDims& d = c->d;
  if (d.n_attn == 0) return LING_B200_OK;
  LB_TRY(check_positions(c, slot, 0, from, n));
  for (int al = 0; al < d.n_attn; ++al) {
    const uint64_t base = kStreamKv + (uint64_t(slot) * d.n_attn + al) * 2;
    LB_TRY(kv_write_launch(nullptr, nullptr, stream_key(seed, base), stream_key(seed, base + 1), 1, d, al, slot, from, n, c->kv,
                           c->sb.err, c->stream));
  }
  return read_err(c);
}
int ling_b200_synth_kv(ling_b200_ctx* c, int slot, int n, uint64_t seed) { return ling_b200_synth_kv_range(c, slot, 0, n, seed); }

int ling_b200_kv_read(ling_b200_ctx* c, int slot, int al, int from, int n, float* k, float* v, uint8_t* kcodes, float* kscales,
                      uint8_t* vcodes, float* vscales) {
  LB_TRY(check_ctx(c));
  LB_TRY(check_positions(c, slot, al, from, n));
  LB_TRY(finish(c));
  const ModelDims& d = c->d;
  std::vector<int> table(d.max_pages);
  LB_CUDA(cudaMemcpy(table.data(), c->kv.tables + size_t(slot) * d.max_pages, table.size() * 4, cudaMemcpyDeviceToHost));
  std::vector<uint8_t> codes(d.D);
  for (int i = 0; i < n; ++i)
    for (int hh = 0; hh < d.Hkv; ++hh)
      for (int kvi = 0; kvi < 2; ++kvi) {
        const int pos = from + i;
        const int page = table[pos / d.page_tokens], tok = pos % d.page_tokens;
        float sc;
        // a K position's bytes are contiguous; a V position's bytes are page_tokens apart (the V page is [D][token])
        LB_CUDA(cudaMemcpy2D(codes.data(), 1, c->kv.codes + kv_code_index(d, al, kvi, hh, page, tok, 0), kvi ? size_t(d.page_tokens) : 1, 1,
                             size_t(d.D), cudaMemcpyDeviceToHost));
        LB_CUDA(cudaMemcpy(&sc, c->kv.scales + kv_slot_index(d, al, kvi, hh, page, tok), 4, cudaMemcpyDeviceToHost));
        const size_t o = size_t(i) * d.Hkv + hh;
        float* f = kvi ? v : k;
        uint8_t* cc = kvi ? vcodes : kcodes;
        float* ss = kvi ? vscales : kscales;
        if (ss) ss[o] = sc;
        for (int dd = 0; dd < d.D; ++dd) {
          if (cc) cc[o * d.D + dd] = codes[dd];
          if (f) {
            const int code = codes[dd], e = (code >> 3) & 15, mm = code & 7;
            float val = e == 0 ? std::ldexp(float(mm), -9) : std::ldexp(1.f + mm / 8.f, e - 7);
            if (e == 15 && mm == 7) val = NAN;
            f[o * d.D + dd] = (code & 0x80 ? -val : val) * sc;
          }
        }
      }
  return LING_B200_OK;
}

int ling_b200_state_write(ling_b200_ctx* c, int slot, int gl, const float* state, const float* conv) {
  LB_TRY(check_ctx(c));
  if (slot < 0 || slot >= c->opt.sessions || gl < 0 || gl >= c->d.n_gdn) {
    set_error("state: slot or layer out of range");
    return LING_B200_ERR_ARG;
  }
  const size_t at = size_t(slot) * c->d.n_gdn + gl;
  if (state) LB_CUDA(cudaMemcpyAsync(c->gdn_state + at * c->state_layer, state, c->state_layer * 4, cudaMemcpyHostToDevice, c->stream));
  if (conv) LB_CUDA(cudaMemcpyAsync(c->conv_state + at * c->conv_layer, conv, c->conv_layer * 4, cudaMemcpyHostToDevice, c->stream));
  return finish(c);
}
int ling_b200_state_read(ling_b200_ctx* c, int slot, int gl, float* state, float* conv) {
  LB_TRY(check_ctx(c));
  if (slot < 0 || slot >= c->opt.sessions || gl < 0 || gl >= c->d.n_gdn) {
    set_error("state: slot or layer out of range");
    return LING_B200_ERR_ARG;
  }
  const size_t at = size_t(slot) * c->d.n_gdn + gl;
  if (state) LB_CUDA(cudaMemcpyAsync(state, c->gdn_state + at * c->state_layer, c->state_layer * 4, cudaMemcpyDeviceToHost, c->stream));
  if (conv) LB_CUDA(cudaMemcpyAsync(conv, c->conv_state + at * c->conv_layer, c->conv_layer * 4, cudaMemcpyDeviceToHost, c->stream));
  return finish(c);
}
int ling_b200_synth_state(ling_b200_ctx* c, int slot, uint64_t seed) {
  LB_TRY(check_ctx(c));
  if (slot < 0 || slot >= c->opt.sessions) {
    set_error("state: slot out of range");
    return LING_B200_ERR_ARG;
  }
  for (int gl = 0; gl < c->d.n_gdn; ++gl) {
    const size_t at = size_t(slot) * c->d.n_gdn + gl;
    LB_TRY(fill_f32_launch(stream_key(seed, kStreamState + uint64_t(slot) * c->d.n_gdn + gl), 0.1f,
                           c->gdn_state + at * c->state_layer, c->state_layer, c->stream));
    LB_TRY(fill_f32_launch(stream_key(seed, kStreamConv + uint64_t(slot) * c->d.n_gdn + gl), 1.f,
                           c->conv_state + at * c->conv_layer, c->conv_layer, c->stream));
  }
  return finish(c);
}
// One session's recurrent state as the prefix KV store and the checkpoints keep it (Engine::copy_slot, engine.cpp:1125-1137):
// every DeltaNet layer's state, then every conv window.  A slot's layers are consecutive, so each half is one run.
size_t ling_b200_state_bytes(const ling_b200_ctx* c) {
  return c ? size_t(c->d.n_gdn) * (c->state_layer + c->conv_layer) * sizeof(float) : 0;
}
int ling_b200_state_arena_reserve(ling_b200_ctx* c, size_t bytes) {
  LB_TRY(check_ctx(c));
  if (c->sibling) {
    set_error("a sibling context takes no weights and owns no state arena: use its parent");
    return LING_B200_ERR_ARG;
  }
  if (c->state_arena || bytes == 0) {
    set_error("state_arena_reserve: already reserved, or an empty arena");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(c->alloc(&c->state_arena, bytes, false));
  c->state_arena_bytes = bytes;
  return LING_B200_OK;
}
static int state_move(ling_b200_ctx* c, int slot, size_t offset, bool save) {
  LB_TRY(check_ctx(c));
  const size_t gdn = size_t(c->d.n_gdn) * c->state_layer * sizeof(float), conv = size_t(c->d.n_gdn) * c->conv_layer * sizeof(float);
  if (slot < 0 || slot >= c->opt.sessions || !c->state_arena || offset % 16 != 0 || offset > c->state_arena_bytes ||
      gdn + conv > c->state_arena_bytes - offset) {
    set_error("state save/restore: slot out of range, no arena, or a range outside it");
    return LING_B200_ERR_ARG;
  }
  float* s_gdn = c->gdn_state + size_t(slot) * c->d.n_gdn * c->state_layer;
  float* s_conv = c->conv_state + size_t(slot) * c->d.n_gdn * c->conv_layer;
  uint8_t* a = c->state_arena + offset;
  if (save) {
    LB_CUDA(cudaMemcpyAsync(a, s_gdn, gdn, cudaMemcpyDeviceToDevice, c->stream));
    LB_CUDA(cudaMemcpyAsync(a + gdn, s_conv, conv, cudaMemcpyDeviceToDevice, c->stream));
  } else {
    LB_CUDA(cudaMemcpyAsync(s_gdn, a, gdn, cudaMemcpyDeviceToDevice, c->stream));
    LB_CUDA(cudaMemcpyAsync(s_conv, a + gdn, conv, cudaMemcpyDeviceToDevice, c->stream));
  }
  return LING_B200_OK;
}
int ling_b200_state_save(ling_b200_ctx* c, int slot, size_t offset) { return state_move(c, slot, offset, true); }
int ling_b200_state_restore(ling_b200_ctx* c, int slot, size_t offset) { return state_move(c, slot, offset, false); }
// Engine::reset_state (engine.cpp:944-952): a prompt that resumes from nothing starts from zero states and windows.
int ling_b200_state_reset(ling_b200_ctx* c, int slot) {
  LB_TRY(check_ctx(c));
  if (slot < 0 || slot >= c->opt.sessions) {
    set_error("state_reset: slot out of range");
    return LING_B200_ERR_ARG;
  }
  LB_CUDA(cudaMemsetAsync(c->gdn_state + size_t(slot) * c->d.n_gdn * c->state_layer, 0, size_t(c->d.n_gdn) * c->state_layer * sizeof(float), c->stream));
  LB_CUDA(cudaMemsetAsync(c->conv_state + size_t(slot) * c->d.n_gdn * c->conv_layer, 0, size_t(c->d.n_gdn) * c->conv_layer * sizeof(float), c->stream));
  return LING_B200_OK;
}
// Engine::state_hash (src/core/engine.cpp:954-971): FNV-1a, byte by byte, each DeltaNet layer's state then its window.
int ling_b200_state_hash(ling_b200_ctx* c, int slot, uint64_t* hash) {
  LB_TRY(check_ctx(c));
  if (slot < 0 || slot >= c->opt.sessions || !hash) {
    set_error("state_hash: bad argument");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(finish(c));
  uint64_t hh = 1469598103934665603ull;
  std::vector<float> buf(std::max(c->state_layer, c->conv_layer));
  for (int gl = 0; gl < c->d.n_gdn; ++gl) {
    const size_t at = size_t(slot) * c->d.n_gdn + gl;
    for (int part = 0; part < 2; ++part) {
      const size_t n = part ? c->conv_layer : c->state_layer;
      LB_CUDA(cudaMemcpy(buf.data(), part ? c->conv_state + at * c->conv_layer : c->gdn_state + at * c->state_layer, n * 4,
                         cudaMemcpyDeviceToHost));
      const unsigned char* b = reinterpret_cast<const unsigned char*>(buf.data());
      for (size_t i = 0; i < n * 4; ++i) hh = (hh ^ b[i]) * 1099511628211ull;
    }
  }
  *hash = hh;
  return LING_B200_OK;
}

// ------------------------------------------------------------------------------------------------ the step
// Attention partial slots: what a sequence with `pos` cached positions takes in a step, and what the context holds.
int ling_b200_attn_slot_need(const ling_b200_ctx* c, int pos) {
  if (!c || c->d.n_attn == 0) return 0;
  return ((std::max(pos, 0) + kAttnChunk - 1) / kAttnChunk + 1) * c->d.Hkv;
}
int ling_b200_attn_slot_capacity(const ling_b200_ctx* c) { return c ? c->chunk_slots : 0; }
static int stage_impl(ling_b200_ctx* c, const ling_b200_seq_step* seqs, int n_seqs, int flags, bool same_slot_ok) {
  LB_TRY(check_ctx(c));
  const ModelDims& d = c->d;
  if (!seqs || n_seqs < 1 || n_seqs > d.max_seqs) {
    set_error("step: sequence count out of range");
    return LING_B200_ERR_ARG;
  }
  if ((flags & (LING_B200_STEP_KEEP_LOGITS | LING_B200_STEP_KEEP_TAPS)) && c->opt.debug_rows <= 0) {
    set_error("step: logits/taps need options.debug_rows > 0");
    return LING_B200_ERR_ARG;
  }
  int rows = 0;
  for (int s = 0; s < n_seqs; ++s) {
    const ling_b200_seq_step& q = seqs[s];
    if (q.slot < 0 || q.slot >= c->opt.sessions || q.n_rows < 1 || q.n_rows > kTreeRows || q.pos < 0 || !q.tokens || !q.parent ||
        q.chain < 0 || q.pos + q.n_rows > d.max_pages * d.page_tokens) {
      set_error("step: bad sequence entry");
      return LING_B200_ERR_ARG;
    }
    for (int t = 0; t < s && !same_slot_ok; ++t)
      if (seqs[t].slot == q.slot) {
        set_error("step: a session twice");  // speculate_batch's rule (src/core/speculate.cpp:1107-1108)
        return LING_B200_ERR_ARG;
      }
    rows += q.n_rows;
  }
  if (rows > c->opt.max_rows) {
    set_error("step: more rows than options.max_rows");
    return LING_B200_ERR_ARG;
  }
  if ((flags & (LING_B200_STEP_KEEP_LOGITS | LING_B200_STEP_KEEP_TAPS)) && rows > c->opt.debug_rows) {
    set_error("step: more rows than options.debug_rows");
    return LING_B200_ERR_ARG;
  }
  uint8_t* hb = c->stage_host;
  const uint8_t* db = c->stage_dev;
  auto host_of = [&](const void* dev) { return hb + (reinterpret_cast<const uint8_t*>(dev) - db); };
  *reinterpret_cast<int*>(host_of(c->sb.n_seqs)) = n_seqs;
  SeqDev* hs = reinterpret_cast<SeqDev*>(host_of(c->sb.seqs));
  int* hp = reinterpret_cast<int*>(host_of(c->sb.in_parent));
  int* ht = reinterpret_cast<int*>(host_of(c->sb.in_token));
  int* hf = reinterpret_cast<int*>(host_of(c->sb.in_force));
  for (int s = 0; s < n_seqs; ++s) {
    const ling_b200_seq_step& q = seqs[s];
    hs[s] = SeqDev{q.slot, q.pos, q.rope_delta, q.n_rows, q.chain, q.force_argmax ? 1 : 0};
    for (int r = 0; r < kTreeRows; ++r) {
      hp[s * kTreeRows + r] = r < q.n_rows ? (r == 0 ? -1 : q.parent[r]) : 0;
      ht[s * kTreeRows + r] = r < q.n_rows ? q.tokens[r] : 0;
      hf[s * kTreeRows + r] = (r < q.n_rows && q.force_argmax) ? q.force_argmax[r] : 0;
    }
  }
  c->staged_seqs = n_seqs, c->staged_rows = rows, c->staged_flags = flags;
  c->staged_slots = 0;
  for (int i = 0; i < n_seqs; ++i) c->staged_slots += long(ling_b200_attn_slot_need(c, seqs[i].pos));
  LB_CUDA(cudaMemcpyAsync(c->stage_dev, c->stage_host, c->stage_bytes, cudaMemcpyHostToDevice, c->stream));
  return LING_B200_OK;
}

int ling_b200_step_stage(ling_b200_ctx* c, const ling_b200_seq_step* seqs, int n_seqs, int flags) {
  return stage_impl(c, seqs, n_seqs, flags, false);
}

// The flash-decoding partials have a slot per (kv head, chunk of a sequence's context) (chunk_slots): a staged step whose
// contexts need more is refused here, before anything that runs the attention kernels is launched.
static int check_attn_slots(ling_b200_ctx* c) {
  if (c->d.n_attn > 0 && c->staged_slots > c->chunk_slots) {
    set_error("step: the batch's contexts need " + std::to_string(c->staged_slots) + " attention partial slots, the context has " +
              std::to_string(c->chunk_slots) + " (sized for the pool's positions or options.attn_positions)");
    return LING_B200_ERR_ARG;
  }
  return LING_B200_OK;
}

int ling_b200_step_launch(ling_b200_ctx* c) {
  LB_TRY(check_ctx(c));
  if (c->staged_seqs < 1) {
    set_error("step: nothing staged");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(check_attn_slots(c));
  const int rows = row_class(c->staged_rows), flags = c->staged_flags;
  c->last_rows = c->staged_rows, c->last_seqs = c->staged_seqs, c->last_flags = flags;
  if (!c->opt.use_graph) return enqueue_step(c, rows, flags);
  const auto key = std::make_pair(rows, flags);
  auto it = c->graphs.find(key);
  if (it == c->graphs.end()) {
    cudaGraph_t graph = nullptr;
    LB_CUDA(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
    const int rc = enqueue_step(c, rows, flags);
    const cudaError_t e = cudaStreamEndCapture(c->stream, &graph);
    if (rc != LING_B200_OK) {
      if (graph) cudaGraphDestroy(graph);
      return rc;
    }
    LB_CUDA(e);
    cudaGraphExec_t exec = nullptr;
    const cudaError_t ie = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    LB_CUDA(ie);
    it = c->graphs.emplace(key, exec).first;
  }
  LB_CUDA(cudaGraphLaunch(it->second, c->stream));
  return LING_B200_OK;
}

int ling_b200_step_fetch(ling_b200_ctx* c, ling_b200_seq_result* results) {
  LB_TRY(check_ctx(c));
  if (c->last_seqs < 1) {
    set_error("step: nothing launched");
    return LING_B200_ERR_ARG;
  }
  LB_CUDA(cudaMemcpyAsync(c->results_host, c->sb.results, size_t(c->last_seqs) * sizeof(ling_b200_seq_result),
                          cudaMemcpyDeviceToHost, c->stream));
  LB_TRY(read_err(c));
  if (results) std::memcpy(results, c->results_host, size_t(c->last_seqs) * sizeof(ling_b200_seq_result));
  return LING_B200_OK;
}

int ling_b200_verify_step(ling_b200_ctx* c, const ling_b200_seq_step* seqs, int n_seqs, int flags, ling_b200_seq_result* results) {
  LB_TRY(ling_b200_step_stage(c, seqs, n_seqs, flags));
  LB_TRY(ling_b200_step_launch(c));
  return ling_b200_step_fetch(c, results);
}

int ling_b200_step_launch_count(ling_b200_ctx* c) { return c ? c->launches_per_step : 0; }

// Debugging aid (needs LING_B200_TIMELINE=1 when the context is created): clears the stamps, replays the staged step once
// and returns, per GEMM launch in order, {first CTA start, first and last producer past the dependency wait, last CTA end}
// in nanoseconds of the GPU's global timer.  Returns the number of launches written.
int ling_b200_gemm_timeline(ling_b200_ctx* c, unsigned long long* out, int max_launches) {
  if (!c || !c->timeline || !out) return 0;
  if (finish(c) != LING_B200_OK) return 0;
  std::vector<unsigned long long> init(size_t(4) * ling_b200_ctx::kTimelineLaunches);
  for (size_t i = 0; i < init.size(); i += 4) init[i] = init[i + 1] = ~0ull, init[i + 2] = init[i + 3] = 0;
  if (cudaMemcpy(c->timeline, init.data(), init.size() * 8, cudaMemcpyHostToDevice) != cudaSuccess) return 0;
  if (ling_b200_step_launch(c) != LING_B200_OK || finish(c) != LING_B200_OK) return 0;
  const int n = max_launches >= ling_b200_ctx::kTimelineLaunches
                    ? ling_b200_ctx::kTimelineLaunches  // everything, the DeltaNet kernel's phase stamps in the last four slots included
                    : std::min(max_launches, c->timeline_next > 0 ? c->timeline_next : 4 * c->cfg.layers + 1);
  if (cudaMemcpy(out, c->timeline, size_t(n) * 32, cudaMemcpyDeviceToHost) != cudaSuccess) return 0;
  return n;
}

int ling_b200_profile_step(ling_b200_ctx* c, float ms[8], int* launches) {
  LB_TRY(check_ctx(c));
  if (c->staged_seqs < 1) {
    set_error("profile: nothing staged");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(check_attn_slots(c));
  LB_TRY(finish(c));
  c->profiling = true;
  c->prof.clear();
  const int rc = enqueue_step(c, row_class(c->staged_rows), c->staged_flags & ~LING_B200_STEP_COMMIT);
  c->profiling = false;
  const int fin = finish(c);
  for (int i = 0; i < 8; ++i) ms[i] = 0.f;
  for (auto& p : c->prof) {
    float t = 0.f;
    if (rc == LING_B200_OK && fin == LING_B200_OK) cudaEventElapsedTime(&t, p.second.first, p.second.second);
    ms[p.first] += t;
    cudaEventDestroy(p.second.first), cudaEventDestroy(p.second.second);
  }
  if (launches) *launches = c->launches_per_step;
  c->prof.clear();
  return rc != LING_B200_OK ? rc : fin;
}

int ling_b200_gemm_chain_ms(ling_b200_ctx* c, int iters, float* ms) {
  LB_TRY(check_ctx(c));
  if (c->staged_seqs < 1 || iters < 1 || !ms) {
    set_error("gemm_chain: nothing staged, or bad argument");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(finish(c));
  const int rows = row_class(c->staged_rows);
  PdlScope pdl(c->opt.pdl != 0);
  int rc = LING_B200_OK;
  auto chain = [&]() -> int {
    for (const LayerW& L : c->layers) {
      LB_TRY(run_gemm(c, L.full ? L.qkv : L.in, c->xq_h, 0, rows));
      LB_TRY(run_gemm(c, L.full ? L.o : L.out, L.full ? c->xq_a : c->xq_v, 1, rows));
      LB_TRY(run_gemm(c, L.gu, c->xq_h, 0, rows));
      LB_TRY(run_gemm(c, L.down, c->xq_i, 1, rows));
    }
    HeadEpilogue ep = c->head_ep;
    ep.store_logits = false;
    return run_gemm(c, c->head, c->xq_h, 0, rows, &ep);
  };
  // captured once and replayed, like the step itself (launching 257 kernels from the host one by one would time the host)
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  if (!cuda_ok(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture")) return LING_B200_ERR_CUDA;
  rc = chain();
  const cudaError_t ce = cudaStreamEndCapture(c->stream, &graph);
  if (rc == LING_B200_OK && !cuda_ok(ce, "cudaStreamEndCapture")) rc = LING_B200_ERR_CUDA;
  if (rc == LING_B200_OK && !cuda_ok(cudaGraphInstantiate(&exec, graph, 0), "cudaGraphInstantiate")) rc = LING_B200_ERR_CUDA;
  if (graph) cudaGraphDestroy(graph);
  float t = 0.f;
  if (rc == LING_B200_OK) {
    cudaGraphLaunch(exec, c->stream);  // warm-up
    cudaEventRecord(c->ev0, c->stream);
    for (int i = 0; i < iters; ++i) cudaGraphLaunch(exec, c->stream);
    cudaEventRecord(c->ev1, c->stream);
    if (!cuda_ok(cudaEventSynchronize(c->ev1), "cudaEventSynchronize") || !cuda_ok(cudaEventElapsedTime(&t, c->ev0, c->ev1), "cudaEventElapsedTime"))
      rc = LING_B200_ERR_CUDA;
  }
  if (exec) cudaGraphExecDestroy(exec);
  LB_TRY(rc);
  *ms = t / iters;
  return read_err(c);
}

int ling_b200_timer_begin(ling_b200_ctx* c) {
  LB_TRY(check_ctx(c));
  LB_CUDA(cudaEventRecord(c->ev0, c->stream));
  return LING_B200_OK;
}
int ling_b200_timer_end(ling_b200_ctx* c, float* ms) {
  LB_TRY(check_ctx(c));
  LB_CUDA(cudaEventRecord(c->ev1, c->stream));
  LB_CUDA(cudaEventSynchronize(c->ev1));
  LB_CUDA(cudaEventElapsedTime(ms, c->ev0, c->ev1));
  return LING_B200_OK;
}
int ling_b200_flush_l2(ling_b200_ctx* c) {
  LB_TRY(check_ctx(c));
  return flush_launch(c->flush, c->flush_floats, c->stream);
}
int ling_b200_sync(ling_b200_ctx* c) {
  LB_TRY(check_ctx(c));
  return finish(c);
}

// One attention layer alone, for parity checks: packs `seqs` on the device, takes q [rows][heads][head_dim] from the host,
// runs the tree attention over the slot's cache (context and in-flight positions as the cache holds them) and returns
// the merged rows before the output gate.
int ling_b200_attention_host(ling_b200_ctx* c, const ling_b200_seq_step* seqs, int n_seqs, int attn_layer, const float* q, float* out) {
  LB_TRY(ling_b200_step_stage(c, seqs, n_seqs, 0));
  const ModelDims& d = c->d;
  if (attn_layer < 0 || attn_layer >= d.n_attn || !q || !out) {
    set_error("attention_host: bad argument");
    return LING_B200_ERR_ARG;
  }
  const int rows = c->staged_rows, cls = row_class(rows);
  const size_t n = size_t(rows) * d.Hq * d.D;
  if (n > c->upload_floats || n > c->plane_floats) {
    set_error("attention_host: too many rows for the staging buffers");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(check_attn_slots(c));
  c->last_rows = rows, c->last_seqs = n_seqs, c->last_flags = 0;
  LB_TRY(pack_launch(c->sb, d, c->stream));
  LB_CUDA(cudaMemcpyAsync(c->upload, q, n * 4, cudaMemcpyHostToDevice, c->stream));
  LB_TRY(f32_to_half_launch(c->upload, c->qh, n, c->stream));
  const bool tc = c->opt.gemm_impl == 0 && attention_tc_supported(d);
  if (tc)
    LB_TRY(attention_tc_launch(c->qh, c->sb, d, attn_layer, c->kv, c->part_o, c->part_ml, c->chunk_slots, c->sm_count, PrefetchPlan(), nullptr, c->stream));
  else
    LB_TRY(attention_launch(c->qh, c->sb, d, attn_layer, c->kv, c->part_o, c->part_ml, c->chunk_slots, c->sm_count * 2, c->stream));
  Planes none;
  none.p = nullptr;
  LB_TRY(attn_combine_launch(c->part_o, c->part_ml, none, c->sb, d, c->qout(c->xq_a), c->planes[0], cls,
                             c->opt.max_context / kAttnChunkShort + 2, tc ? kAttnTcRows : kAttnRowTile,
                             tc ? c->sm_count : c->sm_count * 2, c->chunk_slots, c->stream));
  LB_CUDA(cudaMemcpyAsync(out, c->planes[0], n * 4, cudaMemcpyDeviceToHost, c->stream));
  return read_err(c);
}

// attn_prepare alone, for parity checks: packs `seqs` on the device, takes the q|k|v projection's rows from the host, runs
// the prepare kernel of one attention layer (head norms, rotation at the rows' positions, K and V into the slot's cache
// through its page table) and returns the queries as the attention kernel receives them (FP16, widened to fp32).
int ling_b200_attn_prepare_host(ling_b200_ctx* c, const ling_b200_seq_step* seqs, int n_seqs, int attn_layer, const float* qkv,
                                float* q_out) {
  LB_TRY(ling_b200_step_stage(c, seqs, n_seqs, 0));
  const ModelDims& d = c->d;
  if (attn_layer < 0 || attn_layer >= d.n_attn || !qkv || !q_out) {
    set_error("attn_prepare_host: bad argument");
    return LING_B200_ERR_ARG;
  }
  int layer = -1;
  for (int l = 0; l < c->cfg.layers; ++l)
    if (c->attn_index[l] == attn_layer) layer = l;
  const LayerW& L = c->layers[layer];
  const int rows = c->staged_rows, W = d.Hq * 2 * d.D + 2 * d.Hkv * d.D;
  if (size_t(rows) * W > c->plane_floats) {
    set_error("attn_prepare_host: too many rows for the staging buffers");
    return LING_B200_ERR_ARG;
  }
  c->last_rows = rows, c->last_seqs = n_seqs, c->last_flags = 0;
  PdlScope pdl(c->opt.pdl != 0);
  LB_TRY(pack_launch(c->sb, d, c->stream));
  LB_CUDA(cudaMemcpyAsync(c->planes[0], qkv, size_t(rows) * W * 4, cudaMemcpyHostToDevice, c->stream));
  Planes p;
  p.p = c->planes[0], p.n = 1, p.stride = 0, p.ld = W;
  LB_TRY(attn_prepare_launch(p, c->sb, d, attn_layer, L.q_norm, L.k_norm, c->qh, c->kv, row_class(rows), c->stream));
  const size_t n = size_t(rows) * d.Hq * d.D;
  std::vector<__half> hq(n);
  LB_CUDA(cudaMemcpyAsync(hq.data(), c->qh, n * sizeof(__half), cudaMemcpyDeviceToHost, c->stream));
  LB_TRY(read_err(c));
  for (size_t i = 0; i < n; ++i) q_out[i] = __half2float(hq[i]);
  return LING_B200_OK;
}

// The next pass over a prefill chunk's rows: chains of up to 32 rows of one session at consecutive positions, as many as the
// step's sequences and rows, `row_floats` floats a row in one staging plane, and the attention partials' slots hold.  A
// later chain's context covers the earlier chains' rows: the prepare kernel has written them when the attention kernel starts.
// Returns the rows taken (0: the step's capacity holds no chain).
static int chunk_pass(ling_b200_ctx* c, int slot, int pos, int left, size_t row_floats, const int* zeros, const int* chain,
                      std::vector<ling_b200_seq_step>& seqs) {
  seqs.clear();
  long slots = 0;
  int rows = 0;
  while (rows < left && int(seqs.size()) < c->d.max_seqs) {
    const int n = std::min(kTreeRows, left - rows);
    const long need = ling_b200_attn_slot_need(c, pos + rows);
    if (rows + n > c->opt.max_rows || size_t(rows + n) * row_floats > c->plane_floats || (slots + need > c->chunk_slots && !seqs.empty())) break;
    seqs.push_back(ling_b200_seq_step{slot, pos + rows, 0, n, n - 1, zeros, chain, nullptr});
    slots += need, rows += n;
  }
  return rows;
}
struct ChunkChains {
  std::vector<int> zeros, chain;
  ChunkChains() : zeros(kTreeRows, 0), chain(kTreeRows) {
    for (int i = 0; i < kTreeRows; ++i) chain[i] = i - 1;
  }
};
static int attn_layer_of(const ling_b200_ctx* c, int attn_layer) {
  for (int l = 0; l < c->cfg.layers; ++l)
    if (c->attn_index[l] == attn_layer) return l;
  return -1;
}
// the step's three attention launches over the staged rows: q|k|v planes -> cache and queries -> partials -> merged rows
// (gated; FP8 copy for the o projection in xq_a, fp32 copy in `raw` if given)
static int attention_over_planes(ling_b200_ctx* c, const LayerW& L, int al, const Planes& p, float* raw, int cls) {
  const ModelDims& d = c->d;
  const bool tc = c->opt.gemm_impl == 0 && attention_tc_supported(d);
  {
    Timed t(c, kFamStep);  // (a profile of the chunk layer reads: Step = prepare, Attn = attention, Gdn = combine, Elem = norms)
    LB_TRY(attn_prepare_launch(p, c->sb, d, al, L.q_norm, L.k_norm, c->qh, c->kv, cls, c->stream));
  }
  {
    Timed t(c, kFamAttn);
    if (tc)
      LB_TRY(attention_tc_launch(c->qh, c->sb, d, al, c->kv, c->part_o, c->part_ml, c->chunk_slots, c->sm_count, PrefetchPlan(), nullptr, c->stream));
    else
      LB_TRY(attention_launch(c->qh, c->sb, d, al, c->kv, c->part_o, c->part_ml, c->chunk_slots, c->sm_count * 2, c->stream));
  }
  Timed t(c, kFamGdn);
  return attn_combine_launch(c->part_o, c->part_ml, p, c->sb, d, c->qout(c->xq_a), raw, cls, c->opt.max_context / kAttnChunkShort + 2,
                             tc ? kAttnTcRows : kAttnRowTile, tc ? c->sm_count : c->sm_count * 2, c->chunk_slots, c->stream);
}

// Attention over a prefill chunk: the M rows at positions pos0.. of one session, q|k|v rows in (host, the q|k|v
// projection's layout), gated attention rows out (host, [M][heads][head_dim]); K and V of the rows go to the session's pages.
// The rows pass through the step's own kernels as chains of 32 (the reference runs its prefill attention in slices of
// queries as well, src/core/engine.cpp:1448-1460): correct for any M, not a many-row attention kernel.
int ling_b200_prefill_attention_host(ling_b200_ctx* c, int slot, int attn_layer, int pos0, int M, const float* qkv, float* out) {
  LB_TRY(check_ctx(c));
  const ModelDims& d = c->d;
  if (slot < 0 || slot >= c->opt.sessions || attn_layer < 0 || attn_layer >= d.n_attn || pos0 < 0 || M < 1 || !qkv || !out ||
      pos0 + M > d.max_pages * d.page_tokens) {
    set_error("prefill_attention_host: bad argument");
    return LING_B200_ERR_ARG;
  }
  const LayerW& L = c->layers[attn_layer_of(c, attn_layer)];
  const int W = d.Hq * 2 * d.D + 2 * d.Hkv * d.D, O = d.Hq * d.D;
  struct Unstage {  // the chains staged here are no step to launch: a verify step is staged again afterwards
    ling_b200_ctx* c;
    ~Unstage() { c->staged_seqs = 0, c->staged_rows = 0; }
  } unstage{c};
  ChunkChains cc;
  std::vector<ling_b200_seq_step> seqs;
  PdlScope pdl(c->opt.pdl != 0);
  for (int done = 0; done < M;) {
    const int rows = chunk_pass(c, slot, pos0 + done, M - done, size_t(std::max(W, O)), cc.zeros.data(), cc.chain.data(), seqs);
    if (rows == 0) {
      set_error("prefill_attention_host: the context's step capacity holds no chain of the chunk");
      return LING_B200_ERR_ARG;
    }
    LB_TRY(stage_impl(c, seqs.data(), int(seqs.size()), 0, true));
    LB_TRY(check_attn_slots(c));
    const int cls = row_class(rows);
    c->last_rows = rows, c->last_seqs = int(seqs.size()), c->last_flags = 0;
    LB_TRY(pack_launch(c->sb, d, c->stream));
    LB_CUDA(cudaMemcpyAsync(c->planes[0], qkv + size_t(done) * W, size_t(rows) * W * 4, cudaMemcpyHostToDevice, c->stream));
    Planes p;
    p.p = c->planes[0], p.n = 1, p.stride = 0, p.ld = W;
    LB_TRY(attention_over_planes(c, L, attn_layer, p, c->planes[1], cls));
    LB_CUDA(cudaMemcpyAsync(out + size_t(done) * O, c->planes[1], size_t(rows) * O * 4, cudaMemcpyDeviceToHost, c->stream));
    LB_TRY(read_err(c));  // also: the staging buffers are free for the next pass
    done += rows;
  }
  return LING_B200_OK;
}

// A full-attention layer's whole mixer over a prefill chunk: h [M][hidden] (DEVICE memory, fp32; the residual rows at positions
// pos0.. of one session) += o( gate * attention( prepare( q|k|v( norm(h) ) ) ) ) with the layer's own FP8 projections -- the
// reference keeps the attention projections in FP8 on the prefill path too (src/core/kernels.cuh:1-4).  The rows pass through
// the step's kernels as chains of 32, many chains a launch (see ling_b200_prefill_attention_host); the work is ordered on the
// context's stream and the call returns when it is complete.  A staged verify step is replaced: stage again before the next launch.
int ling_b200_chunk_attention_layer(ling_b200_ctx* c, int slot, int layer, int pos0, int M, float* h) {
  LB_TRY(check_ctx(c));
  const ModelDims& d = c->d;
  if (slot < 0 || slot >= c->opt.sessions || layer < 0 || layer >= c->cfg.layers || !c->layers[layer].full || pos0 < 0 || M < 1 || !h ||
      pos0 + M > d.max_pages * d.page_tokens) {
    set_error("chunk_attention_layer: bad argument (the layer must be a full-attention layer)");
    return LING_B200_ERR_ARG;
  }
  const LayerW& L = c->layers[layer];
  const int al = c->attn_index[layer];
  struct KeepCount {  // the verify step's launch count stays what its capture counted; the chains staged here are no step to launch
    ling_b200_ctx* c;
    int n;
    ~KeepCount() { c->launches_per_step = n, c->staged_seqs = 0, c->staged_rows = 0; }
  } keep{c, c->launches_per_step};
  ChunkChains cc;
  std::vector<ling_b200_seq_step> seqs;
  Planes none;
  none.p = nullptr;
  PdlScope pdl(c->opt.pdl != 0);
  for (int done = 0; done < M;) {
    const int rows = chunk_pass(c, slot, pos0 + done, M - done, 0, cc.zeros.data(), cc.chain.data(), seqs);
    if (rows == 0) {
      set_error("chunk_attention_layer: the context's step capacity holds no chain of the chunk");
      return LING_B200_ERR_ARG;
    }
    LB_TRY(stage_impl(c, seqs.data(), int(seqs.size()), 0, true));
    LB_TRY(check_attn_slots(c));
    const int cls = row_class(rows);
    c->last_rows = rows, c->last_seqs = int(seqs.size()), c->last_flags = 0;
    float* hs = h + size_t(done) * d.H;
    LB_TRY(pack_launch(c->sb, d, c->stream));
    {
      // the norm reads every row of its grid before it knows the row count (the step's residual buffer has them all): the pass's
      // rows go through that buffer, since the caller's array ends with the chunk
      Timed t(c, kFamElem);
      LB_CUDA(cudaMemcpyAsync(c->h, hs, size_t(rows) * d.H * 4, cudaMemcpyDeviceToDevice, c->stream));
      LB_TRY(norm_quant_launch(c->h, none, nullptr, c->embed, L.input_norm, nullptr, c->qout(c->xq_h), c->sb.n_rows_total, cls, d.H, d.eps, c->stream));
    }
    LB_TRY(run_gemm(c, L.qkv, c->xq_h, 0, cls));
    LB_TRY(attention_over_planes(c, L, al, planes_of(c, 0, L.qkv), nullptr, cls));
    LB_TRY(run_gemm(c, L.o, c->xq_a, 1, cls));
    // the o projection's partial sums into the residual rows, in place
    {
      Timed t(c, kFamElem);
      LB_TRY(add_planes_launch(hs, planes_of(c, 1, L.o), c->sb.n_rows_total, cls, d.H, c->stream));
    }
    LB_TRY(read_err(c));
    done += rows;
  }
  return LING_B200_OK;
}
// Where a chunk layer's device time goes: the layer over M zero rows with an event pair around every launch; ms[0] the two
// FP8 projections, [1] the attention kernel, [2] the combine, [3] the two norms, [5] the prepare kernel; *passes = launches of chains.
int ling_b200_chunk_attention_layer_profile(ling_b200_ctx* c, int slot, int layer, int pos0, int M, float ms[8], int* passes) {
  LB_TRY(check_ctx(c));
  if (!ms || M < 1) {
    set_error("chunk_attention_layer_profile: bad argument");
    return LING_B200_ERR_ARG;
  }
  float* dev = nullptr;
  const size_t bytes = size_t(M) * c->d.H * 4;
  LB_CUDA(cudaMalloc(&dev, bytes));
  cudaMemset(dev, 0, bytes);
  LB_TRY(finish(c));
  c->profiling = true;
  c->prof.clear();
  const int rc = ling_b200_chunk_attention_layer(c, slot, layer, pos0, M, dev);
  c->profiling = false;
  for (int i = 0; i < 8; ++i) ms[i] = 0.f;
  int norms = 0;
  for (auto& p : c->prof) {
    float t = 0.f;
    if (rc == LING_B200_OK) cudaEventElapsedTime(&t, p.second.first, p.second.second);
    ms[p.first] += t;
    norms += p.first == kFamElem;
    cudaEventDestroy(p.second.first), cudaEventDestroy(p.second.second);
  }
  if (passes) *passes = norms / 2;
  c->prof.clear();
  cudaFree(dev);
  return rc;
}
// The same with the residual rows in host memory (in and out).
int ling_b200_chunk_attention_layer_host(ling_b200_ctx* c, int slot, int layer, int pos0, int M, float* h) {
  LB_TRY(check_ctx(c));
  if (!h || M < 1) {
    set_error("chunk_attention_layer_host: bad argument");
    return LING_B200_ERR_ARG;
  }
  float* dev = nullptr;
  const size_t bytes = size_t(M) * c->d.H * 4;
  LB_CUDA(cudaMalloc(&dev, bytes));
  int rc = cudaMemcpy(dev, h, bytes, cudaMemcpyHostToDevice) == cudaSuccess ? LING_B200_OK : LING_B200_ERR_CUDA;
  if (rc == LING_B200_OK) rc = ling_b200_chunk_attention_layer(c, slot, layer, pos0, M, dev);
  if (rc == LING_B200_OK && cudaMemcpy(h, dev, bytes, cudaMemcpyDeviceToHost) != cudaSuccess) rc = LING_B200_ERR_CUDA;
  cudaFree(dev);
  return rc;
}

// ------------------------------------------------------------------------------------------------ read-backs
int ling_b200_read_tree_desc(ling_b200_ctx* c, int seq, ling_b200_tree_desc* out) {
  LB_TRY(check_ctx(c));
  if (seq < 0 || seq >= c->last_seqs || !out) {
    set_error("read_tree_desc: bad sequence index");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(finish(c));
  LB_CUDA(cudaMemcpy(out, c->sb.trees + seq, sizeof(ling_b200_tree_desc), cudaMemcpyDeviceToHost));
  return LING_B200_OK;
}
int ling_b200_read_packing(ling_b200_ctx* c, int* row0, int* token, int* seq_of, int* depth, int* rope_pos, int* cache_slot,
                           uint32_t* anc_mask) {
  LB_TRY(check_ctx(c));
  LB_TRY(finish(c));
  const size_t n = size_t(c->last_rows);
  if (row0) LB_CUDA(cudaMemcpy(row0, c->sb.row0, size_t(c->last_seqs + 1) * 4, cudaMemcpyDeviceToHost));
  if (token) LB_CUDA(cudaMemcpy(token, c->sb.token, n * 4, cudaMemcpyDeviceToHost));
  if (seq_of) LB_CUDA(cudaMemcpy(seq_of, c->sb.seq_of, n * 4, cudaMemcpyDeviceToHost));
  if (depth) LB_CUDA(cudaMemcpy(depth, c->sb.depth, n * 4, cudaMemcpyDeviceToHost));
  if (rope_pos) LB_CUDA(cudaMemcpy(rope_pos, c->sb.rope_pos, n * 4, cudaMemcpyDeviceToHost));
  if (cache_slot) LB_CUDA(cudaMemcpy(cache_slot, c->sb.cache_slot, n * 4, cudaMemcpyDeviceToHost));
  if (anc_mask) LB_CUDA(cudaMemcpy(anc_mask, c->sb.anc, n * 4, cudaMemcpyDeviceToHost));
  return LING_B200_OK;
}
int ling_b200_read_argmax(ling_b200_ctx* c, int* ids, float* vals) {
  LB_TRY(check_ctx(c));
  LB_TRY(finish(c));
  if (ids) LB_CUDA(cudaMemcpy(ids, c->sb.argmax_id, size_t(c->last_rows) * 4, cudaMemcpyDeviceToHost));
  if (vals) LB_CUDA(cudaMemcpy(vals, c->sb.argmax_val, size_t(c->last_rows) * 4, cudaMemcpyDeviceToHost));
  return LING_B200_OK;
}
int ling_b200_read_logits(ling_b200_ctx* c, float* out) {
  LB_TRY(check_ctx(c));
  if (!(c->last_flags & LING_B200_STEP_KEEP_LOGITS) || !c->logits) {
    set_error("read_logits: the last step did not keep logits");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(finish(c));
  LB_CUDA(cudaMemcpy(out, c->logits, size_t(c->last_rows) * c->d.V * 4, cudaMemcpyDeviceToHost));
  return LING_B200_OK;
}
int ling_b200_read_tap(ling_b200_ctx* c, int layer, float* out) {
  LB_TRY(check_ctx(c));
  if (!(c->last_flags & LING_B200_STEP_KEEP_TAPS) || !c->taps || layer < 0 || layer > c->cfg.layers) {
    set_error("read_tap: the last step did not keep taps, or bad layer");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(finish(c));
  LB_CUDA(cudaMemcpy(out, c->taps + size_t(layer) * c->opt.debug_rows * c->d.H, size_t(c->last_rows) * c->d.H * 4,
                     cudaMemcpyDeviceToHost));
  return LING_B200_OK;
}

// ------------------------------------------------------------------------------------------------ the drafter's last stage
// Engine::draft_launch from its final norm on (src/core/speculate.cpp:598-617) and draft_head's full-head branch
// (speculate.cpp:405-416): the drafted rows through the target's LM head (this context's FP8 head and activation
// quantizer), the top 16 of each row, the selector's projection and lattice; candidates and scores come back to the host,
// where build_tree takes them.  The weights of the selector are uploaded once.
}  // extern "C"

struct ling_b200_draft_head {
  ling_b200_ctx* c = nullptr;
  __nv_bfloat16 *proj = nullptr, *pred = nullptr, *succ = nullptr;
  float *x = nullptr, *logits = nullptr, *hp = nullptr, *unary = nullptr, *scores = nullptr, *scratch = nullptr;
  int* cand = nullptr;
  int max_rows = 0;
  // the sparse head (ling_b200_draft_head_enable_sparse): the rank-256 factors, one mask per session, the selection and the
  // compact matrix of the selected rows
  __nv_bfloat16 *us = nullptr, *vt = nullptr;
  uint8_t* masks = nullptr;   // [sessions][vocab]
  float *p = nullptr, *sparse_logits = nullptr;
  void* sel_scratch = nullptr;
  int *rows = nullptr, *nrows = nullptr, *ids_tmp = nullptr;
  int dynamic = 0, cap = 0;
  Fp8Matrix compact;
};

extern "C" {

int ling_b200_draft_head_create(ling_b200_ctx* c, const uint16_t* selector_projection, const uint16_t* predecessor_codebook,
                                const uint16_t* successor_codebook, ling_b200_draft_head** out) {
  LB_TRY(check_ctx(c));
  if (!selector_projection || !predecessor_codebook || !successor_codebook || !out || c->d.H % 256 != 0) {
    set_error("draft_head_create: bad argument (the hidden size must be a multiple of 256)");
    return LING_B200_ERR_ARG;
  }
  auto* h = new ling_b200_draft_head;
  h->c = c;
  h->max_rows = std::min(kTreeRows - 1, c->d.rows_alloc);
  const size_t V = size_t(c->d.V), R = size_t(h->max_rows);
  auto up = [&](__nv_bfloat16** dst, const uint16_t* src, size_t n) -> int {
    LB_TRY(c->alloc(dst, n, false));
    LB_CUDA(cudaMemcpy(*dst, src, n * 2, cudaMemcpyHostToDevice));
    return LING_B200_OK;
  };
  int rc = up(&h->proj, selector_projection, size_t(kSelRank) * c->d.H);
  if (rc == LING_B200_OK) rc = up(&h->pred, predecessor_codebook, V * kSelRank);
  if (rc == LING_B200_OK) rc = up(&h->succ, successor_codebook, V * kSelRank);
  if (rc == LING_B200_OK) rc = c->alloc(&h->x, R * c->d.H);
  if (rc == LING_B200_OK) rc = c->alloc(&h->logits, R * V, false);
  if (rc == LING_B200_OK) rc = c->alloc(&h->hp, R * kSelRank);
  if (rc == LING_B200_OK) rc = c->alloc(&h->unary, R * kSelTop);
  if (rc == LING_B200_OK) rc = c->alloc(&h->cand, R * kSelTop);
  if (rc == LING_B200_OK) rc = c->alloc(&h->scores, R * kSelTop * kSelTop);
  if (rc == LING_B200_OK) rc = c->alloc(&h->scratch, topk_scratch_floats(h->max_rows, c->d.V, kSelTop));
  if (rc != LING_B200_OK) {  // what was allocated stays with the context and is freed with it
    delete h;
    return rc;
  }
  *out = h;
  return LING_B200_OK;
}
void ling_b200_draft_head_destroy(ling_b200_draft_head* h) { delete h; }  // its device memory belongs to the context

int ling_b200_draft_head_run(ling_b200_draft_head* h, const float* x, int E, int anchor, int* cand, float* unary, float* scores) {
  if (!h) {
    set_error("draft_head_run: no handle");
    return LING_B200_ERR_ARG;
  }
  ling_b200_ctx* c = h->c;
  LB_TRY(check_ctx(c));
  if (!x || !cand || !scores || E < 1 || E > h->max_rows || anchor < 0 || anchor >= c->d.V) {
    set_error("draft_head_run: bad argument (1 <= rows <= 31 and within the context's row capacity; the anchor a token id)");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(finish(c));  // the head's activation buffer is the step's
  cudaStream_t s = c->stream;
  LB_CUDA(cudaMemcpyAsync(h->x, x, size_t(E) * c->d.H * 4, cudaMemcpyHostToDevice, s));
  LB_TRY(quant_acts_launch(h->x, E, c->qout(c->xq_h), s));
  {
    HeadEpilogue ep = c->head_ep;
    ep.store_logits = true;
    GemmCall g;
    g.W = &c->head, g.X = &c->xq_h, g.M = E;
    g.out = h->logits, g.ld = c->head.N;
    g.split_stride = size_t(c->d.rows_alloc) * c->head.N_pad;
    g.head = &ep;
    g.impl = c->opt.gemm_impl;
    g.err_flag = c->sb.err;
    LB_TRY(gemm_launch(g, s));
  }
  LB_TRY(topk_rows_launch(h->logits, E, c->d.V, kSelTop, h->scratch, h->unary, h->cand, s));
  LB_TRY(selector_project_launch(h->x, h->proj, E, c->d.H, h->hp, s));
  LB_TRY(selector_lattice_launch(h->hp, h->cand, h->unary, h->pred, h->succ, c->d.V, anchor, nullptr, E, h->scores, c->sb.err, s));
  LB_CUDA(cudaMemcpyAsync(cand, h->cand, size_t(E) * kSelTop * 4, cudaMemcpyDeviceToHost, s));
  if (unary) LB_CUDA(cudaMemcpyAsync(unary, h->unary, size_t(E) * kSelTop * 4, cudaMemcpyDeviceToHost, s));
  LB_CUDA(cudaMemcpyAsync(scores, h->scores, size_t(E) * kSelTop * kSelTop * 4, cudaMemcpyDeviceToHost, s));
  return read_err(c);
}

// The sparse head (src/core/sparse_head.cu; EngineOptions::sparse_head_dynamic, src/core/engine.hpp:160-173): us [vocab][256] and
// vt [256][hidden] are the rank-256 factors of the head (BF16); `dynamic` rows are chosen by the factors every step, `cap` bounds
// the selection.  Every session gets an empty mask.
int ling_b200_draft_head_enable_sparse(ling_b200_draft_head* h, const uint16_t* us_bf16, const uint16_t* vt_bf16, int dynamic, int cap) {
  if (!h || !us_bf16 || !vt_bf16 || dynamic < 0 || cap < kSelTop || h->us) {
    set_error("draft_head_enable_sparse: bad argument (capacity >= 16), or enabled already");
    return LING_B200_ERR_ARG;
  }
  ling_b200_ctx* c = h->c;
  LB_TRY(check_ctx(c));
  const size_t V = size_t(c->d.V);
  const Fp8Matrix& W = c->head;
  LB_TRY(c->alloc(&h->us, V * kSelRank, false));
  LB_TRY(c->alloc(&h->vt, size_t(kSelRank) * c->d.H, false));
  LB_CUDA(cudaMemcpy(h->us, us_bf16, V * kSelRank * 2, cudaMemcpyHostToDevice));
  LB_CUDA(cudaMemcpy(h->vt, vt_bf16, size_t(kSelRank) * c->d.H * 2, cudaMemcpyHostToDevice));
  LB_TRY(c->alloc(&h->masks, size_t(c->opt.sessions) * V));
  LB_TRY(c->alloc(&h->p, size_t(32) * kSelRank));
  uint8_t* scratch = nullptr;
  LB_TRY(c->alloc(&scratch, sparse_scratch_bytes(int(V))));
  h->sel_scratch = scratch;
  LB_TRY(c->alloc(&h->rows, size_t(cap)));
  LB_TRY(c->alloc(&h->nrows, size_t(1)));
  LB_TRY(c->alloc(&h->ids_tmp, size_t(c->d.V > 65536 ? 65536 : c->d.V)));
  Fp8Matrix& m = h->compact;
  m.N = cap, m.K = W.K, m.N_pad = round_up(cap, kTileN), m.K_pad = W.K_pad, m.KB = W.KB, m.splits = 1;
  LB_TRY(c->alloc(&m.codes, size_t(m.N_pad) * m.K_pad));
  LB_TRY(c->alloc(&m.scales, size_t(m.KB) * m.N_pad));
  LB_TRY(make_weight_map(m));
  LB_TRY(c->alloc(&h->sparse_logits, size_t(h->max_rows) * cap, false));
  h->dynamic = dynamic, h->cap = cap;
  return LING_B200_OK;
}

// A session's mask: reset = cleared, then the ids marked (the fixed list and the prompt's ids); mark = more ids (its output).
static int mask_ids(ling_b200_draft_head* h, int session, const int* ids, int n, bool clear) {
  if (!h || !h->us || session < 0 || session >= h->c->opt.sessions || n < 0 || (n > 0 && !ids)) {
    set_error("draft_head_mask: bad argument, or the sparse head is not enabled");
    return LING_B200_ERR_ARG;
  }
  ling_b200_ctx* c = h->c;
  LB_TRY(check_ctx(c));
  uint8_t* mask = h->masks + size_t(session) * c->d.V;
  if (clear) LB_CUDA(cudaMemsetAsync(mask, 0, size_t(c->d.V), c->stream));
  for (int done = 0; done < n; done += 65536) {
    const int m = std::min(65536, n - done);
    LB_CUDA(cudaMemcpyAsync(h->ids_tmp, ids + done, size_t(m) * 4, cudaMemcpyHostToDevice, c->stream));
    LB_TRY(sparse_mark_launch(mask, h->ids_tmp, m, c->d.V, c->stream));
    LB_CUDA(cudaStreamSynchronize(c->stream));  // ids_tmp and the caller's array are free again
  }
  return LING_B200_OK;
}
int ling_b200_draft_head_mask_reset(ling_b200_draft_head* h, int session, const int* ids, int n) { return mask_ids(h, session, ids, n, true); }
int ling_b200_draft_head_mask_mark(ling_b200_draft_head* h, int session, const int* ids, int n) { return mask_ids(h, session, ids, n, false); }

// ling_b200_draft_head_run through the sparse head for one session's rows (draft_head_rows' sparse branch,
// src/core/sparse_head.cu:262-276): p = x . vt^T, the selection under the session's mask, the selected rows gathered and multiplied by the head
// GEMM (their logits are the full head's bits), top 16 among them mapped back to token ids, then the selector as before.
// *n_selected (may be NULL): how many rows were scored; selected (may be NULL): their ids, up to the capacity.
int ling_b200_draft_head_run_sparse(ling_b200_draft_head* h, int session, const float* x, int E, int anchor, int* cand, float* unary,
                                    float* scores, int* n_selected, int* selected) {
  if (!h || !h->us) {
    set_error("draft_head_run_sparse: the sparse head is not enabled");
    return LING_B200_ERR_ARG;
  }
  ling_b200_ctx* c = h->c;
  LB_TRY(check_ctx(c));
  if (!x || !cand || !scores || E < 1 || E > h->max_rows || anchor < 0 || anchor >= c->d.V || session < 0 || session >= c->opt.sessions) {
    set_error("draft_head_run_sparse: bad argument");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(finish(c));
  cudaStream_t s = c->stream;
  LB_CUDA(cudaMemcpyAsync(h->x, x, size_t(E) * c->d.H * 4, cudaMemcpyHostToDevice, s));
  LB_TRY(selector_project_launch(h->x, h->vt, E, c->d.H, h->p, s));
  SparseMasks ms;
  ms.n = 1, ms.m[0] = h->masks + size_t(session) * c->d.V;
  for (int i = 1; i < kSparseMasks; ++i) ms.m[i] = ms.m[0];
  LB_TRY(sparse_select_launch(h->p, E, h->us, c->d.V, ms, h->dynamic, h->cap, h->sel_scratch, c->sm_count, h->rows, h->nrows, c->sb.err, s));
  const Fp8Matrix& W = c->head;
  Fp8Matrix& m = h->compact;
  LB_TRY(sparse_gather_launch(W.codes, W.scales, W.N_pad, W.K_pad, W.KB, h->rows, h->nrows, h->cap, m.codes, m.scales, m.N_pad, s));
  LB_TRY(quant_acts_launch(h->x, E, c->qout(c->xq_h), s));
  {
    HeadEpilogue ep = c->head_ep;
    ep.store_logits = true;
    GemmCall g;
    g.W = &m, g.X = &c->xq_h, g.M = E;
    g.out = h->sparse_logits, g.ld = m.N;
    g.split_stride = size_t(c->d.rows_alloc) * m.N_pad;
    g.head = &ep;
    g.impl = c->opt.gemm_impl;
    g.err_flag = c->sb.err;
    LB_TRY(gemm_launch(g, s));
  }
  LB_TRY(sparse_tail_launch(h->sparse_logits, E, h->cap, h->cap, h->nrows, s));
  LB_TRY(topk_rows_launch(h->sparse_logits, E, h->cap, kSelTop, h->scratch, h->unary, h->cand, s));
  LB_TRY(sparse_ids_launch(h->rows, h->nrows, h->cand, E * kSelTop, s));
  LB_TRY(selector_project_launch(h->x, h->proj, E, c->d.H, h->hp, s));
  LB_TRY(selector_lattice_launch(h->hp, h->cand, h->unary, h->pred, h->succ, c->d.V, anchor, nullptr, E, h->scores, c->sb.err, s));
  LB_CUDA(cudaMemcpyAsync(cand, h->cand, size_t(E) * kSelTop * 4, cudaMemcpyDeviceToHost, s));
  if (unary) LB_CUDA(cudaMemcpyAsync(unary, h->unary, size_t(E) * kSelTop * 4, cudaMemcpyDeviceToHost, s));
  LB_CUDA(cudaMemcpyAsync(scores, h->scores, size_t(E) * kSelTop * kSelTop * 4, cudaMemcpyDeviceToHost, s));
  LB_TRY(read_err(c));
  int n = 0;
  LB_CUDA(cudaMemcpy(&n, h->nrows, 4, cudaMemcpyDeviceToHost));
  if (n_selected) *n_selected = n;
  if (selected && n > 0) LB_CUDA(cudaMemcpy(selected, h->rows, size_t(n) * 4, cudaMemcpyDeviceToHost));
  return LING_B200_OK;
}

}  // extern "C"
