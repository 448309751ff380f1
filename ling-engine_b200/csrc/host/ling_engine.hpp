// ling_engine.hpp -- the reference engine's C++ surface for the verify-step path, as a header-only facade over the C ABI
// (include/ling_b200.h).  Names, argument meaning and error behaviour follow the reference project
// (dreamference/ling-engine: src/core/engine.hpp, tree.hpp, lookup.hpp, kv_pool.hpp, sampling.hpp, src/serve/*.hpp), so a
// caller written against it keeps its source.  Every body forwards to the library; nothing here computes on its own.
#pragma once

#include <algorithm>
#include <chrono>
#include <cstdint>
#include <deque>
#include <exception>
#include <functional>
#include <memory>
#include <span>
#include <stdexcept>
#include <string>
#include <vector>

#include "ling_b200.h"

namespace ling {

namespace kernels {
constexpr int kMaxSeqs = LING_B200_MAX_SEQS;                  // src/core/kernels.cuh:52 (4 there)
constexpr int kMaxStreamRows = LING_B200_MAX_TREE_ROWS;       // rows of one sequence's tree (kernels.cuh:107)
constexpr int kMaxTreeVariants = LING_B200_MAX_TREE_VARIANTS;
struct TreeDesc : ling_b200_tree_desc {                       // src/core/kernels.cuh:119-130, the same field order
  static constexpr int kLeaf = LING_B200_TREE_LEAF, kWrite = LING_B200_TREE_WRITE;
};
}  // namespace kernels

// ---- src/core/sampling.hpp
struct SamplingParams {
  float temperature = 1.0f;  // 0 = greedy; the verify step implements the greedy contract
  int top_k = 20;
  float top_p = 0.95f, min_p = 0.f, presence_penalty = 0.f, repetition_penalty = 1.f;
  uint64_t seed = 0;
};
class NonFiniteLogits : public std::runtime_error {
 public:
  NonFiniteLogits() : std::runtime_error("the model produced non-finite logits (NaN or inf); the request was stopped") {}
};
class KvPoolExhausted : public std::runtime_error {  // src/core/engine.hpp:227-232
 public:
  using std::runtime_error::runtime_error;
};

// ---- src/core/tree.hpp
struct TreeShape {
  int nodes = 0;
  double temp = 1.0;
  int width = 16, max_depth = 1000, chain = 1000;
};
struct DraftTree {
  int E = 0;
  std::vector<int> parent, depth, token, pick;
  std::vector<std::vector<int>> children;
  double extra_mass = 0;
  int rows() const { return static_cast<int>(parent.size()); }
};
inline DraftTree build_tree(int anchor, const int* cand, const float* scores, int E, int K16, const std::vector<int>& chain_tokens,
                            const std::vector<int>& chain_picks, const TreeShape& shape) {
  DraftTree t;
  std::vector<int> par(64), dep(64), tok(64), pk(64);
  const int r = ling_b200_build_tree(anchor, cand, scores, E, K16, chain_tokens.data(), chain_picks.data(), shape.nodes, shape.temp,
                                     shape.width, shape.max_depth, shape.chain, kernels::kMaxStreamRows, par.data(), dep.data(),
                                     tok.data(), pk.data(), &t.extra_mass);
  const int rows = r & 0xffff;
  t.E = r >> 16;
  t.parent.assign(par.begin(), par.begin() + rows), t.depth.assign(dep.begin(), dep.begin() + rows);
  t.token.assign(tok.begin(), tok.begin() + rows), t.pick.assign(pk.begin(), pk.begin() + rows);
  t.children.assign(rows, {});
  for (int i = 1; i < rows; ++i) t.children[t.parent[i]].push_back(i);
  return t;
}
// Fills the device description; returns the number of DeltaNet paths.  Throws like the reference on too many rows,
// leaves or paths (src/core/tree.cpp:83,93,139).
inline int describe_tree(const DraftTree& t, kernels::TreeDesc& d) {
  if (ling_b200_describe_tree(t.parent.data(), t.rows(), t.E, &d) != LING_B200_OK)
    throw std::runtime_error("tree: more rows, leaves or gdn paths than the description holds");
  return d.ngdn;
}
inline std::vector<int> accept_tree_greedy(const DraftTree& t, const int* argmax, int& next) {
  std::vector<int> path(t.rows());
  path.resize(ling_b200_accept_tree_greedy(t.parent.data(), t.token.data(), t.rows(), argmax, path.data(), &next));
  return path;
}

// ---- src/core/lookup.hpp
struct LookupProposal {
  std::vector<int> tokens;
  int match = 0;
};
inline LookupProposal lookup_propose(const std::vector<int>& seq, int max, int ngram = 3) {
  LookupProposal p;
  p.tokens.resize(std::max(max, 0));
  p.tokens.resize(ling_b200_lookup_propose(seq.data(), static_cast<int>(seq.size()), max, ngram, p.tokens.data(), &p.match));
  return p;
}

// ---- src/core/kv_pool.hpp
class KvPool {
 public:
  struct Copy {
    int src, dst;
  };
  using Refs = std::vector<const std::vector<int>*>;
  // `pages` ids, 1 .. pages - 1 usable.  page_tokens: 64 in the reference; a parameter here (16-token pages exist).
  explicit KvPool(int pages, int page_tokens = 64) : p_(ling_b200_kvpool_create(pages, page_tokens)), page_tokens_(page_tokens) {}
  ~KvPool() { ling_b200_kvpool_destroy(p_); }
  KvPool(const KvPool&) = delete;
  KvPool& operator=(const KvPool&) = delete;
  int capacity() const { return ling_b200_kvpool_capacity(p_); }
  int free_pages() const { return ling_b200_kvpool_free_pages(p_); }
  int pending_pages() const { return ling_b200_kvpool_pending_pages(p_); }
  int refs(int page) const { return ling_b200_kvpool_refs(p_, page); }
  int index_of(int pos) const { return pos / page_tokens_; }
  int pages_for(int positions) const { return (positions + page_tokens_ - 1) / page_tokens_; }
  int needed(const std::vector<int>& table, int from, int to) const {
    return ling_b200_kvpool_needed(p_, table.data(), static_cast<int>(table.size()), from, to);
  }
  int net_need(const std::vector<int>& table, int pages) const {
    return ling_b200_kvpool_net_need(p_, table.data(), static_cast<int>(table.size()), pages);
  }
  // All or nothing: false, with nothing changed, when the free list is short.
  bool ensure(std::vector<int>& table, int from, int to, std::vector<Copy>* copies) {
    const int cap = std::max(static_cast<int>(table.size()), pages_for(to));
    int len = static_cast<int>(table.size()), nc = 0;
    table.resize(cap, 0);
    std::vector<int> cp(2 * size_t(cap));
    const int r = ling_b200_kvpool_ensure(p_, table.data(), &len, cap, from, to, cp.data(), cap, &nc);
    table.resize(len);
    if (r < 0) throw std::invalid_argument("KvPool::ensure: bad range");
    if (copies)
      for (int i = 0; i < nc; ++i) copies->push_back({cp[2 * i], cp[2 * i + 1]});
    return r == 1;
  }
  void share(std::vector<int>& dst, const std::vector<int>& src, int n) {
    const int cap = std::max(static_cast<int>(dst.size()), pages_for(n));
    int len = static_cast<int>(dst.size());
    dst.resize(cap, 0);
    const int r = ling_b200_kvpool_share(p_, dst.data(), &len, cap, src.data(), static_cast<int>(src.size()), n);
    dst.resize(len);
    if (r != 0) throw std::invalid_argument("KvPool::share: src does not hold [0, n)");
  }
  void truncate(std::vector<int>& table, int n) { ling_b200_kvpool_truncate(p_, table.data(), static_cast<int>(table.size()), n); }
  void unshare(std::vector<int>& table, int n) { ling_b200_kvpool_unshare(p_, table.data(), static_cast<int>(table.size()), n); }
  int resume_need(const std::vector<int>& table, int reuse, int pages, const std::vector<int>* donor) const {
    return ling_b200_kvpool_resume_need(p_, table.data(), static_cast<int>(table.size()), reuse, pages,
                                        donor ? donor->data() : nullptr, donor ? static_cast<int>(donor->size()) : 0);
  }
  int reclaimable(const Refs& refs) const {
    std::vector<const int*> t;
    std::vector<int> n;
    for (const std::vector<int>* r : refs)
      if (r) t.push_back(r->data()), n.push_back(static_cast<int>(r->size()));
    return ling_b200_kvpool_reclaimable(p_, t.data(), n.data(), static_cast<int>(t.size()));
  }
  void retain(int page) {
    if (ling_b200_kvpool_retain(p_, page)) throw std::logic_error("KvPool::retain: not a live page");
  }
  void release(int page) {
    if (ling_b200_kvpool_release(p_, page)) throw std::logic_error("KvPool::release: not a live page");
  }
  void retire() { ling_b200_kvpool_retire(p_); }

 private:
  ling_b200_kvpool* p_;
  int page_tokens_;
};

// ---- src/core/model.hpp, src/core/engine.hpp
using ModelConfig = ling_b200_model_config;
// The resident sessions and their KV pages as the scheduler sees them (the host-side half of Engine's session functions,
// src/core/engine.cpp:581-648,724-800,881-912, and of its Session struct, engine.hpp:760-800).  No device work: Engine
// keeps one and adds the device side; a scheduler test can keep one alone.  This build has no prefix KV store and no
// donor sessions (a resumed prompt reuses only its own session's positions), so pages are never shared between holders
// and a need planned "with holders gone" (Engine::KvGone) equals the need planned now.
struct Session {
  std::vector<int> history, table;  // tokens processed; page ids by page index (0 = unmapped)
  int pos = 0;
  bool owned = false;               // bound to a conversation (free_session hands out the others first)
  std::string key;
  uint64_t scope = 0;
  int prompt_len = 0, turn_start = 0;
  double last_used = 0;             // seconds on the book's clock
};
class SessionBook {
 public:
  static constexpr int kKvGrowthPages = 2;  // src/core/engine.hpp:433
  SessionBook(int sessions, int pool_pages, int page_tokens, int max_context, int step_rows = kernels::kMaxStreamRows)
      : pool_(pool_pages + 1, page_tokens), sess_(size_t(sessions)), page_tokens_(page_tokens), max_context_(max_context), step_rows_(step_rows) {}
  std::function<double()> clock = [] {
    return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
  };
  KvPool& pool() { return pool_; }
  const KvPool& pool() const { return pool_; }
  int sessions() const { return static_cast<int>(sess_.size()); }
  int max_context() const { return max_context_; }
  Session& at(int i) { return sess_.at(size_t(i)); }
  const Session& at(int i) const { return sess_.at(size_t(i)); }

  // Engine::match_session (engine.cpp:581-603): the owned session of the same scope whose history shares the longest prefix
  // with the prompt, at least up to where its last turn began; a key breaks ties and, failing every prefix, names it.
  int match_session(const std::vector<int>& prompt, const std::string& key, uint64_t scope) const {
    int best = -1, best_lcp = 0;
    for (int i = 0; i < sessions(); ++i) {
      const Session& s = sess_[size_t(i)];
      if (!s.owned || s.history.empty() || s.prompt_len == 0 || s.scope != scope) continue;
      const int lcp = common_prefix(s.history, prompt);
      if (lcp < s.turn_start) continue;
      if (lcp > best_lcp || (lcp == best_lcp && !key.empty() && s.key == key)) best = i, best_lcp = lcp;
    }
    if (best >= 0 || key.empty()) return best;
    for (int i = 0; i < sessions(); ++i)
      if (sess_[size_t(i)].owned && sess_[size_t(i)].key == key && sess_[size_t(i)].scope == scope) return i;
    return -1;
  }
  // Engine::free_session (engine.cpp:605-619): an unowned slot first; else the least recently used one that is neither
  // pinned nor (keyed and used within protect_seconds).
  int free_session(double protect_seconds, const std::vector<bool>& pinned) const {
    auto is_pinned = [&](int i) { return size_t(i) < pinned.size() && pinned[size_t(i)]; };
    for (int i = 0; i < sessions(); ++i)
      if (!sess_[size_t(i)].owned && !is_pinned(i)) return i;
    const double now = clock();
    int best = -1;
    for (int i = 0; i < sessions(); ++i) {
      const Session& s = sess_[size_t(i)];
      if (is_pinned(i) || (!s.key.empty() && now - s.last_used < protect_seconds)) continue;
      if (best < 0 || s.last_used < sess_[size_t(best)].last_used) best = i;
    }
    return best;
  }
  // The bookkeeping of Engine::activate_session (engine.cpp:621-646); returns whether an owned session was taken over.
  bool activate(int i, const std::string& key, bool fresh, uint64_t scope) {
    Session& s = at(i);
    bool took_over = false;
    if (s.scope != scope) {  // another scope's history is never resumed from; its pages stay until the prefill rewrites them
      s.history.clear();
      s.prompt_len = s.turn_start = s.pos = 0;
      s.scope = scope;
    }
    if (fresh) {
      took_over = s.owned;
      s.owned = true;
      s.key = key;
    } else if (!key.empty()) {
      s.key = key;
    }
    touch(i);
    return took_over;
  }
  void touch(int i) { at(i).last_used = clock(); }
  int resident() const { return static_cast<int>(std::count_if(sess_.begin(), sess_.end(), [](const Session& s) { return s.owned; })); }

  // ---- pages (engine.cpp:724-800,881-912)
  int kv_admit_pages(size_t prompt_len) const { return pool_.pages_for(static_cast<int>(prompt_len)) + kKvGrowthPages; }
  int kv_step_rows(const Session& s, bool spec) const {
    const int room = max_context_ - s.pos;
    return std::max(0, std::min(spec ? step_rows_ : 1, room));
  }
  int kv_step_need(int session, bool spec) const {
    const Session& s = at(session);
    return pool_.needed(s.table, s.pos, s.pos + kv_step_rows(s, spec));
  }
  // Positions of the session's own history that a prompt resumes from (the no-donor, no-store case of plan_resume,
  // engine.cpp:1747-1842): the common prefix, never the whole prompt (its last token is processed again for the logits).
  int resume_reuse(int session, const std::vector<int>& prompt, uint64_t scope, bool from_scratch) const {
    const Session& s = at(session);
    if (from_scratch || s.scope != scope || prompt.empty()) return 0;
    return std::min(common_prefix(s.history, prompt), static_cast<int>(prompt.size()) - 1);
  }
  int kv_admit_need(int session, const std::vector<int>& prompt, uint64_t scope, bool from_scratch = false) const {
    if (prompt.empty()) return 0;
    return pool_.resume_need(at(session).table, resume_reuse(session, prompt, scope, from_scratch), kv_admit_pages(prompt.size()), nullptr);
  }
  int kv_reclaimable(const std::vector<int>& sessions) const {
    KvPool::Refs refs;
    for (int i : sessions) refs.push_back(&at(i).table);
    return pool_.reclaimable(refs);
  }
  int kv_lru_idle(const std::vector<bool>& busy) const {
    int best = -1;
    for (int i = 0; i < sessions(); ++i) {
      const Session& s = sess_[size_t(i)];
      if (size_t(i) < busy.size() && busy[size_t(i)]) continue;
      const bool holds = std::any_of(s.table.begin(), s.table.end(), [](int p) { return p != 0; });
      if (holds && (best < 0 || s.last_used < sess_[size_t(best)].last_used)) best = i;
    }
    return best;
  }
  // Engine::kv_evict's bookkeeping (engine.cpp:881-898): pages released (deferred), history forgotten, slot unowned.
  bool evict(int session) {
    Session& s = at(session);
    if (s.table.empty() && s.history.empty()) return false;
    pool_.truncate(s.table, 0);
    s.history.clear();
    s.prompt_len = s.turn_start = s.pos = 0;
    const bool was_owned = s.owned;
    s.owned = false;
    s.key.clear();
    return was_owned;
  }
  static int common_prefix(const std::vector<int>& a, const std::vector<int>& b) {
    const size_t n = std::min(a.size(), b.size());
    size_t i = 0;
    while (i < n && a[i] == b[i]) ++i;
    return static_cast<int>(i);
  }

 private:
  KvPool pool_;
  std::vector<Session> sess_;
  int page_tokens_, max_context_, step_rows_;
};

struct EngineOptions {
  int max_context = 65536;
  int sessions = 1;
  bool step_graphs = true;  // one CUDA graph per step (the reference replays three, engine.hpp:125)
  bool pdl = false;
  bool kv_pages = true;     // the KV lives in the page pool (always, here)
  int kv_pool_pages = 0;    // 0: every session's max_context
  int page_tokens = 16;
  int max_seqs = 4, max_rows = 128;
  int device = 0;
  int boundary_token = -1;  // the token that starts a message (engine.hpp:171); -1: prompts carry no boundaries
};

class Engine {
 public:
  static constexpr int kKvGrowthPages = 2;
  struct SeqStep {                            // src/core/engine.hpp:337-344
    int session = -1;
    int anchor = 0;                           // the next token, chosen but not yet processed
    const SamplingParams* params = nullptr;
    std::vector<float>* row_logits = nullptr;
    std::vector<int> out;                     // the accepted drafts, then the next token
    std::exception_ptr error;                 // NonFiniteLogits: nothing committed for this sequence
  };
  // The drafter is outside this path: the caller supplies each step's tree (row 0 the anchor) through this hook, which
  // stands in for plan_draft + build_tree (src/core/speculate.cpp:970-987).
  using TreeSource = std::function<DraftTree(int session, int anchor, const std::vector<int>& history)>;

  static int pool_pages_for(const EngineOptions& o) {
    return o.kv_pool_pages > 0 ? o.kv_pool_pages : (o.max_context + o.page_tokens - 1) / o.page_tokens * o.sessions;
  }
  Engine(const ModelConfig& cfg, EngineOptions opts = {})
      : cfg_(cfg), opts_(opts), book_(opts.sessions, pool_pages_for(opts), opts.page_tokens, opts.max_context) {
    ling_b200_options o{};
    o.sessions = opts.sessions, o.max_context = opts.max_context, o.page_tokens = opts.page_tokens;
    o.pool_pages = pool_pages_for(opts);
    o.max_seqs = opts.max_seqs, o.max_rows = opts.max_rows, o.use_graph = opts.step_graphs, o.device = opts.device, o.pdl = opts.pdl;
    if (ling_b200_create(&cfg_, &o, &ctx_) != LING_B200_OK) {
      const std::string why = ling_b200_last_error();
      ling_b200_destroy(ctx_);
      throw std::runtime_error("Engine: " + why);
    }
  }
  ~Engine() { ling_b200_destroy(ctx_); }
  Engine(const Engine&) = delete;
  Engine& operator=(const Engine&) = delete;

  ling_b200_ctx* handle() { return ctx_; }
  const ModelConfig& config() const { return cfg_; }
  int sessions() const { return book_.sessions(); }
  SessionBook& book() { return book_; }
  int max_context() const { return opts_.max_context; }
  void set_tree_source(TreeSource f) { tree_source_ = std::move(f); }
  void select_session(int i) { active_ = i; }
  int active_session() const { return active_; }
  const std::vector<int>& history() const { return book_.at(active_).history; }
  int position(int session) const { return book_.at(session).pos; }
  // What a prefill would leave: `tokens` become the session's history, its KV positions are mapped; the caller fills the
  // cache and the state through the handle (ling_b200_kv_write / ling_b200_state_write or the synthetic fills).
  void adopt_context(int session, const std::vector<int>& tokens) {
    Session& s = book_.at(session);
    s.history = tokens;
    s.pos = static_cast<int>(tokens.size());
    kv_ensure(s, session, 0, s.pos);
  }

  bool can_speculate(const SamplingParams& p) const { return p.temperature <= 0.f && static_cast<bool>(tree_source_); }
  bool can_batch(int session, const SamplingParams& p) const {
    return can_speculate(p) && session >= 0 && session < sessions() &&
           book_.at(session).pos + kernels::kMaxStreamRows <= opts_.max_context;
  }

  // ---- the KV page pool as the scheduler sees it (src/core/engine.hpp:428-493)
  bool kv_paged() const { return true; }
  int kv_pages_total() const { return book_.pool().capacity(); }
  int kv_pages_free() { return book_.pool().free_pages(); }
  int kv_pages_pending() const { return book_.pool().pending_pages(); }
  int kv_admit_pages(size_t prompt_len) const { return book_.kv_admit_pages(prompt_len); }
  int kv_step_need(int session, bool spec) const { return book_.kv_step_need(session, spec); }
  int kv_admit_need(int session, const std::vector<int>& prompt, uint64_t scope, bool from_scratch = false) const {
    return book_.kv_admit_need(session, prompt, scope, from_scratch);
  }
  int kv_session_pages(int session) const { return book_.kv_reclaimable({session}); }
  int kv_reclaimable(const std::vector<int>& sessions) const { return book_.kv_reclaimable(sessions); }
  int kv_lru_idle(const std::vector<bool>& busy) const { return book_.kv_lru_idle(busy); }
  void kv_evict(int session) {
    if (book_.evict(session)) ++kv_evictions_;
  }
  // ---- the session book (src/core/engine.hpp:380-426)
  int match_session(const std::vector<int>& prompt, const std::string& key, uint64_t scope = 0) const {
    return book_.match_session(prompt, key, scope);
  }
  int free_session(double protect_seconds, const std::vector<bool>& pinned) const { return book_.free_session(protect_seconds, pinned); }
  void activate_session(int i, const std::string& key, bool fresh, uint64_t scope = 0) {
    if (i < 0 || i >= sessions()) throw std::runtime_error("no such session");
    if (book_.activate(i, key, fresh, scope)) ++evictions_;
    active_ = i;
  }
  void touch_session(int i) { book_.touch(i); }
  int sessions_resident() const { return book_.resident(); }
  long session_evictions() const { return evictions_; }
  int max_batch() const { return opts_.max_seqs; }
  // What the prefill path would do for an admitted prompt (Engine::begin_prefill + prefill_chunk, engine.cpp:1747-1990): the
  // session keeps the positions it shares with the prompt, maps pages for the rest plus the growth reserve and takes the
  // prompt as its history.  The prefill pass itself is outside this build: `fill` stands in for it and leaves the KV of
  // positions [from, to) and the DeltaNet state of the slot on the device (synthetic in the tests and the benchmark); it
  // returns the first token.  Throws KvPoolExhausted with nothing changed when the pool is short.
  using PrefillFill = std::function<int(ling_b200_ctx*, int session, int from, int to)>;
  void set_prefill_fill(PrefillFill f) { prefill_fill_ = std::move(f); }
  int begin_prefill(int session, const std::vector<int>& prompt, uint64_t scope = 0) {
    Session& s = book_.at(session);
    const int L = static_cast<int>(prompt.size());
    const int reuse = book_.resume_reuse(session, prompt, scope, false);
    const int target = std::min(L + SessionBook::kKvGrowthPages * opts_.page_tokens, opts_.max_context);
    if (book_.kv_admit_need(session, prompt, scope) > book_.pool().free_pages()) book_.pool().retire();
    if (book_.kv_admit_need(session, prompt, scope) > book_.pool().free_pages()) throw KvPoolExhausted("KV page pool exhausted: prefill");
    book_.pool().truncate(s.table, book_.pool().pages_for(target) * opts_.page_tokens);
    kv_ensure(s, session, reuse, target);
    s.history = prompt;
    s.prompt_len = L;
    s.pos = L;
    s.turn_start = L;  // a prompt without message boundaries is bound again only when extended whole (engine.cpp:2276-2282)
    for (int k = L - 1; k >= 0; --k)
      if (prompt[size_t(k)] == opts_.boundary_token) {
        s.turn_start = k + 1;
        break;
      }
    return prefill_fill_ ? prefill_fill_(ctx_, session, reuse, L) : 0;
  }
  long kv_evictions() const { return kv_evictions_; }
  bool kv_retire(bool) {
    book_.pool().retire();  // the step has been fetched: no stream still reads a released page
    return book_.pool().pending_pages() == 0;
  }
  uint64_t state_hash() {
    uint64_t h = 0;
    ling_b200_state_hash(ctx_, active_, &h);
    return h;
  }

  // One step for each of several sessions in one pass (src/core/speculate.cpp:1101-1282).  Throws std::runtime_error on a
  // bad entry and KvPoolExhausted before anything is launched; a non-finite row fails only its sequence (SeqStep::error).
  void speculate_batch(std::span<SeqStep> seqs) {
    if (seqs.empty()) return;
    for (const SeqStep& q : seqs) {
      if (q.session < 0 || q.session >= sessions() || !q.params) throw std::runtime_error("speculate_batch: bad entry");
      if (!can_batch(q.session, *q.params)) throw std::runtime_error("speculate_batch: a sequence cannot join the batch");
      for (const SeqStep& o : seqs)
        if (&o != &q && o.session == q.session) throw std::runtime_error("speculate_batch: a session twice");
    }
    if (static_cast<int>(seqs.size()) > opts_.max_seqs) throw std::runtime_error("speculate_batch: more sequences than max_seqs");
    std::vector<DraftTree> trees;
    int need = 0;
    for (const SeqStep& q : seqs) {
      trees.push_back(tree_source_(q.session, q.anchor, book_.at(q.session).history));
      const Session& s = book_.at(q.session);
      need += book_.pool().needed(s.table, s.pos, s.pos + trees.back().rows());
    }
    if (need > book_.pool().free_pages()) book_.pool().retire();
    if (need > book_.pool().free_pages())
      throw KvPoolExhausted("KV page pool exhausted: the batch's step needs " + std::to_string(need) + " pages, " +
                            std::to_string(book_.pool().free_pages()) + " free");
    std::vector<ling_b200_seq_step> steps(seqs.size());
    std::vector<ling_b200_seq_result> res(seqs.size());
    bool logits = false;
    for (size_t i = 0; i < seqs.size(); ++i) {
      Session& s = book_.at(seqs[i].session);
      kv_ensure(s, seqs[i].session, s.pos, s.pos + trees[i].rows());
      steps[i] = ling_b200_seq_step{seqs[i].session, s.pos, 0, trees[i].rows(), trees[i].E, trees[i].token.data(),
                                    trees[i].parent.data(), nullptr};
      logits = logits || seqs[i].row_logits != nullptr;
    }
    const int flags = LING_B200_STEP_COMMIT | (logits ? LING_B200_STEP_KEEP_LOGITS : 0);
    if (ling_b200_verify_step(ctx_, steps.data(), static_cast<int>(steps.size()), flags, res.data()) != LING_B200_OK)
      throw std::runtime_error(std::string("speculate_batch: ") + ling_b200_last_error());
    for (size_t i = 0; i < seqs.size(); ++i) {
      Session& s = book_.at(seqs[i].session);
      if (res[i].status != LING_B200_SEQ_OK) {  // nothing committed; the session is reset (speculate.cpp:1266-1272)
        seqs[i].error = std::make_exception_ptr(NonFiniteLogits());
        seqs[i].out.clear();
        kv_evict(seqs[i].session);
        continue;
      }
      seqs[i].out.assign(res[i].out, res[i].out + res[i].n_out);
      for (int j = 0; j < res[i].n_path; ++j) s.history.push_back(trees[i].token[res[i].path[j]]);
      s.pos += res[i].n_path;
    }
    book_.pool().retire();
  }
  std::vector<int> speculate(int anchor, const SamplingParams& p, std::vector<float>* row_logits = nullptr) {
    SeqStep q;
    q.session = active_, q.anchor = anchor, q.params = &p, q.row_logits = row_logits;
    speculate_batch(std::span<SeqStep>(&q, 1));
    if (q.error) std::rethrow_exception(q.error);
    return q.out;
  }

 private:
  // kv_ensure (src/core/engine.cpp:841-869): pages for [from, to), copy-on-write copies made before the write, changed
  // table entries pushed to the device.
  void kv_ensure(Session& s, int slot, int from, int to) {
    const std::vector<int> before = s.table;
    std::vector<KvPool::Copy> copies;
    if (!book_.pool().ensure(s.table, from, to, &copies)) throw KvPoolExhausted("KV page pool exhausted");
    std::vector<int> src, dst, idx, val;
    for (const KvPool::Copy& c : copies) src.push_back(c.src), dst.push_back(c.dst);
    if (!src.empty()) ling_b200_kv_pages_copy(ctx_, src.data(), dst.data(), static_cast<int>(src.size()));
    for (size_t i = 0; i < s.table.size(); ++i)
      if (i >= before.size() || before[i] != s.table[i]) idx.push_back(static_cast<int>(i)), val.push_back(s.table[i]);
    if (!idx.empty()) ling_b200_kv_table_set(ctx_, slot, idx.data(), val.data(), static_cast<int>(idx.size()));
  }

  ModelConfig cfg_;
  EngineOptions opts_;
  ling_b200_ctx* ctx_ = nullptr;
  SessionBook book_;
  TreeSource tree_source_;
  PrefillFill prefill_fill_;
  long evictions_ = 0;
  int active_ = 0;
  long kv_evictions_ = 0;
};

namespace serve {

// ---- src/serve/pairing.hpp
inline constexpr long kFairWindow = 16;
struct PassWindow {
  std::deque<long> marks;
  void record(long pass) {
    marks.push_back(pass);
    trim(pass);
  }
  void trim(long now) {
    while (!marks.empty() && marks.front() <= now - kFairWindow) marks.pop_front();
  }
  long last() const { return marks.empty() ? 0 : marks.back(); }
  int count(long now) const {
    return static_cast<int>(std::count_if(marks.begin(), marks.end(), [&](long m) { return m > now - kFairWindow; }));
  }
};
struct PairCandidate {
  bool batchable = false;
  int recent = 0;
  long last = 0;
};
namespace detail {
inline void split(const std::vector<PairCandidate>& c, std::vector<int>& b, std::vector<int>& r, std::vector<long>& l) {
  for (const PairCandidate& x : c) b.push_back(x.batchable), r.push_back(x.recent), l.push_back(x.last);
}
}  // namespace detail
inline std::vector<size_t> pair_order(const std::vector<PairCandidate>& c, bool fair) {
  std::vector<int> b, r, o(c.size());
  std::vector<long> l;
  detail::split(c, b, r, l);
  ling_b200_pair_order(b.data(), r.data(), l.data(), static_cast<int>(c.size()), fair, o.data());
  return std::vector<size_t>(o.begin(), o.end());
}
inline std::vector<size_t> select_batch(const std::vector<PairCandidate>& c, size_t self, int fit, bool fair) {
  std::vector<int> b, r, o(c.size());
  std::vector<long> l;
  detail::split(c, b, r, l);
  const int n = ling_b200_select_batch(b.data(), r.data(), l.data(), static_cast<int>(c.size()), static_cast<int>(self), fit, fair, o.data());
  return std::vector<size_t>(o.begin(), o.begin() + n);
}

// ---- src/serve/kv_policy.hpp
struct KvPoolView {
  int free = 0, pending = 0, idle = 0;
};
enum class KvVerdict { Go, Retire, Reclaim, Wait };
inline KvVerdict kv_verdict(int need, const KvPoolView& v) {
  return static_cast<KvVerdict>(ling_b200_kv_verdict(need, v.free, v.pending, v.idle));
}
struct KvRunner {
  long admitted = 0;
  bool waiting = false;
  int need = 0;
};
inline int kv_last_resort(const std::vector<KvRunner>& running, const KvPoolView& v) {
  std::vector<long> a;
  std::vector<int> w, n;
  for (const KvRunner& r : running) a.push_back(r.admitted), w.push_back(r.waiting), n.push_back(r.need);
  return ling_b200_kv_last_resort(a.data(), w.data(), n.data(), static_cast<int>(running.size()), v.free, v.pending, v.idle);
}

// kv_reclaim (src/serve/kv_policy.hpp:58-72): the reference's signature; the closures travel behind one user pointer.
using KvEvictNext = std::function<bool()>;
inline bool kv_reclaim(const std::function<int()>& need, const std::function<int()>& have, const std::vector<KvEvictNext>& kept,
                       int need_kept, int reach_kept, const std::vector<KvEvictNext>& source, int need_all, int reach_all, bool must) {
  struct Calls {
    const std::function<int()>*need, *have;
    const std::vector<KvEvictNext>*kept, *source;
  } calls{&need, &have, &kept, &source};
  return ling_b200_kv_reclaim(
             [](void* u) { return (*static_cast<Calls*>(u)->need)(); }, [](void* u) { return (*static_cast<Calls*>(u)->have)(); },
             [](void* u, int g) {
               const Calls& c = *static_cast<Calls*>(u);
               const size_t nk = c.kept->size();
               return int(size_t(g) < nk ? (*c.kept)[size_t(g)]() : (*c.source)[size_t(g) - nk]());
             },
             &calls, static_cast<int>(kept.size()), need_kept, reach_kept, static_cast<int>(source.size()), need_all, reach_all,
             must) != 0;
}

// ---- src/serve/admission.hpp
// refuse_request (admission.hpp:312-319): the 503 text while the host is below the admission reserve; empty: may run.
inline std::string refuse_request(long avail_mb, long reserve_mb) {
  std::string buf(256, '\0');
  const int n = ling_b200_refuse_request(avail_mb, reserve_mb, buf.data(), static_cast<int>(buf.size()));
  buf.resize(n > 0 ? size_t(n) : 0);
  return buf;
}
struct MemoryPlan : ling_b200_memory_plan {};
struct KvPlanInputs {
  bool on = false;
  size_t store_bytes = 0;
  long pool_mb = -1;
  int page_tokens = 64, kv_elem_bytes = 2;  // the reference's constants; 16 or 64 / 1 for the FP8 pool
};
struct StartPlan {
  MemoryPlan plan;
  bool refused = false;
};
inline StartPlan start_plan(const ModelConfig& c, size_t weight_bytes, size_t scratch, bool drafter, int sessions, int max_context,
                            long avail_mb, long reserve_mb, const KvPlanInputs& kv = {}) {
  StartPlan s;
  ling_b200_start_plan(&c, weight_bytes, scratch, drafter, sessions, max_context, avail_mb, reserve_mb, kv.on, kv.store_bytes,
                       kv.pool_mb, kv.page_tokens, kv.kv_elem_bytes, &s.plan);
  s.refused = s.plan.refused != 0;
  return s;
}

// ---- src/serve/step_trace.hpp
struct StepCandidate {
  int session = 0;
  long request = 0;
  int state = 0, recent = 0;
  long last = 0;
};
struct StepRecord {
  double t = 0;
  long pass = 0;
  const char* kind = "decode";
  size_t turn = 0;
  std::vector<int> sessions, rows, tokens, left;
  std::vector<StepCandidate> cand;
  double ms = 0;
  bool side = false;
};
inline std::string format_step(const StepRecord& s) {
  std::vector<int> c;
  std::vector<long> req, last;
  for (const StepCandidate& x : s.cand) c.insert(c.end(), {x.session, x.state, x.recent}), req.push_back(x.request), last.push_back(x.last);
  std::string buf(4096 + 64 * (s.sessions.size() + s.cand.size()), '\0');
  const int n = ling_b200_format_step(s.t, s.pass, s.kind, s.turn, s.sessions.data(), s.rows.data(), s.tokens.data(), s.left.data(),
                                      static_cast<int>(s.sessions.size()), c.data(), req.data(), last.data(),
                                      static_cast<int>(s.cand.size()), s.ms, s.side, buf.data(), static_cast<int>(buf.size()));
  buf.resize(n > 0 ? n : 0);
  return buf;
}

}  // namespace serve
}  // namespace ling
