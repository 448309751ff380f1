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
#include <utility>
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

// ---- src/core/prefix_kv.hpp
class ArenaAlloc {
 public:
  ArenaAlloc(size_t size, size_t align) : a_(ling_b200_arena_create(size, align)) {}
  ~ArenaAlloc() { ling_b200_arena_destroy(a_); }
  ArenaAlloc(const ArenaAlloc&) = delete;
  ArenaAlloc& operator=(const ArenaAlloc&) = delete;
  bool alloc(size_t bytes, size_t* offset) {  // false: no free range is large enough
    const long long at = ling_b200_arena_alloc(a_, bytes);
    if (at < 0) return false;
    *offset = static_cast<size_t>(at);
    return true;
  }
  void release(size_t offset) { ling_b200_arena_release(a_, offset); }
  size_t size() const { return ling_b200_arena_size(a_); }
  size_t in_use() const { return ling_b200_arena_in_use(a_); }

 private:
  ling_b200_arena* a_;
};

// The prefix KV store's tree, always in the reference's paged mode (prefix_kv.hpp:12-18): nodes hold references to pool
// pages, the budget covers the saved states.  The buffer mode's members (Ops::store, segments, buffers) have no counterpart.
class PrefixKvTree {
 public:
  struct Ops {
    std::function<void*(size_t bytes)> alloc;  // storage for one state, or nullptr
    std::function<void(void* p)> release;
    std::function<std::vector<int>(int from, int to)> hold;
    std::function<void(int page)> retain;
    std::function<void(int page)> drop;
  };
  struct Match {
    int len = 0;
    std::vector<int> path;
  };
  PrefixKvTree(size_t budget_bytes, size_t /*bytes_per_token: the KV is the pool's*/, size_t state_bytes, Ops ops, int page_tokens = 64)
      : ops_(std::move(ops)), page_tokens_(page_tokens) {
    ling_b200_prefix_ops c{this, &hold_cb, &retain_cb, &drop_cb, &alloc_cb, &release_cb};
    if (ops_.hold && ops_.retain && ops_.drop && ops_.alloc && ops_.release)
      t_ = ling_b200_prefix_create(budget_bytes, state_bytes, page_tokens, &c);
    if (!t_) throw std::invalid_argument("PrefixKvTree: hold, retain, drop, alloc and release are all needed");
  }
  ~PrefixKvTree() { ling_b200_prefix_destroy(t_); }
  PrefixKvTree(const PrefixKvTree&) = delete;
  PrefixKvTree& operator=(const PrefixKvTree&) = delete;

  Match match(const std::vector<int>& prompt, uint64_t scope = 0) const {
    Match m;
    int n = 0;
    m.path.resize(prompt.size() + 1);
    m.len = ling_b200_prefix_match(t_, prompt.data(), static_cast<int>(prompt.size()), scope, m.path.data(),
                                   static_cast<int>(m.path.size()), &n);
    m.path.resize(size_t(n));
    return m;
  }
  int best_state(const Match& m, int limit, const void** state) const {
    void* st = nullptr;
    const int pos = ling_b200_prefix_best_state(t_, m.path.data(), static_cast<int>(m.path.size()), m.len, limit, &st);
    *state = st;
    return pos;
  }
  std::vector<int> pages(const Match& m, int n) const {
    std::vector<int> out(size_t((std::max(n, 0) + page_tokens_ - 1) / page_tokens_) + 1);
    const int c = ling_b200_prefix_pages(t_, m.path.data(), static_cast<int>(m.path.size()), n, out.data(), static_cast<int>(out.size()));
    out.resize(size_t(std::max(c, 0)));
    return out;
  }
  void touch(const Match& m, uint64_t epoch) { ling_b200_prefix_touch(t_, m.path.data(), static_cast<int>(m.path.size()), epoch); }
  std::vector<std::pair<int, int>> insert(const std::vector<int>& prompt, int q, const std::vector<int>& cuts, uint64_t epoch,
                                          uint64_t scope = 0) {
    std::vector<int> node(cuts.size() + 1), pos(cuts.size() + 1);
    const int n = ling_b200_prefix_insert(t_, prompt.data(), static_cast<int>(prompt.size()), q, cuts.data(), static_cast<int>(cuts.size()),
                                          epoch, scope, node.data(), pos.data(), static_cast<int>(node.size()));
    std::vector<std::pair<int, int>> want;
    for (int i = 0; i < std::min(n, static_cast<int>(node.size())); ++i) want.push_back({node[size_t(i)], pos[size_t(i)]});
    return want;
  }
  void* add_state(int node, uint64_t epoch) { return ling_b200_prefix_add_state(t_, node, epoch); }
  bool evict_lru_leaf(const std::vector<int>& keep = {}) {
    return ling_b200_prefix_evict_lru_leaf(t_, keep.data(), static_cast<int>(keep.size())) != 0;
  }
  void clear() { ling_b200_prefix_clear(t_); }
  size_t bytes() const { return ling_b200_prefix_bytes(t_); }
  size_t budget() const { return ling_b200_prefix_budget(t_); }
  int nodes() const { return ling_b200_prefix_nodes(t_); }
  int states() const { return ling_b200_prefix_states(t_); }
  bool paged() const { return true; }
  int pages_held() const { return ling_b200_prefix_pages_held(t_); }
  std::vector<std::vector<int>> page_lists(const std::vector<int>& skip = {}) const {
    std::vector<int> pages(size_t(std::max(pages_held(), 1))), lens(size_t(std::max(nodes(), 1)));
    const int n = ling_b200_prefix_page_lists(t_, skip.data(), static_cast<int>(skip.size()), pages.data(), static_cast<int>(pages.size()),
                                              lens.data(), static_cast<int>(lens.size()));
    std::vector<std::vector<int>> out;
    size_t at = 0;
    for (int i = 0; i < n; ++i) {
      out.emplace_back(pages.begin() + static_cast<long>(at), pages.begin() + static_cast<long>(at) + lens[size_t(i)]);
      at += size_t(lens[size_t(i)]);
    }
    return out;
  }

 private:
  static PrefixKvTree& self(void* u) { return *static_cast<PrefixKvTree*>(u); }
  static int hold_cb(void* u, int from, int to, int* pages, int cap) {
    const std::vector<int> ids = self(u).ops_.hold(from, to);
    for (size_t i = 0; i < ids.size(); ++i) {
      if (static_cast<int>(i) < cap) pages[i] = ids[i];
      else if (ids[i] != 0) self(u).ops_.drop(ids[i]);  // more than the range's pages: nothing may leak
    }
    return static_cast<int>(ids.size());
  }
  static void retain_cb(void* u, int page) { self(u).ops_.retain(page); }
  static void drop_cb(void* u, int page) { self(u).ops_.drop(page); }
  static void* alloc_cb(void* u, size_t bytes) { return self(u).ops_.alloc(bytes); }
  static void release_cb(void* u, void* p) { self(u).ops_.release(p); }

  Ops ops_;
  int page_tokens_;
  ling_b200_prefix* t_ = nullptr;
};

// ---- src/core/model.hpp, src/core/engine.hpp
using ModelConfig = ling_b200_model_config;
// The resident sessions and their KV pages as the scheduler sees them (the host-side half of Engine's session functions,
// src/core/engine.cpp:581-648,724-800,881-912, and of its Session struct, engine.hpp:760-800).  No device work: Engine
// keeps one and adds the device side and the prefix KV store; a scheduler test can keep one alone.  The book itself knows
// no store and no donor sessions: its kv_admit_need is the plan of a prompt that resumes from its own session only.
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
  // engine.cpp:1747-1842).  A recurrent state cannot be wound back, so a prompt resumes only from a position whose state is
  // kept.  The reference keeps a snapshot at the end of the session's last prompt; here the kept state is the session's
  // live one, after exactly its history (every pass of this build is the same verify pass, so the state does not depend on
  // how it was reached): a prompt that extends the whole history by at least one token resumes at the history's end,
  // any other prompt from nothing (or, in Engine, from the prefix KV store).
  int resume_reuse(int session, const std::vector<int>& prompt, uint64_t scope, bool from_scratch) const {
    const Session& s = at(session);
    if (from_scratch || s.scope != scope || prompt.size() <= s.history.size()) return 0;
    return common_prefix(s.history, prompt) == static_cast<int>(s.history.size()) ? static_cast<int>(s.history.size()) : 0;
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
  int prefix_kv_mb = 0;     // the prefix KV store's budget for saved states (engine.hpp:97-103; 4096 there); 0: no store
  int checkpoint_limit = 32768;  // no state is kept past this position (engine.hpp:87)
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
    if (opts.prefix_kv_mb > 0) {
      // Sessions that resume from the store share pages, so a pass's sequences can hold more context between them than the
      // pool has positions: the attention's partial buffers are sized for twice the pool (at most every sequence at the limit).
      const long long pool = 1LL * o.pool_pages * opts.page_tokens, all = 1LL * opts.max_seqs * opts.max_context;
      o.attn_positions = static_cast<int>(std::min<long long>(std::min(2 * pool, all), 2000000000LL));
    }
    if (ling_b200_create(&cfg_, &o, &ctx_) != LING_B200_OK) {
      const std::string why = ling_b200_last_error();
      ling_b200_destroy(ctx_);
      throw std::runtime_error("Engine: " + why);
    }
    if (opts_.prefix_kv_mb > 0) kv_store_setup();
  }
  ~Engine() {
    kv_tree_.reset();  // drops its page references while the pool is still there
    ling_b200_destroy(ctx_);
  }
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
    if (prompt.empty()) return 0;
    return kv_resume_need(session, plan_resume(session, prompt, scope, from_scratch), prompt);
  }
  int kv_session_pages(int session) const { return book_.kv_reclaimable({session}); }
  int kv_reclaimable(const std::vector<int>& sessions) const { return book_.kv_reclaimable(sessions); }
  // ---- the prefix KV store as the scheduler sees it (src/core/engine.hpp:444-460; engine.cpp:761-768)
  bool kv_store_on() const { return static_cast<bool>(kv_tree_); }
  const PrefixKvTree* kv_store() const { return kv_tree_.get(); }
  // The pages freed once the listed sessions and, with `store`, the store's nodes other than `store_keep` are gone: a page
  // several of them hold counts when all its holders are among them (engine.cpp:741-759).
  int kv_reclaimable(const std::vector<int>& sessions, bool store, const std::vector<int>& store_keep = {}) const {
    std::vector<std::vector<int>> lists;
    if (store && kv_tree_) lists = kv_tree_->page_lists(store_keep);
    KvPool::Refs refs;
    for (int i : sessions) refs.push_back(&book_.at(i).table);
    for (const std::vector<int>& l : lists) refs.push_back(&l);
    return book_.pool().reclaimable(refs);
  }
  // The pages that evicting the whole store would free.
  int kv_store_pages() const { return kv_reclaimable({}, true); }
  // Evicts the store's least recently used leaf outside `keep` (the path an admitted prompt resumes from).
  bool kv_store_evict(const std::vector<int>& keep = {}) { return kv_tree_ && kv_tree_->evict_lru_leaf(keep); }
  // The store nodes a prompt admitted into `session` would resume from (empty: it resumes elsewhere or from nothing).
  std::vector<int> kv_store_path(int session, const std::vector<int>& prompt, uint64_t scope) const {
    const ResumePlan plan = plan_resume(session, prompt, scope, false);
    return plan.from_kv ? plan.kvm.path : std::vector<int>{};
  }
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
  // The attention kernels' partial-result slots a session's next step takes, and how many a pass has (a scheduler counts them
  // when it picks a pass's partners: shared pages let the pass's contexts exceed the pool).
  int attn_slot_need(int session) const { return ling_b200_attn_slot_need(ctx_, book_.at(session).pos); }
  int attn_slot_capacity() const { return ling_b200_attn_slot_capacity(ctx_); }
  // What the prefill path does for an admitted prompt (Engine::begin_prefill + prefill_chunk, engine.cpp:1886-2300): the
  // prompt resumes from the furthest kept state (the session's own, or one of the prefix KV store's, whose pages are then
  // mapped by reference), pages are taken for the rest plus the growth reserve, the rest is processed in pieces that end
  // at the positions the store will keep a state at, and the prompt's shareable beginning goes into the store.
  // The pass that processes a piece is `fill`: it leaves the KV of positions [from, to) and the recurrent state after
  // `to` on the device and returns the token after `to`.  The reference's prefill pass is outside this build; the fill is
  // either chain_prefill below (the verify pass over linear chains, the real model) or a synthetic stand-in a test or
  // benchmark sets.  Throws KvPoolExhausted with nothing changed when the pool is short.
  using PrefillFill = std::function<int(ling_b200_ctx*, int session, int from, int to)>;
  void set_prefill_fill(PrefillFill f) { prefill_fill_ = std::move(f); }
  void use_chain_prefill() {
    prefill_fill_ = [this](ling_b200_ctx*, int session, int from, int to) { return chain_prefill(session, from, to); };
  }
  struct PrefillStats {  // src/core/engine.hpp:190-200, the fields this path has
    int reused_tokens = 0, store_tokens = 0, prefill_tokens = 0, chunks = 0;
  };
  const PrefillStats& last_prefill() const { return last_prefill_; }
  static constexpr int kResumeAlign = 32;  // kept states sit at multiples of this (engine.hpp:533)

  int begin_prefill(int session, const std::vector<int>& prompt, uint64_t scope = 0, bool from_scratch = false) {
    if (prompt.empty()) throw std::runtime_error("empty prompt");
    Session& s = book_.at(session);
    const int L = static_cast<int>(prompt.size());
    const ResumePlan plan = plan_resume(session, prompt, scope, from_scratch);
    const int reuse = plan.reuse;
    const int target = std::min(L + SessionBook::kKvGrowthPages * opts_.page_tokens, opts_.max_context);
    if (kv_resume_need(session, plan, prompt) > book_.pool().free_pages()) book_.pool().retire();
    if (kv_resume_need(session, plan, prompt) > book_.pool().free_pages()) throw KvPoolExhausted("KV page pool exhausted: prefill");
    const uint64_t epoch = ++kv_epoch_;
    if (kv_tree_ && !from_scratch) kv_tree_->touch(plan.kvm, epoch);
    last_prefill_ = PrefillStats{};
    last_prefill_.reused_tokens = reuse, last_prefill_.prefill_tokens = L - reuse;
    const std::vector<int> before = s.table;
    if (plan.from_kv) {
      // The store's pages for [0, reuse) mapped by reference, no copy (kv_restore, engine.cpp:1095-1104); the partly used
      // last one is copied by kv_ensure below before this session writes into it.
      book_.pool().share(s.table, kv_tree_->pages(plan.kvm, reuse), reuse);
      if (ling_b200_state_restore(ctx_, session, state_offset(plan.kv_state)) != LING_B200_OK)
        throw std::runtime_error(std::string("begin_prefill: ") + ling_b200_last_error());
      last_prefill_.store_tokens = reuse;
    } else if (reuse == 0) {
      ling_b200_state_reset(ctx_, session);
    }
    // Pages past the target go back; shared pages past the resume point are let go (fresh ones are taken instead of
    // copies of what is overwritten anyway); the page `reuse` falls in is copied if it is shared (engine.cpp:1997-2010).
    book_.pool().truncate(s.table, book_.pool().pages_for(target) * opts_.page_tokens);
    book_.pool().unshare(s.table, reuse);
    table_sync(s, session, before);
    kv_ensure(s, session, reuse, target);
    s.history = prompt;
    s.scope = scope;
    s.pos = reuse;
    // Piece ends: the store's cuts past the resume point, then the prompt's end.  Each cut's state is saved when its piece ends.
    const std::vector<int> cuts = kv_tree_ ? kv_store_cuts(prompt, plan.branch_at) : std::vector<int>{};
    std::vector<std::pair<int, size_t>> kept;  // (position, arena offset) of the states saved on the way
    int first = 0, from = reuse;
    auto piece = [&](int to) {
      if (to <= from) return;
      first = prefill_fill_ ? prefill_fill_(ctx_, session, from, to) : 0;
      ++last_prefill_.chunks;
      s.pos = from = to;
    };
    for (int c : cuts) {
      if (c <= reuse || c >= L) continue;
      piece(c);
      size_t off = 0;
      if (kv_arena_->alloc(state_unit_, &off)) {
        if (ling_b200_state_save(ctx_, session, off) == LING_B200_OK) kept.push_back({c, off});
        else kv_arena_->release(off);
      }
    }
    piece(L);
    s.prompt_len = L;
    s.turn_start = L;  // a prompt without message boundaries is bound again only when extended whole (engine.cpp:2276-2282)
    for (int k = L - 1; k >= 0; --k)
      if (prompt[size_t(k)] == opts_.boundary_token) {
        s.turn_start = k + 1;
        break;
      }
    if (kv_tree_ && !cuts.empty()) kv_insert(session, prompt, cuts, epoch, scope, kept);
    for (const auto& k : kept) kv_arena_->release(k.second);  // the states no node took
    return first;
  }

  // The verify pass as a prefill pass: positions [from, to) of the session's history as linear chains of at most
  // kResumeAlign rows, each ending at a multiple of kResumeAlign, every row accepted (the next chain token imposed as
  // the row's argmax) and committed; the last row's own argmax is the token after `to`.  A prompt resumed at a kept state
  // runs the same passes over the same positions as one prefilled from nothing, so it reaches the same bits.
  int chain_prefill(int session, int from, int to) {
    const Session& s = book_.at(session);
    if (from < 0 || to > static_cast<int>(s.history.size())) throw std::runtime_error("chain_prefill: positions outside the history");
    int next = 0;
    for (int at = from; at < to;) {
      const int end = std::min(to, at - at % kResumeAlign + kResumeAlign), n = end - at;
      const std::vector<int> tok(s.history.begin() + at, s.history.begin() + end);
      std::vector<int> par(static_cast<size_t>(n), 0), force(static_cast<size_t>(n), -1);
      for (int i = 0; i < n; ++i) par[size_t(i)] = i - 1;
      for (int i = 0; i + 1 < n; ++i) force[size_t(i)] = tok[size_t(i) + 1];
      ling_b200_seq_step step{session, at, 0, n, n - 1, tok.data(), par.data(), force.data()};
      ling_b200_seq_result res{};
      if (ling_b200_verify_step(ctx_, &step, 1, LING_B200_STEP_COMMIT, &res) != LING_B200_OK)
        throw std::runtime_error(std::string("chain_prefill: ") + ling_b200_last_error());
      if (res.status != LING_B200_SEQ_OK) throw NonFiniteLogits();
      if (res.n_path != n) throw std::logic_error("chain_prefill: a chain row was not accepted");
      next = res.next_token;
      at = end;
    }
    return next;
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
    std::vector<int> src, dst;
    for (const KvPool::Copy& c : copies) src.push_back(c.src), dst.push_back(c.dst);
    if (!src.empty()) ling_b200_kv_pages_copy(ctx_, src.data(), dst.data(), static_cast<int>(src.size()));
    table_sync(s, slot, before);
  }

  void table_sync(const Session& s, int slot, const std::vector<int>& before) {
    std::vector<int> idx, val;
    for (size_t i = 0; i < std::max(s.table.size(), before.size()); ++i) {
      const int now = i < s.table.size() ? s.table[i] : 0, was = i < before.size() ? before[i] : 0;
      if (now != was) idx.push_back(static_cast<int>(i)), val.push_back(now);
    }
    if (!idx.empty()) ling_b200_kv_table_set(ctx_, slot, idx.data(), val.data(), static_cast<int>(idx.size()));
  }

  // ---- the prefix KV store (engine.cpp:380-425,1095-1122,1747-1884)
  // Where a prompt resumes: the furthest kept state inside what it shares with the session's own history or with the store.
  struct ResumePlan {
    int reuse = 0;
    bool from_kv = false;
    PrefixKvTree::Match kvm;
    const void* kv_state = nullptr;
    int branch_at = 0;  // where the prompt leaves the longest prefix it shares with another conversation, aligned
  };
  ResumePlan plan_resume(int session, const std::vector<int>& prompt, uint64_t scope, bool from_scratch) const {
    ResumePlan plan;
    const int L = static_cast<int>(prompt.size());
    const int own = book_.resume_reuse(session, prompt, scope, from_scratch);
    int kv_reuse = 0;
    if (kv_tree_ && !from_scratch) {
      plan.kvm = kv_tree_->match(prompt, scope);
      kv_reuse = kv_tree_->best_state(plan.kvm, std::min(plan.kvm.len, L - 1), &plan.kv_state);
    }
    plan.from_kv = kv_reuse > own;
    plan.reuse = plan.from_kv ? kv_reuse : own;
    if (kv_tree_) {
      const Session& self = book_.at(session);
      for (int i = 0; i < book_.sessions(); ++i) {
        const Session& o = book_.at(i);
        if (o.history.empty() || o.scope != scope) continue;
        const int l = SessionBook::common_prefix(o.history, prompt);
        if (&o == &self && o.prompt_len > 0 && l >= o.turn_start) continue;  // its own next turn: its own state covers that
        plan.branch_at = std::max(plan.branch_at, l);
      }
      plan.branch_at = std::max(plan.branch_at, plan.kvm.len);
      plan.branch_at -= plan.branch_at % kResumeAlign;
    }
    return plan;
  }
  // The pages the admission takes beyond the free ones it may count on (kv_resume_need, engine.cpp:1844-1868).
  int kv_resume_need(int session, const ResumePlan& plan, const std::vector<int>& prompt) const {
    const int L = static_cast<int>(prompt.size()), pages = book_.kv_admit_pages(prompt.size());
    std::vector<int> donor;
    if (plan.from_kv) donor = kv_tree_->pages(plan.kvm, plan.reuse);
    int need = book_.pool().resume_need(book_.at(session).table, plan.reuse, pages, plan.from_kv ? &donor : nullptr);
    // The store's hold reaches up to its last cut: when that cut lies in the page position L is in, the store shares the page
    // the first decode step writes, which copies it first: one page more.
    if (kv_tree_ && L < opts_.max_context && pages < book_.pool().capacity()) {
      const std::vector<int> cuts = kv_store_cuts(prompt, plan.branch_at);
      if (!cuts.empty() && book_.pool().index_of(cuts.back() - 1) == book_.pool().index_of(L)) need += 1;
    }
    return need;
  }
  // The positions a prefill of `prompt` adds to the store with a state each (kv_store_cuts, engine.cpp:1870-1884): the end
  // of each of its first two messages and its branch point, below its end and checkpoint_limit, at multiples of kResumeAlign.
  std::vector<int> kv_store_cuts(const std::vector<int>& prompt, int branch_at) const {
    const int L = static_cast<int>(prompt.size());
    std::vector<int> cuts;
    for (int i = 0, messages = 0; i < L && messages < 2; ++i)
      if (prompt[size_t(i)] == opts_.boundary_token) {
        const int c = i + 1 - (i + 1) % kResumeAlign;
        if (c > 0) cuts.push_back(c);
        ++messages;
      }
    if (branch_at > 0) cuts.push_back(branch_at);
    std::erase_if(cuts, [&](int c) { return c >= L || c > opts_.checkpoint_limit; });
    std::sort(cuts.begin(), cuts.end());
    cuts.erase(std::unique(cuts.begin(), cuts.end()), cuts.end());
    return cuts;
  }
  // A saved state is named by its arena offset + 1, so that offset 0 is not a null pointer.
  static void* state_token(size_t offset) { return reinterpret_cast<void*>(offset + 1); }
  static size_t state_offset(const void* token) { return reinterpret_cast<size_t>(token) - 1; }
  static constexpr int kSpareStates = 3;  // states saved during a prefill before the tree takes them: two message ends and a branch point
  void kv_store_setup() {
    const size_t bytes = ling_b200_state_bytes(ctx_);
    state_unit_ = (bytes + 255) / 256 * 256;
    const size_t states = (size_t(opts_.prefix_kv_mb) << 20) / state_unit_;
    kv_arena_ = std::make_unique<ArenaAlloc>((states + kSpareStates) * state_unit_, 256);
    if (ling_b200_state_arena_reserve(ctx_, kv_arena_->size()) != LING_B200_OK)
      throw std::runtime_error(std::string("Engine: prefix KV store: ") + ling_b200_last_error());
    PrefixKvTree::Ops ops;
    ops.alloc = [this](size_t n) -> void* {
      if (handoff_) return std::exchange(handoff_, nullptr);  // a state this prefill already saved becomes the node's
      size_t off = 0;
      return kv_arena_->alloc(n, &off) ? state_token(off) : nullptr;
    };
    ops.release = [this](void* p) { kv_arena_->release(state_offset(p)); };
    ops.hold = [this](int from, int to) -> std::vector<int> {
      const std::vector<int>& table = book_.at(hold_session_).table;
      const int a = book_.pool().index_of(from), b = book_.pool().index_of(to - 1);
      if (b >= static_cast<int>(table.size())) return {};
      for (int j = a; j <= b; ++j)
        if (table[size_t(j)] == 0) return {};
      for (int j = a; j <= b; ++j) book_.pool().retain(table[size_t(j)]);
      return std::vector<int>(table.begin() + a, table.begin() + b + 1);
    };
    ops.retain = [this](int page) { book_.pool().retain(page); };
    ops.drop = [this](int page) { book_.pool().release(page); };
    kv_tree_ = std::make_unique<PrefixKvTree>(states * state_unit_, 0, state_unit_, std::move(ops), opts_.page_tokens);
  }
  // The prompt's shareable beginning (up to its last cut) into the store: new nodes hold the session's pages, and each cut's
  // state saved during this prefill becomes its node's (kv_insert, engine.cpp:1108-1122).
  void kv_insert(int session, const std::vector<int>& prompt, const std::vector<int>& cuts, uint64_t epoch, uint64_t scope,
                 std::vector<std::pair<int, size_t>>& kept) {
    hold_session_ = session;
    for (const auto& [node, pos] : kv_tree_->insert(prompt, cuts.back(), cuts, epoch, scope)) {
      const auto k = std::find_if(kept.begin(), kept.end(), [&](const auto& e) { return e.first == pos; });
      if (k == kept.end()) continue;
      handoff_ = state_token(k->second);
      if (kv_tree_->add_state(node, epoch)) kept.erase(k);
      handoff_ = nullptr;
    }
  }

  ModelConfig cfg_;
  EngineOptions opts_;
  ling_b200_ctx* ctx_ = nullptr;
  SessionBook book_;
  std::unique_ptr<ArenaAlloc> kv_arena_;
  std::unique_ptr<PrefixKvTree> kv_tree_;
  size_t state_unit_ = 0;
  void* handoff_ = nullptr;
  int hold_session_ = 0;
  uint64_t kv_epoch_ = 0;
  PrefillStats last_prefill_;
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
