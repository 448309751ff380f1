// ref_shim.cpp -- C wrappers around the REFERENCE's own host sources, compiled where they lie into
// oracle/_ref/libling_ref.so (see oracle/Makefile).  TEST INFRASTRUCTURE ONLY.  Nothing of the reference is copied
// into this repository: this file only includes the reference's headers and calls its functions, so that the oracle
// and the product's host logic can be compared with the real thing (tree description, greedy acceptance, context
// lookup, tree building, the KV page pool's bookkeeping, pairing, pool policy, admission arithmetic, trace line, the prefix KV
// store's tree in its paged mode and its arena).
#include <cstring>
#include <optional>
#include <vector>

#include "core/kv_pool.hpp"
#include "core/lookup.hpp"
#include "core/prefix_kv.hpp"
#include "core/tree.hpp"
#include "serve/admission.hpp"
#include "serve/kv_policy.hpp"
#include "serve/pairing.hpp"
#include "serve/step_trace.hpp"

namespace {
ling::DraftTree make_tree(const int* parent, const int* token, int n, int chain) {
  ling::DraftTree t;
  t.E = chain;
  t.parent.assign(parent, parent + n);
  t.parent[0] = -1;
  t.token.resize(n);
  t.pick.assign(n, 0);
  t.depth.assign(n, 0);
  t.children.assign(n, {});
  for (int r = 0; r < n; ++r) {
    t.token[r] = token ? token[r] : 0;
    if (r > 0) {
      t.depth[r] = t.depth[parent[r]] + 1;
      t.children[parent[r]].push_back(r);
    }
  }
  return t;
}
ling::ModelConfig make_config(const int* c, const unsigned char* full) {
  // c: hidden, intermediate, layers, vocab, heads, kv_heads, head_dim, rotary_dim, lin_k_heads, lin_v_heads,
  //    lin_k_dim, lin_v_dim, conv_kernel
  ling::ModelConfig m;
  m.hidden = c[0], m.intermediate = c[1], m.layers = c[2], m.vocab = c[3], m.heads = c[4], m.kv_heads = c[5];
  m.head_dim = c[6], m.rotary_dim = c[7], m.lin_k_heads = c[8], m.lin_v_heads = c[9], m.lin_k_dim = c[10];
  m.lin_v_dim = c[11], m.conv_kernel = c[12];
  m.full_attention.resize(m.layers);
  for (int l = 0; l < m.layers; ++l) m.full_attention[l] = full[l] != 0;
  return m;
}
}  // namespace

extern "C" {

int ref_tree_desc_bytes() { return int(sizeof(ling::kernels::TreeDesc)); }

int ref_describe_tree(const int* parent, int n, int chain, void* out) {
  try {
    ling::kernels::TreeDesc d;
    ling::describe_tree(make_tree(parent, nullptr, n, chain), d);
    std::memcpy(out, &d, sizeof d);
    return 0;
  } catch (...) {
    return 1;
  }
}

int ref_accept_tree_greedy(const int* parent, const int* token, int n, const int* argmax, int* path, int* next) {
  const std::vector<int> p = ling::accept_tree_greedy(make_tree(parent, token, n, 0), argmax, *next);
  std::copy(p.begin(), p.end(), path);
  return int(p.size());
}

int ref_lookup_propose(const int* seq, int len, int max, int ngram, int* out, int* match) {
  const ling::LookupProposal p = ling::lookup_propose(std::vector<int>(seq, seq + len), max, ngram);
  std::copy(p.tokens.begin(), p.tokens.end(), out);
  *match = p.match;
  return int(p.tokens.size());
}

int ref_build_tree(int anchor, const int* cand, const float* scores, int E, int K16, const int* chain_tokens,
                   const int* chain_picks, int nodes, double temp, int width, int max_depth, int chain, int* parent,
                   int* depth, int* token, int* pick, double* extra_mass) {
  ling::TreeShape sh;
  sh.nodes = nodes, sh.temp = temp, sh.width = width, sh.max_depth = max_depth, sh.chain = chain;
  const ling::DraftTree t = ling::build_tree(anchor, cand, scores, E, K16, std::vector<int>(chain_tokens, chain_tokens + E),
                                             std::vector<int>(chain_picks, chain_picks + E), sh);
  for (int r = 0; r < t.rows(); ++r) parent[r] = t.parent[r], depth[r] = t.depth[r], token[r] = t.token[r], pick[r] = t.pick[r];
  *extra_mass = t.extra_mass;
  return t.rows() | (t.E << 16);
}

// ---- KvPool (64-position pages, the reference's compile-time constant)
void* ref_kvpool_create(int pages) { return new ling::KvPool(pages); }
void ref_kvpool_destroy(void* p) { delete static_cast<ling::KvPool*>(p); }
int ref_kvpool_capacity(void* p) { return static_cast<ling::KvPool*>(p)->capacity(); }
int ref_kvpool_free_pages(void* p) { return static_cast<ling::KvPool*>(p)->free_pages(); }
int ref_kvpool_pending_pages(void* p) { return static_cast<ling::KvPool*>(p)->pending_pages(); }
int ref_kvpool_refs(void* p, int page) {
  try {
    return static_cast<ling::KvPool*>(p)->refs(page);
  } catch (...) {
    return -1;
  }
}
int ref_kvpool_needed(void* p, const int* table, int len, int from, int to) {
  return static_cast<ling::KvPool*>(p)->needed(std::vector<int>(table, table + len), from, to);
}
int ref_kvpool_ensure(void* p, int* table, int* len, int cap, int from, int to, int* copies, int max_copies, int* n_copies) {
  std::vector<int> t(table, table + *len);
  std::vector<ling::KvPool::Copy> cp;
  bool ok;
  try {
    ok = static_cast<ling::KvPool*>(p)->ensure(t, from, to, &cp);
  } catch (...) {
    return -1;
  }
  if (int(t.size()) > cap) return -2;
  std::copy(t.begin(), t.end(), table);
  *len = int(t.size());
  *n_copies = int(cp.size());
  for (int i = 0; i < int(cp.size()) && i < max_copies; ++i) copies[2 * i] = cp[i].src, copies[2 * i + 1] = cp[i].dst;
  return ok ? 1 : 0;
}
int ref_kvpool_share(void* p, int* dst, int* dst_len, int cap, const int* src, int src_len, int n) {
  std::vector<int> d(dst, dst + *dst_len);
  try {
    static_cast<ling::KvPool*>(p)->share(d, std::vector<int>(src, src + src_len), n);
  } catch (...) {
    return -1;
  }
  if (int(d.size()) > cap) return -2;
  std::copy(d.begin(), d.end(), dst);
  *dst_len = int(d.size());
  return 0;
}
void ref_kvpool_truncate(void* p, int* table, int len, int n) {
  std::vector<int> t(table, table + len);
  static_cast<ling::KvPool*>(p)->truncate(t, n);
  std::copy(t.begin(), t.end(), table);
}
void ref_kvpool_unshare(void* p, int* table, int len, int n) {
  std::vector<int> t(table, table + len);
  static_cast<ling::KvPool*>(p)->unshare(t, n);
  std::copy(t.begin(), t.end(), table);
}
int ref_kvpool_net_need(const int* table, int len, int pages) {
  return ling::KvPool::net_need(std::vector<int>(table, table + len), pages);
}
int ref_kvpool_resume_need(void* p, const int* table, int len, int reuse, int pages, const int* donor, int donor_len) {
  std::vector<int> d;
  if (donor) d.assign(donor, donor + donor_len);
  try {
    return static_cast<ling::KvPool*>(p)->resume_need(std::vector<int>(table, table + len), reuse, pages, donor ? &d : nullptr);
  } catch (...) {
    return -1;
  }
}
int ref_kvpool_reclaimable(void* p, const int* const* tables, const int* lens, int n) {
  std::vector<std::vector<int>> hold(n);
  ling::KvPool::Refs refs;
  for (int i = 0; i < n; ++i) {
    hold[i].assign(tables[i], tables[i] + lens[i]);
    refs.push_back(&hold[i]);
  }
  return static_cast<ling::KvPool*>(p)->reclaimable(refs);
}
int ref_kvpool_retain(void* p, int page) {
  try {
    static_cast<ling::KvPool*>(p)->retain(page);
    return 0;
  } catch (...) {
    return 1;
  }
}
int ref_kvpool_release(void* p, int page) {
  try {
    static_cast<ling::KvPool*>(p)->release(page);
    return 0;
  } catch (...) {
    return 1;
  }
}
void ref_kvpool_retire(void* p) { static_cast<ling::KvPool*>(p)->retire(); }

// ---- pairing, pool policy
static std::vector<ling::serve::PairCandidate> cands(const int* batchable, const int* recent, const long* last, int n) {
  std::vector<ling::serve::PairCandidate> c(n);
  for (int i = 0; i < n; ++i) c[i] = {batchable[i] != 0, recent[i], last[i]};
  return c;
}
int ref_pair_order(const int* batchable, const int* recent, const long* last, int n, int fair, int* order) {
  const auto o = ling::serve::pair_order(cands(batchable, recent, last, n), fair != 0);
  for (size_t i = 0; i < o.size(); ++i) order[i] = int(o[i]);
  return int(o.size());
}
int ref_select_batch(const int* batchable, const int* recent, const long* last, int n, int self, int fit, int fair, int* batch) {
  const auto b = ling::serve::select_batch(cands(batchable, recent, last, n), size_t(self), fit, fair != 0);
  for (size_t i = 0; i < b.size(); ++i) batch[i] = int(b[i]);
  return int(b.size());
}
int ref_pass_window_count(const long* marks, int n, long now, long* last_out) {
  ling::serve::PassWindow w;
  for (int i = 0; i < n; ++i) w.record(marks[i]);
  w.trim(now);
  *last_out = w.last();
  return w.count(now);
}
int ref_kv_verdict(int need, int free_pages, int pending, int idle) {
  return int(ling::serve::kv_verdict(need, {free_pages, pending, idle}));
}
int ref_kv_last_resort(const long* admitted, const int* waiting, const int* need, int n, int free_pages, int pending, int idle) {
  std::vector<ling::serve::KvRunner> r(n);
  for (int i = 0; i < n; ++i) r[i] = {admitted[i], waiting[i] != 0, need[i]};
  return ling::serve::kv_last_resort(r, {free_pages, pending, idle});
}

// ---- admission
struct ref_plan {
  size_t weights, per_session, sessions, scratch, kv_pool;
  int session_count;
  long kv_pool_pages;
  size_t total;
  int refused;
};
int ref_start_plan(const int* cfg, const unsigned char* full, size_t weight_bytes, size_t scratch, int drafter, int sessions,
                   int max_context, long avail_mb, long reserve_mb, int kv_on, size_t store_bytes, long pool_mb,
                   ref_plan* out) {
  ling::serve::KvPlanInputs kv;
  kv.on = kv_on != 0, kv.store_bytes = store_bytes, kv.pool_mb = pool_mb;
  const ling::serve::StartPlan s =
      ling::serve::start_plan(make_config(cfg, full), weight_bytes, scratch, drafter != 0, sessions, max_context, avail_mb, reserve_mb, kv);
  out->weights = s.plan.weights, out->per_session = s.plan.per_session, out->sessions = s.plan.sessions;
  out->scratch = s.plan.scratch, out->kv_pool = s.plan.kv_pool, out->session_count = s.plan.session_count;
  out->kv_pool_pages = s.plan.kv_pool_pages, out->total = s.plan.total(), out->refused = !s.refusal.empty();
  return 0;
}
int ref_choose_size(const int* cfg, const unsigned char* full, size_t weight_bytes, size_t scratch, int drafter, long avail_mb,
                    long reserve_mb, int full_context, int sessions, int max_context, int auto_size, int kv_on,
                    size_t store_bytes, long pool_mb, int* out) {
  ling::serve::KvPlanInputs kv;
  kv.on = kv_on != 0, kv.store_bytes = store_bytes, kv.pool_mb = pool_mb;
  const ling::serve::SizeChoice s = ling::serve::choose_size(
      make_config(cfg, full), weight_bytes, scratch, drafter != 0, avail_mb, reserve_mb, full_context,
      sessions >= 0 ? std::optional<int>(sessions) : std::nullopt, max_context >= 0 ? std::optional<int>(max_context) : std::nullopt,
      auto_size != 0, kv);
  out[0] = s.sessions, out[1] = s.max_context, out[2] = s.sessions_auto, out[3] = s.context_auto, out[4] = s.sized;
  return 0;
}
int ref_refuse_request(long avail_mb, long reserve_mb) { return !ling::serve::refuse_request(avail_mb, reserve_mb).empty(); }
int ref_refuse_request_text(long avail_mb, long reserve_mb, char* buf, int buf_len) {
  const std::string text = ling::serve::refuse_request(avail_mb, reserve_mb);
  if (int(text.size()) + 1 > buf_len) return -1;
  std::memcpy(buf, text.c_str(), text.size() + 1);
  return int(text.size());
}
// kv_reclaim (src/serve/kv_policy.hpp:58-72) on a scripted scenario: group g holds group_size[g] holders; evicting the
// e-th holder overall (groups concatenated) changes the unit's need by dneed[e] and the free + pending pages by dhave[e].
// evicted[g] returns how many holders of each group went.
int ref_kv_reclaim(int need0, int have0, const int* group_size, const int* dneed, const int* dhave, int n_kept, int need_kept,
                   int reach_kept, int n_source, int need_all, int reach_all, int must, int* evicted) {
  int need = need0, have = have0;
  const int groups = n_kept + n_source;
  std::vector<int> first(groups + 1, 0);
  for (int g = 0; g < groups; ++g) first[g + 1] = first[g] + group_size[g], evicted[g] = 0;
  auto group = [&](int g) {
    return ling::serve::KvEvictNext([&, g]() {
      if (evicted[g] >= group_size[g]) return false;
      const int e = first[g] + evicted[g]++;
      need += dneed[e], have += dhave[e];
      return true;
    });
  };
  std::vector<ling::serve::KvEvictNext> kept, source;
  for (int g = 0; g < n_kept; ++g) kept.push_back(group(g));
  for (int g = n_kept; g < groups; ++g) source.push_back(group(g));
  return ling::serve::kv_reclaim([&] { return need; }, [&] { return have; }, kept, need_kept, reach_kept, source, need_all,
                                 reach_all, must != 0) ? 1 : 0;
}

// ---- step trace
int ref_format_step(double t, long pass, const char* kind, size_t turn, const int* sessions, const int* rows, const int* tokens,
                    const int* left, int n, const int* cand, const long* cand_request, const long* cand_last, int n_cand,
                    double ms, int side, char* buf, int buf_len) {
  ling::serve::StepRecord s;
  s.t = t, s.pass = pass, s.kind = kind, s.turn = turn, s.ms = ms, s.side = side != 0;
  s.sessions.assign(sessions, sessions + n), s.rows.assign(rows, rows + n), s.tokens.assign(tokens, tokens + n);
  s.left.assign(left, left + n);
  for (int i = 0; i < n_cand; ++i) s.cand.push_back({cand[3 * i], cand_request[i], cand[3 * i + 1], cand[3 * i + 2], cand_last[i]});
  const std::string line = ling::serve::format_step(s);
  if (int(line.size()) + 1 > buf_len) return -1;
  std::memcpy(buf, line.c_str(), line.size() + 1);
  return int(line.size());
}

// ---- the prefix KV store (core/prefix_kv.hpp), paged mode; the callbacks mirror the product's C interface
struct ref_prefix_ops {
  void* user;
  int (*hold)(void* user, int from, int to, int* pages, int cap);
  void (*retain)(void* user, int page);
  void (*drop)(void* user, int page);
  void* (*state_alloc)(void* user, size_t bytes);
  void (*state_release)(void* user, void* state);
};
void* ref_prefix_create(size_t budget, size_t state_bytes, const ref_prefix_ops* o) {
  const ref_prefix_ops c = *o;
  ling::PrefixKvTree::Ops ops;
  ops.alloc = [c](size_t n) { return c.state_alloc(c.user, n); };
  ops.release = [c](void* p) { c.state_release(c.user, p); };
  ops.store = [](void*, int, int, int, int) {};
  ops.hold = [c](int from, int to) {
    const int want = ling::KvPool::index_of(to - 1) - ling::KvPool::index_of(from) + 1;
    std::vector<int> ids(want, 0);
    const int got = c.hold(c.user, from, to, ids.data(), want);
    ids.resize(got < 0 ? 0 : (got > want ? want : got));
    return ids;
  };
  ops.retain = [c](int pg) { c.retain(c.user, pg); };
  ops.drop = [c](int pg) { c.drop(c.user, pg); };
  return new ling::PrefixKvTree(budget, 0, state_bytes, std::move(ops));
}
void ref_prefix_destroy(void* t) { delete static_cast<ling::PrefixKvTree*>(t); }
static ling::PrefixKvTree::Match as_match(const int* path, int n_path, int len) {
  ling::PrefixKvTree::Match m;
  m.len = len;
  m.path.assign(path, path + n_path);
  return m;
}
int ref_prefix_match(void* t, const int* prompt, int n, uint64_t scope, int* path, int cap, int* n_path) {
  const auto m = static_cast<ling::PrefixKvTree*>(t)->match(std::vector<int>(prompt, prompt + n), scope);
  *n_path = int(m.path.size());
  for (int i = 0; i < *n_path && i < cap; ++i) path[i] = m.path[i];
  return m.len;
}
int ref_prefix_best_state(void* t, const int* path, int n_path, int len, int limit, void** state) {
  const void* st = nullptr;
  const int pos = static_cast<ling::PrefixKvTree*>(t)->best_state(as_match(path, n_path, len), limit, &st);
  *state = const_cast<void*>(st);
  return pos;
}
int ref_prefix_pages(void* t, const int* path, int n_path, int len, int n, int* pages, int cap) {
  const std::vector<int> pg = static_cast<ling::PrefixKvTree*>(t)->pages(as_match(path, n_path, len), n);
  if (int(pg.size()) > cap) return -1;
  for (size_t i = 0; i < pg.size(); ++i) pages[i] = pg[i];
  return int(pg.size());
}
void ref_prefix_touch(void* t, const int* path, int n_path, uint64_t epoch) {
  static_cast<ling::PrefixKvTree*>(t)->touch(as_match(path, n_path, 0), epoch);
}
int ref_prefix_insert(void* t, const int* prompt, int n, int q, const int* cuts, int n_cuts, uint64_t epoch, uint64_t scope,
                      int* want_node, int* want_pos, int cap) {
  const auto want = static_cast<ling::PrefixKvTree*>(t)->insert(std::vector<int>(prompt, prompt + n), q,
                                                                std::vector<int>(cuts, cuts + n_cuts), epoch, scope);
  for (size_t i = 0; i < want.size() && int(i) < cap; ++i) want_node[i] = want[i].first, want_pos[i] = want[i].second;
  return int(want.size());
}
void* ref_prefix_add_state(void* t, int node, uint64_t epoch) { return static_cast<ling::PrefixKvTree*>(t)->add_state(node, epoch); }
int ref_prefix_evict_lru_leaf(void* t, const int* keep, int n_keep) {
  return static_cast<ling::PrefixKvTree*>(t)->evict_lru_leaf(std::vector<int>(keep, keep + n_keep));
}
void ref_prefix_clear(void* t) { static_cast<ling::PrefixKvTree*>(t)->clear(); }
size_t ref_prefix_bytes(void* t) { return static_cast<ling::PrefixKvTree*>(t)->bytes(); }
int ref_prefix_nodes(void* t) { return static_cast<ling::PrefixKvTree*>(t)->nodes(); }
int ref_prefix_states(void* t) { return static_cast<ling::PrefixKvTree*>(t)->states(); }
int ref_prefix_pages_held(void* t) { return static_cast<ling::PrefixKvTree*>(t)->pages_held(); }
int ref_prefix_page_lists(void* t, const int* skip, int n_skip, int* pages, int cap_pages, int* lens, int cap_lists) {
  const auto lists = static_cast<ling::PrefixKvTree*>(t)->page_lists(std::vector<int>(skip, skip + n_skip));
  int used = 0, n = 0;
  for (const auto& l : lists) {
    if (n >= cap_lists || used + int(l.size()) > cap_pages) return -1;
    for (int pg : l) pages[used++] = pg;
    lens[n++] = int(l.size());
  }
  return n;
}
void* ref_arena_create(size_t size, size_t align) { return new ling::ArenaAlloc(size, align); }
void ref_arena_destroy(void* a) { delete static_cast<ling::ArenaAlloc*>(a); }
long long ref_arena_alloc(void* a, size_t bytes) {
  size_t off = 0;
  return static_cast<ling::ArenaAlloc*>(a)->alloc(bytes, &off) ? (long long)off : -1;
}
void ref_arena_release(void* a, size_t off) { static_cast<ling::ArenaAlloc*>(a)->release(off); }
size_t ref_arena_size(void* a) { return static_cast<ling::ArenaAlloc*>(a)->size(); }
size_t ref_arena_in_use(void* a) { return static_cast<ling::ArenaAlloc*>(a)->in_use(); }

}  // extern "C"
