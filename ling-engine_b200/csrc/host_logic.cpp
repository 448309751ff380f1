// host_logic.cpp -- the CUDA-free half of the verify-step library: tree description and greedy acceptance, the
// context-lookup proposal, the best-first tree builder, the KV page pool's bookkeeping, pairing, pool policy,
// admission arithmetic and the step-trace line.  The reference keeps this policy in CUDA-free classes so that it is
// testable on the host (src/core/kv_pool.hpp:5-6, src/serve/kv_policy.hpp:1-3, src/serve/pairing.hpp:11 in the
// reference project); each function below names the reference declaration whose behaviour it reproduces.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <map>
#include <numeric>
#include <queue>
#include <set>
#include <string>
#include <vector>

#include "../../include/ling_b200.h"

namespace {

// ---------------------------------------------------------------------------------------------- trees
struct Shape {  // a tree as parent links plus what follows from them
  int n = 0;
  std::vector<int> parent, depth;
  std::vector<std::vector<int>> kids;  // row order
  bool build(const int* par, int rows) {
    if (rows < 1) return false;
    n = rows;
    parent.assign(rows, -1), depth.assign(rows, 0), kids.assign(rows, {});
    for (int r = 1; r < rows; ++r) {
      if (par[r] < 0 || par[r] >= r) return false;
      parent[r] = par[r];
      depth[r] = depth[par[r]] + 1;
      kids[par[r]].push_back(r);
    }
    return true;
  }
  bool leaf(int r) const { return kids[r].empty(); }
};

}  // namespace

extern "C" {

// describe_tree (src/core/tree.cpp:81-146).
int ling_b200_describe_tree(const int* parent, int n_rows, int chain, ling_b200_tree_desc* out) {
  Shape t;
  if (!parent || !out || n_rows > LING_B200_MAX_TREE_ROWS || !t.build(parent, n_rows)) return LING_B200_ERR_ARG;
  std::memset(out, 0, sizeof *out);
  out->n = n_rows;
  // Variants: one per leaf, row order; a variant's path holds the leaf's ancestor at every depth.
  std::vector<int> variant_of_leaf(n_rows, -1);
  for (int r = 0; r < n_rows; ++r) {
    out->depth[r] = t.depth[r];
    if (!t.leaf(r)) continue;
    if (out->nvar == LING_B200_MAX_TREE_VARIANTS) return LING_B200_ERR_ARG;
    variant_of_leaf[r] = out->nvar;
    int a = r;
    while (a >= 0) {
      out->path[out->nvar][t.depth[a]] = a;
      a = t.parent[a];
    }
    ++out->nvar;
  }
  // A row belongs to the variant of the leaf its first-child descent ends in.
  for (int r = 0; r < n_rows; ++r) {
    int a = r;
    while (!t.leaf(a)) a = t.kids[a][0];
    out->var[r] = variant_of_leaf[a];
  }
  // DeltaNet paths.  A path lists nodes that advance the state; right after a node come its leaf children (computed
  // from the node's state).  The write flag marks the first emission of a row.
  std::vector<bool> done(n_rows, false);
  auto emit_path = [&](const std::vector<int>& nodes) {
    int* step = out->gdn_step[out->ngdn];
    int k = 0;
    for (int w : nodes) {
      step[k++] = done[w] ? w : (w | LING_B200_TREE_WRITE);
      done[w] = true;
      for (int ch : t.kids[w])
        if (t.leaf(ch) && !done[ch]) {
          step[k++] = ch | LING_B200_TREE_LEAF | LING_B200_TREE_WRITE;
          done[ch] = true;
        }
    }
    out->gdn_len[out->ngdn++] = k;
  };
  std::vector<int> nodes;
  for (int r = 0; r <= chain && r < n_rows; ++r) nodes.push_back(r);
  emit_path(nodes);
  for (int r = 0; r < n_rows; ++r) {
    if (done[r] || t.leaf(r)) continue;
    nodes.assign(size_t(t.depth[r]) + 1, 0);
    for (int a = r; a >= 0; a = t.parent[a]) nodes[t.depth[a]] = a;
    int a = r;
    for (;;) {  // continue through first internal children
      auto it = std::find_if(t.kids[a].begin(), t.kids[a].end(), [&](int ch) { return !t.leaf(ch); });
      if (it == t.kids[a].end()) break;
      nodes.push_back(*it);
      a = *it;
    }
    if (out->ngdn == LING_B200_MAX_TREE_VARIANTS) return LING_B200_ERR_ARG;
    emit_path(nodes);
  }
  return std::all_of(done.begin(), done.end(), [](bool b) { return b; }) ? LING_B200_OK : LING_B200_ERR_ARG;
}

// accept_tree_greedy (src/core/tree.cpp:148-166).
int ling_b200_accept_tree_greedy(const int* parent, const int* token, int n_rows, const int* argmax, int* path, int* next) {
  int len = 0, at = 0;
  path[len++] = 0;
  while (true) {
    const int want = argmax[at];
    int hit = -1;
    for (int r = at + 1; r < n_rows && hit < 0; ++r)
      if (parent[r] == at && token[r] == want) hit = r;
    if (hit < 0) {
      *next = want;
      return len;
    }
    path[len++] = at = hit;
  }
}

// lookup_propose (src/core/lookup.cpp:7-24).
int ling_b200_lookup_propose(const int* seq, int len, int max, int ngram, int* out, int* match) {
  *match = 0;
  if (len <= ngram || max <= 0) return 0;
  const int* tail = seq + len - ngram;
  for (int at = len - ngram - 1; at >= 0; --at) {
    if (!std::equal(tail, tail + ngram, seq + at)) continue;
    int agree = ngram;  // extend the agreement backwards, up to 64
    while (agree < 64 && at - (agree - ngram) - 1 >= 0 && seq[at - (agree - ngram) - 1] == seq[len - agree - 1]) ++agree;
    const int first = at + ngram, count = std::min(max, len - first);
    std::copy(seq + first, seq + first + count, out);
    *match = agree;
    return count;
  }
  return 0;
}

// build_tree (src/core/tree.cpp:30-79): the chain, then extra nodes best first by path probability (product of
// softmax(scores / temp) along the path); ties to the lower parent row, then the lower candidate; at most `width`
// children per node; no (parent, candidate) twice.
int ling_b200_build_tree(int anchor, const int* cand, const float* scores, int E, int K16, const int* chain_tokens,
                         const int* chain_picks, int nodes, double temp, int width, int max_depth, int chain, int max_rows,
                         int* parent, int* depth, int* token, int* pick, double* extra_mass) {
  const int positions = E;
  const int chain_len = std::min(E, std::max(1, chain));
  auto probs = [&](int pos, int prev_pick) {
    const float* row = scores + (size_t(pos) * K16 + (pos == 0 ? 0 : prev_pick)) * K16;
    std::vector<double> p(K16);
    double top = row[0];
    for (int k = 1; k < K16; ++k) top = std::max(top, double(row[k]));
    double z = 0;
    for (int k = 0; k < K16; ++k) z += p[k] = std::exp((row[k] - top) / temp);
    for (double& v : p) v /= z;
    return p;
  };
  int rows = 0;
  std::vector<double> mass;
  std::vector<int> nkids;
  auto add = [&](int par, int tok, int pk, double m) {
    parent[rows] = par, depth[rows] = par < 0 ? 0 : depth[par] + 1, token[rows] = tok, pick[rows] = pk;
    mass.push_back(m), nkids.push_back(0);
    if (par >= 0) ++nkids[par];
    return rows++;
  };
  add(-1, anchor, 0, 1.0);
  for (int e = 0; e < chain_len; ++e) add(e, chain_tokens[e], chain_picks[e], mass[e] * probs(e, pick[e])[chain_picks[e]]);
  *extra_mass = 0;
  const int limit = std::min({LING_B200_MAX_TREE_ROWS, max_rows, chain_len + 1 + nodes});
  if (rows >= limit) return rows | (chain_len << 16);
  struct Item {
    double p;
    int par, k;
    bool operator<(const Item& o) const {  // max-heap: larger p, then lower parent, then lower candidate
      if (p != o.p) return p < o.p;
      if (par != o.par) return par > o.par;
      return k > o.k;
    }
  };
  std::priority_queue<Item> heap;
  std::set<std::pair<int, int>> used;
  for (int r = 1; r <= chain_len; ++r) used.insert({parent[r], pick[r]});
  auto offer_children = [&](int r) {
    const int pos = depth[r];
    if (pos >= positions || pos + 1 > max_depth) return;
    const std::vector<double> p = probs(pos, pick[r]);
    for (int k = 0; k < K16; ++k)
      if (!used.count({r, k})) heap.push({mass[r] * p[k], r, k});
  };
  for (int r = 0; r < rows; ++r) offer_children(r);
  while (rows < limit && !heap.empty()) {
    const Item it = heap.top();
    heap.pop();
    if (used.count({it.par, it.k}) || nkids[it.par] >= width) continue;
    used.insert({it.par, it.k});
    const int r = add(it.par, cand[size_t(depth[it.par]) * K16 + it.k], it.k, it.p);
    *extra_mass += it.p;
    offer_children(r);
  }
  return rows | (chain_len << 16);
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------- KV page pool
// KvPool (src/core/kv_pool.hpp:20-83, src/core/kv_pool.cpp).  Page ids 1 .. pages-1 (0 = unmapped, never handed out);
// a free stack that hands out the lowest ids first; a reference count per page; released pages wait in `pending`
// until retire() and come back so that the earliest released is handed out first.
struct ling_b200_kvpool {
  int page_tokens;
  std::vector<int> refs, free_stack, pending;
  int index_of(int pos) const { return pos / page_tokens; }
  int pages_for(int positions) const { return (positions + page_tokens - 1) / page_tokens; }
  bool live(int p) const { return p > 0 && p < int(refs.size()) && refs[p] > 0; }
  int take() {
    const int p = free_stack.back();
    free_stack.pop_back();
    refs[p] = 1;
    return p;
  }
  bool drop(int p) {
    if (!live(p)) return false;
    if (--refs[p] == 0) pending.push_back(p);
    return true;
  }
  // pages a write of [from, to) would take: unmapped indices below pages_for(to), plus shared pages the write touches
  int needed(const int* table, int len, int from, int to, const std::map<int, int>* gone) const {
    const int n = pages_for(to), first_written = index_of(from);
    int need = 0;
    for (int i = 0; i < n; ++i) {
      const int p = i < len ? table[i] : 0;
      if (p == 0) {
        ++need;
        continue;
      }
      int r = refs[p];
      if (gone) {
        auto it = gone->find(p);
        if (it != gone->end()) r -= it->second;
      }
      if (i >= first_written && from < to && r > 1) ++need;
    }
    return need;
  }
};

extern "C" {

ling_b200_kvpool* ling_b200_kvpool_create(int pages, int page_tokens) {
  if (page_tokens < 1) return nullptr;
  ling_b200_kvpool* p = new ling_b200_kvpool;
  p->page_tokens = page_tokens;
  p->refs.assign(size_t(std::max(pages, 1)), 0);
  for (int id = pages - 1; id >= 1; --id) p->free_stack.push_back(id);
  return p;
}
void ling_b200_kvpool_destroy(ling_b200_kvpool* p) { delete p; }
int ling_b200_kvpool_capacity(const ling_b200_kvpool* p) { return int(p->refs.size()) - 1; }
int ling_b200_kvpool_free_pages(const ling_b200_kvpool* p) { return int(p->free_stack.size()); }
int ling_b200_kvpool_pending_pages(const ling_b200_kvpool* p) { return int(p->pending.size()); }
int ling_b200_kvpool_refs(const ling_b200_kvpool* p, int page) {
  return page >= 0 && page < int(p->refs.size()) ? p->refs[page] : -1;
}
int ling_b200_kvpool_needed(const ling_b200_kvpool* p, const int* table, int len, int from, int to) {
  return p->needed(table, len, from, to, nullptr);
}

// KvPool::ensure (kv_pool.hpp:44-48): all or nothing; a shared page the write touches is replaced by a fresh one and
// the (src, dst) copy is reported.  Returns 1 (done), 0 (free list short, nothing changed), -1 (bad range), -2 (table
// capacity too small).
int ling_b200_kvpool_ensure(ling_b200_kvpool* p, int* table, int* len, int cap, int from, int to, int* copies, int max_copies,
                            int* n_copies) {
  if (n_copies) *n_copies = 0;
  if (from < 0 || to < from) return -1;
  const int n = p->pages_for(to), first_written = p->index_of(from);
  if (n > cap) return -2;
  if (p->needed(table, *len, from, to, nullptr) > int(p->free_stack.size())) return 0;
  for (int i = *len; i < n; ++i) table[i] = 0;
  *len = std::max(*len, n);
  int nc = 0;
  for (int i = 0; i < n; ++i) {
    if (table[i] == 0) {
      table[i] = p->take();
    } else if (i >= first_written && from < to && p->refs[table[i]] > 1) {
      const int fresh = p->take();
      if (copies && nc < max_copies) copies[2 * nc] = table[i], copies[2 * nc + 1] = fresh;
      ++nc;
      p->drop(table[i]);
      table[i] = fresh;
    }
  }
  if (n_copies) *n_copies = nc;
  return 1;
}

// KvPool::share (kv_pool.hpp:49-51).
int ling_b200_kvpool_share(ling_b200_kvpool* p, int* dst, int* dst_len, int cap, const int* src, int src_len, int n) {
  const int np = p->pages_for(n);
  if (np > src_len) return -1;
  if (np > cap) return -2;
  for (int i = 0; i < np; ++i)
    if (src[i] == 0) return -1;
  for (int i = *dst_len; i < np; ++i) dst[i] = 0;
  *dst_len = std::max(*dst_len, np);
  for (int i = 0; i < np; ++i) {
    if (dst[i] == src[i]) continue;
    if (!p->live(src[i])) return -1;
    ++p->refs[src[i]];
    if (dst[i] != 0) p->drop(dst[i]);
    dst[i] = src[i];
  }
  return 0;
}
// KvPool::truncate (kv_pool.hpp:52-53).
void ling_b200_kvpool_truncate(ling_b200_kvpool* p, int* table, int len, int n) {
  for (int i = p->pages_for(std::max(n, 0)); i < len; ++i)
    if (table[i] != 0) {
      p->drop(table[i]);
      table[i] = 0;
    }
}
// KvPool::unshare (kv_pool.hpp:54-56).
void ling_b200_kvpool_unshare(ling_b200_kvpool* p, int* table, int len, int n) {
  for (int i = p->pages_for(std::max(n, 0)); i < len; ++i)
    if (table[i] != 0 && p->refs[table[i]] > 1) {
      p->drop(table[i]);
      table[i] = 0;
    }
}
// KvPool::net_need (kv_pool.hpp:38-41).
int ling_b200_kvpool_net_need(const ling_b200_kvpool*, const int* table, int len, int pages) {
  int need = 0;
  for (int i = 0; i < std::max(pages, len); ++i) {
    const bool mapped = i < len && table[i] != 0;
    if (i < pages) need += mapped ? 0 : 1;
    else need -= mapped ? 1 : 0;
  }
  return std::max(need, 0);
}
// KvPool::resume_need (kv_pool.hpp:57-66): what a prefill that resumes at position `reuse` and maps every page index below
// `pages` draws from the free list, net.  The documented sequence -- share the donor's pages for [0, reuse), truncate to
// `pages`, unshare from the resume point on, ensure [reuse, end) -- is carried out for real on a scratch copy of the pool
// and of the table (the copy's free list is padded with stand-in pages so that ensure cannot run short), and the answer
// is read off the copy: pages that left its free list, less pages the holder's own releases queued for retirement.
int ling_b200_kvpool_resume_need(const ling_b200_kvpool* p, const int* table, int len, int reuse, int pages, const int* donor,
                                 int donor_len) {
  reuse = std::max(reuse, 0), pages = std::max(pages, 0);
  ling_b200_kvpool sim = *p;
  const int real = int(sim.refs.size());
  sim.refs.resize(size_t(real + pages + 1), 0);
  std::vector<int> stock;  // the stand-ins go under the real free pages: they are handed out only when those run out
  for (int id = real + pages; id >= real; --id) stock.push_back(id);
  stock.insert(stock.end(), sim.free_stack.begin(), sim.free_stack.end());
  sim.free_stack.swap(stock);
  const size_t free_before = sim.free_stack.size(), pending_before = sim.pending.size();
  const int cap = std::max({len, pages, sim.pages_for(reuse)}) + 1;
  std::vector<int> t(size_t(cap), 0);
  std::copy(table, table + len, t.begin());
  int tl = len;
  if (donor && ling_b200_kvpool_share(&sim, t.data(), &tl, cap, donor, donor_len, reuse) != 0) return -1;
  const int end = pages * sim.page_tokens;
  ling_b200_kvpool_truncate(&sim, t.data(), tl, end);
  ling_b200_kvpool_unshare(&sim, t.data(), tl, reuse);
  if (ling_b200_kvpool_ensure(&sim, t.data(), &tl, cap, std::min(reuse, end), end, nullptr, 0, nullptr) != 1) return -1;
  const long taken = long(free_before) - long(sim.free_stack.size());
  const long released = long(sim.pending.size()) - long(pending_before);
  return int(std::max(taken - released, 0L));
}
// KvPool::reclaimable (kv_pool.hpp:67-70).
int ling_b200_kvpool_reclaimable(const ling_b200_kvpool* p, const int* const* tables, const int* lens, int n) {
  std::map<int, int> listed;
  for (int i = 0; i < n; ++i)
    for (int j = 0; j < lens[i]; ++j)
      if (tables[i][j] > 0) ++listed[tables[i][j]];
  int freed = 0;
  for (const auto& kv : listed) freed += kv.second >= p->refs.at(size_t(kv.first)) ? 1 : 0;
  return freed;
}
int ling_b200_kvpool_retain(ling_b200_kvpool* p, int page) {
  if (!p->live(page)) return 1;
  ++p->refs[page];
  return 0;
}
int ling_b200_kvpool_release(ling_b200_kvpool* p, int page) { return p->drop(page) ? 0 : 1; }
// KvPool::retire (kv_pool.hpp:73-74): the earliest released page is the next one handed out.
void ling_b200_kvpool_retire(ling_b200_kvpool* p) {
  for (auto it = p->pending.rbegin(); it != p->pending.rend(); ++it) p->free_stack.push_back(*it);
  p->pending.clear();
}

// ---------------------------------------------------------------------------------------------- pairing, pool policy
// pair_order (src/serve/pairing.hpp:46-54): running order, or (fair) fewest recent passes, then oldest last pass, then
// running order.
int ling_b200_pair_order(const int*, const int* recent, const long* last, int n, int fair, int* order) {
  std::iota(order, order + n, 0);
  if (fair)
    std::stable_sort(order, order + n, [&](int a, int b) {
      if (recent[a] != recent[b]) return recent[a] < recent[b];
      return last[a] < last[b];
    });
  return n;
}
// select_batch (src/serve/pairing.hpp:56-75).
int ling_b200_select_batch(const int* batchable, const int* recent, const long* last, int n, int self, int fit, int fair,
                           int* batch) {
  if (self < 0 || self >= n || !batchable[self]) return 0;
  std::vector<int> order(size_t(n), 0);
  ling_b200_pair_order(batchable, recent, last, n, fair, order.data());
  int k = 0;
  batch[k++] = self;
  for (int o : order)
    if (o != self && k < fit && batchable[o]) batch[k++] = o;
  return k;
}
// kv_verdict (src/serve/kv_policy.hpp:38-43): 0 Go, 1 Retire, 2 Reclaim, 3 Wait.
int ling_b200_kv_verdict(int need, int free_pages, int pending, int idle) {
  if (need <= free_pages) return 0;
  if (need <= free_pages + pending) return 1;
  if (need <= free_pages + pending + idle) return 2;
  return 3;
}
// kv_last_resort (src/serve/kv_policy.hpp:82-93): only when every running request waits and none could be served from
// free + pending + idle pages; the one admitted last.
int ling_b200_kv_last_resort(const long* admitted, const int* waiting, const int* need, int n, int free_pages, int pending,
                             int idle) {
  int pick = -1;
  for (int i = 0; i < n; ++i) {
    if (!waiting[i] || ling_b200_kv_verdict(need[i], free_pages, pending, idle) != 3) return -1;
    if (pick < 0 || admitted[i] > admitted[pick]) pick = i;
  }
  return pick;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------- admission
namespace {
struct Sizes {  // the byte arithmetic of src/serve/admission.hpp:44-80 with the page size and KV width as parameters
  const ling_b200_model_config* c;
  int page_tokens, kv_elem_bytes;
  int full() const {
    int f = 0;
    for (int l = 0; l < c->layers; ++l) f += c->full_attention[l] ? 1 : 0;
    return f;
  }
  size_t kv_per_token() const { return size_t(full()) * 2 * c->kv_heads * c->head_dim * size_t(kv_elem_bytes); }
  size_t page_bytes() const { return kv_per_token() * size_t(page_tokens); }
  long pages_for(long positions) const { return (positions + page_tokens - 1) / page_tokens; }
  size_t session_bytes(int max_context, bool drafter, bool paged) const {
    const int lin = c->layers - full();
    const int conv_channels = 2 * c->lin_k_heads * c->lin_k_dim + c->lin_v_heads * c->lin_v_dim;
    const size_t kv = paged ? 0 : kv_per_token() * size_t(max_context);
    const size_t state = size_t(lin) * c->lin_v_heads * c->lin_k_dim * c->lin_v_dim * 4;
    const size_t conv = size_t(lin) * conv_channels * size_t(c->conv_kernel - 1) * 4;
    const size_t ring = drafter ? size_t(5) * 2 * 8224 * 1024 * 2 : 0;  // kDraftRingBytes
    return kv + 2 * (state + conv) + ring + size_t(max_context) * 4;
  }
};

// How many KV pages the pool gets (plan_kv_pool's rule, src/serve/admission.hpp:104-108): an explicit size in MB wins;
// otherwise, when there is an available-memory figure and a reserve to judge by, whatever is left after the rest of the
// plan, the prefix store's budget, the reserve and the pool's own reserved page 0; otherwise (and never more than) the
// pages that every session at its full context would map.
long pool_pages(const Sizes& z, int sessions, int max_context, long avail_mb, long reserve_mb, long pool_mb, size_t other_bytes) {
  const long ceiling = long(sessions) * z.pages_for(max_context);
  const size_t page = z.page_bytes();
  const auto mb = [](long v) { return size_t(v) << 20; };
  long pages = ceiling;
  if (pool_mb >= 0) {
    pages = long(mb(pool_mb) / page);
  } else if (avail_mb >= 0 && reserve_mb > 0) {
    const size_t spoken_for = other_bytes + mb(reserve_mb) + page;
    pages = mb(avail_mb) > spoken_for ? long((mb(avail_mb) - spoken_for) / page) : 0;
  }
  return std::clamp(pages, 0L, ceiling);
}

// The pool's floor (refuse_kv_pool, admission.hpp:126-142): a pool sized from the plan must hold one conversation at the
// full context plus the two growth pages a request is admitted with -- unless it already holds every session's context.
long pool_floor(const Sizes& z, int sessions, int max_context) {
  return std::min(z.pages_for(max_context) + 2, long(sessions) * z.pages_for(max_context));
}

// start_plan (src/serve/admission.hpp:202-216): the memory plan, the pool and its floor, then the host-memory check
// (refuse_start, 170-186: the plan plus the reserve must fit what is available).
void make_plan(const Sizes& z, size_t weight_bytes, size_t scratch, bool drafter, int sessions, int max_context, long avail_mb,
               long reserve_mb, bool kv_on, size_t store_bytes, long pool_mb, ling_b200_memory_plan* p) {
  *p = ling_b200_memory_plan{};
  p->weights = weight_bytes, p->scratch = scratch, p->session_count = sessions;
  p->per_session = z.session_bytes(max_context, drafter, kv_on);
  p->sessions = p->per_session * size_t(sessions);
  const bool judged = reserve_mb > 0 && avail_mb >= 0;
  bool pool_too_small = false;
  if (kv_on) {
    const size_t rest_of_plan = p->weights + p->sessions + p->scratch;
    p->kv_pool_pages = pool_pages(z, sessions, max_context, avail_mb, reserve_mb, pool_mb, rest_of_plan + store_bytes);
    p->kv_pool = size_t(p->kv_pool_pages + 1) * z.page_bytes();  // the reserved page 0 rides along
    pool_too_small = pool_mb < 0 && judged && p->kv_pool_pages < pool_floor(z, sessions, max_context);
  }
  p->total = p->weights + p->sessions + p->scratch + p->kv_pool;
  const bool host_short = judged && long(p->total >> 20) + reserve_mb > avail_mb;
  p->refused = (pool_too_small || host_short) ? 1 : 0;
}
}  // namespace

extern "C" {

int ling_b200_start_plan(const ling_b200_model_config* cfg, size_t weight_bytes, size_t scratch, int drafter, int sessions,
                         int max_context, long avail_mb, long reserve_mb, int kv_on, size_t store_bytes, long pool_mb,
                         int page_tokens, int kv_elem_bytes, ling_b200_memory_plan* out) {
  if (!cfg || !out || page_tokens < 1) return LING_B200_ERR_ARG;
  make_plan(Sizes{cfg, page_tokens, kv_elem_bytes}, weight_bytes, scratch, drafter != 0, sessions, max_context, avail_mb,
            reserve_mb, kv_on != 0, store_bytes, pool_mb, out);
  return LING_B200_OK;
}

// choose_size (src/serve/admission.hpp:253-262 for the rule): what was given stays as given; what was not is chosen by
// the start check's own plan.  The context is chosen first, from a ladder that starts at the model's full context and
// halves (rounded down to a multiple of 2,048) while it stays at or above 32,768: the first rung at which the given
// session count, or one session, fits.  Then the most sessions that fit at that context, at most 4.  If no rung fits,
// the last rung with the given (or one) session is returned and the start check refuses it.  Without auto-sizing, without
// an available-memory figure or a reserve, or with both values given, the defaults (2 sessions, 65,536) fill the gaps.
int ling_b200_choose_size(const ling_b200_model_config* cfg, size_t weight_bytes, size_t scratch, int drafter, long avail_mb,
                          long reserve_mb, int full_context, int sessions, int max_context, int auto_size, int kv_on,
                          size_t store_bytes, long pool_mb, int page_tokens, int kv_elem_bytes, int* out_sessions,
                          int* out_context, int* sessions_auto, int* context_auto, int* sized) {
  constexpr int kMostSessions = 4, kShortestContext = 32768, kStep = 2048, kDefaultSessions = 2, kDefaultContext = 65536;
  const bool sessions_given = sessions >= 0, context_given = max_context >= 0;
  const bool measurable = avail_mb >= 0 && reserve_mb > 0;
  *sized = (auto_size && measurable) ? 1 : 0;
  if (!*sized || (sessions_given && context_given)) {
    *out_sessions = sessions_given ? sessions : kDefaultSessions;
    *out_context = context_given ? max_context : kDefaultContext;
    *sessions_auto = *context_auto = 0;
    return LING_B200_OK;
  }
  *sessions_auto = sessions_given ? 0 : 1, *context_auto = context_given ? 0 : 1;
  const Sizes z{cfg, page_tokens, kv_elem_bytes};
  const auto fits = [&](int n, int ctx) {
    ling_b200_memory_plan plan;
    make_plan(z, weight_bytes, scratch, drafter != 0, n, ctx, avail_mb, reserve_mb, kv_on != 0, store_bytes, pool_mb, &plan);
    if (plan.refused) return false;
    // paged_sessions_fit (admission.hpp:225-233): the pool must hold one conversation at the full context and half of
    // what n conversations at the full context would map
    return !kv_on || plan.kv_pool_pages >= std::max(pool_floor(z, n, ctx), long(n) * z.pages_for(ctx) / 2);
  };
  std::vector<int> ladder;
  if (context_given) {
    ladder.push_back(max_context);
  } else {
    const int top = full_context > 0 ? full_context : kDefaultContext;
    for (int rung = top; rung >= kShortestContext; rung = (rung / 2) / kStep * kStep) ladder.push_back(rung);
    if (ladder.empty()) ladder.push_back(top);  // a model whose full context is below the shortest rung
  }
  const int least = sessions_given ? sessions : 1;
  const auto rung = std::find_if(ladder.begin(), ladder.end(), [&](int ctx) { return fits(least, ctx); });
  *out_context = rung != ladder.end() ? *rung : ladder.back();
  *out_sessions = least;
  if (rung != ladder.end() && !sessions_given) {
    int n = kMostSessions;
    while (n > 1 && !fits(n, *rung)) --n;
    *out_sessions = n;
  }
  return LING_B200_OK;
}

// refuse_request (src/serve/admission.hpp:312-319): the text of the 503 a generation request gets while the host is below
// the admission reserve, written to buf; returns its length, 0 when the request may run (an unknown figure, avail_mb < 0,
// never refuses), -1 when buf is too small.
int ling_b200_refuse_request(long avail_mb, long reserve_mb, char* buf, int buf_len) {
  if (avail_mb < 0 || avail_mb >= reserve_mb) {
    if (buf && buf_len > 0) buf[0] = 0;
    return 0;
  }
  const std::string text = "host memory low: " + std::to_string(avail_mb) + " MB available, below the " + std::to_string(reserve_mb) +
                           " MB this server keeps free; the request was not started (retry later)";
  if (!buf || int(text.size()) + 1 > buf_len) return -1;
  std::memcpy(buf, text.c_str(), text.size() + 1);
  return int(text.size());
}

// kv_reclaim (src/serve/kv_policy.hpp:58-72): makes room for a unit by evicting holders.  need(user) and have(user) are
// the unit's need and the free + pending pages NOW (both change as holders go); evict(user, group) evicts the next
// holder of a group and returns 1, or 0 when the group has none left.  Groups 0 .. n_kept-1 are holders that may go
// without moving the unit's resume point, groups n_kept .. n_kept+n_source-1 the unit's own source.  The kept groups are
// enough when need_kept <= reach_kept; if they are not, the source groups join the order provided that evicting
// everything suffices (need_all <= reach_all) or `must` says nothing else will ever free pages -- otherwise nothing at
// all is evicted.  Along the order each group is drained while the unit still does not fit.  Returns 1 when it fits.
int ling_b200_kv_reclaim(ling_b200_count_fn need, ling_b200_count_fn have, ling_b200_evict_fn evict, void* user, int n_kept,
                         int need_kept, int reach_kept, int n_source, int need_all, int reach_all, int must) {
  const auto fits = [&] { return need(user) <= have(user); };
  if (fits()) return 1;
  int groups = n_kept;
  if (need_kept > reach_kept) {
    if (!must && need_all > reach_all) return 0;
    groups += n_source;
  }
  for (int g = 0; g < groups; ++g)
    while (!fits() && evict(user, g)) {
    }
  return fits() ? 1 : 0;
}

// format_step (src/serve/step_trace.hpp:66-87): one JSON line of the per-step trace.
int ling_b200_format_step(double t, long pass, const char* kind, size_t turn, const int* sessions, const int* rows,
                          const int* tokens, const int* left, int n, const int* cand, const long* cand_request,
                          const long* cand_last, int n_cand, double ms, int side, char* buf, int buf_len) {
  auto list = [n](const int* v) {
    std::string s = "[";
    for (int i = 0; i < n; ++i) s += (i ? "," : "") + std::to_string(v[i]);
    return s + "]";
  };
  char num[192];
  std::snprintf(num, sizeof num, "{\"t\":%.6f,\"pass\":%ld,\"kind\":\"%s\",\"turn\":%zu,", t, pass, kind, turn);
  std::string line = num;
  line += "\"sessions\":" + list(sessions) + ",\"rows\":" + list(rows) + ",\"tokens\":" + list(tokens) + ",\"left\":" + list(left);
  if (n_cand > 0) {
    line += ",\"cand\":[";
    for (int i = 0; i < n_cand; ++i) {
      line += i ? ",[" : "[";
      line += std::to_string(cand[3 * i]) + "," + std::to_string(cand_request[i]) + "," + std::to_string(cand[3 * i + 1]) + "," +
              std::to_string(cand[3 * i + 2]) + "," + std::to_string(cand_last[i]) + "]";
    }
    line += "]";
  }
  std::snprintf(num, sizeof num, ",\"ms\":%.3f,\"side\":%s}", ms, side ? "true" : "false");
  line += num;
  if (int(line.size()) + 1 > buf_len) return -1;
  std::memcpy(buf, line.c_str(), line.size() + 1);
  return int(line.size());
}

}  // extern "C"
