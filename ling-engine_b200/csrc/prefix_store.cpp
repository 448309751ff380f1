// The prefix KV store's host side: a byte arena's bookkeeping and the radix tree of prompt prefixes whose nodes hold
// references to KV pool pages and, at some ends, saved recurrent states.  Restates the paged mode of the reference's
// PrefixKvTree and its ArenaAlloc (src/core/prefix_kv.hpp:35-124, src/core/prefix_kv.cpp) behind a C interface with
// callbacks; the page size is a parameter here.  No device work: the engine facade supplies pages and state storage.
#include <algorithm>
#include <cstdint>
#include <map>
#include <utility>
#include <vector>

#include "../../include/ling_b200.h"

// ------------------------------------------------------------------------------------------------ the arena
struct ling_b200_arena {
  struct Range {
    size_t at, len;
  };
  size_t size = 0, align = 1, busy = 0;
  std::vector<Range> gaps;            // free ranges, ascending, never adjacent
  std::map<size_t, size_t> taken;     // offset -> length
};

extern "C" ling_b200_arena* ling_b200_arena_create(size_t size, size_t align) {
  if (align == 0) return nullptr;
  auto* a = new ling_b200_arena;
  a->align = align;
  a->size = size - size % align;
  if (a->size > 0) a->gaps.push_back({0, a->size});
  return a;
}
extern "C" void ling_b200_arena_destroy(ling_b200_arena* a) { delete a; }
extern "C" size_t ling_b200_arena_size(const ling_b200_arena* a) { return a ? a->size : 0; }
extern "C" size_t ling_b200_arena_in_use(const ling_b200_arena* a) { return a ? a->busy : 0; }

extern "C" long long ling_b200_arena_alloc(ling_b200_arena* a, size_t bytes) {
  if (!a) return -1;
  const size_t want = (bytes + a->align - 1) / a->align * a->align;
  for (size_t i = 0; i < a->gaps.size(); ++i) {  // first fit = the lowest offset that is large enough
    ling_b200_arena::Range& g = a->gaps[i];
    if (g.len < want) continue;
    const size_t at = g.at;
    if (g.len == want) a->gaps.erase(a->gaps.begin() + static_cast<long>(i));
    else g.at += want, g.len -= want;
    a->taken[at] = want;
    a->busy += want;
    return static_cast<long long>(at);
  }
  return -1;
}

extern "C" void ling_b200_arena_release(ling_b200_arena* a, size_t offset) {
  if (!a) return;
  const auto it = a->taken.find(offset);
  if (it == a->taken.end()) return;
  ling_b200_arena::Range r{it->first, it->second};
  a->busy -= r.len;
  a->taken.erase(it);
  auto& gaps = a->gaps;
  size_t i = 0;
  while (i < gaps.size() && gaps[i].at < r.at) ++i;  // r goes before gaps[i]
  if (i < gaps.size() && r.at + r.len == gaps[i].at) {
    r.len += gaps[i].len;
    gaps.erase(gaps.begin() + static_cast<long>(i));
  }
  if (i > 0 && gaps[i - 1].at + gaps[i - 1].len == r.at) gaps[i - 1].len += r.len;
  else gaps.insert(gaps.begin() + static_cast<long>(i), r);
}

// ------------------------------------------------------------------------------------------------ the tree
namespace {

struct Run {
  int up = -1;
  int first = 0, last = 0;           // the positions [first, last) after the parent's
  std::vector<int> toks;             // their tokens
  std::vector<int> held;             // one page id per page index first / PT .. (last - 1) / PT, a reference each
  std::map<std::pair<uint64_t, int>, int> below;  // children by (scope at the root, else 0; first token)
  uint64_t scope = 0, stamp = 0;
  void* state = nullptr;             // the recurrent state after exactly [0, last)
  bool live = false;
};

struct Walk {
  int len = 0;
  std::vector<int> path;
};

}  // namespace

struct ling_b200_prefix {
  size_t budget = 0, state_bytes = 0, bytes = 0;
  int pt = 64;
  ling_b200_prefix_ops ops{};
  std::vector<Run> runs;   // runs[0] is the root: the empty prefix
  std::vector<int> spare;  // dead slots, reused last in first out

  ling_b200_prefix() { reset(); }
  void reset() {
    runs.assign(1, Run{});
    runs[0].live = true;
    spare.clear();
    bytes = 0;
  }
  int page_of(int pos) const { return pos / pt; }
  std::pair<uint64_t, int> key(int parent, uint64_t scope, int token) const { return {parent == 0 ? scope : 0, token}; }
  bool alive(int id) const { return id > 0 && id < static_cast<int>(runs.size()) && runs[size_t(id)].live; }

  int fresh() {
    int id;
    if (!spare.empty()) {
      id = spare.back();
      spare.pop_back();
      runs[size_t(id)] = Run{};
    } else {
      runs.emplace_back();
      id = static_cast<int>(runs.size()) - 1;
    }
    runs[size_t(id)].live = true;
    return id;
  }

  Walk walk(const int* prompt, int n, uint64_t scope) const {
    Walk w;
    int at = 0;
    while (w.len < n) {
      const Run& here = runs[size_t(at)];
      const auto it = here.below.find(key(at, scope, prompt[w.len]));
      if (it == here.below.end()) break;
      const Run& r = runs[size_t(it->second)];
      const int width = r.last - r.first;
      int same = 0;
      while (same < width && w.len + same < n && r.toks[size_t(same)] == prompt[w.len + same]) ++same;
      w.path.push_back(it->second);
      w.len += same;
      if (same < width) break;
      at = it->second;
    }
    return w;
  }

  void touch(const int* path, int n_path, uint64_t epoch) {
    for (int i = 0; i < n_path; ++i)
      if (alive(path[i])) runs[size_t(path[i])].stamp = std::max(runs[size_t(path[i])].stamp, epoch);
  }

  // `id` keeps [first, at); a new child takes [at, last) with the tail's tokens, pages, children and state.  The page
  // that `at` falls inside (when it is not a page's first position) is then held by both: one more reference.
  int cut(int id, int at) {
    const int tail = fresh();  // may move runs: references are taken after it
    Run& head = runs[size_t(id)];
    Run& t = runs[size_t(tail)];
    const int base = page_of(head.first);
    t.up = id;
    t.first = at, t.last = head.last;
    t.toks.assign(head.toks.begin() + (at - head.first), head.toks.end());
    t.held.assign(head.held.begin() + (page_of(at) - base), head.held.end());
    t.scope = head.scope, t.stamp = head.stamp;
    t.state = std::exchange(head.state, nullptr);
    t.below = std::move(head.below);
    for (const auto& kv : t.below) runs[size_t(kv.second)].up = tail;
    head.toks.resize(size_t(at - head.first));
    head.held.resize(size_t(page_of(at - 1) - base + 1));
    head.last = at;
    head.below.clear();
    head.below[key(id, t.scope, t.toks[0])] = tail;
    if (at % pt != 0) ops.retain(ops.user, t.held.front());
    return tail;
  }

  void remove_leaf(int id) {
    Run& r = runs[size_t(id)];
    runs[size_t(r.up)].below.erase(key(r.up, r.scope, r.toks[0]));
    if (r.state) {
      ops.state_release(ops.user, r.state);
      bytes -= state_bytes;
    }
    for (int pg : r.held) ops.drop(ops.user, pg);
    r = Run{};
    spare.push_back(id);
  }

  // The least recently stamped live leaf that `spared` does not rule out; ties go to the lower id.
  template <class Spared>
  int oldest_leaf(Spared spared) const {
    int pick = -1;
    for (int i = 1; i < static_cast<int>(runs.size()); ++i) {
      const Run& r = runs[size_t(i)];
      if (!r.live || !r.below.empty() || spared(i, r)) continue;
      if (pick < 0 || r.stamp < runs[size_t(pick)].stamp) pick = i;
    }
    return pick;
  }

  bool make_room(size_t need, uint64_t epoch) {
    while (bytes + need > budget) {
      const int v = oldest_leaf([&](int, const Run& r) { return r.stamp >= epoch; });
      if (v < 0) return false;
      remove_leaf(v);
    }
    return true;
  }

  void clear() {
    for (Run& r : runs) {
      if (!r.live) continue;
      if (r.state) ops.state_release(ops.user, r.state);
      for (int pg : r.held) ops.drop(ops.user, pg);
    }
    reset();
  }
};

extern "C" {

ling_b200_prefix* ling_b200_prefix_create(size_t budget_bytes, size_t state_bytes, int page_tokens, const ling_b200_prefix_ops* ops) {
  if (!ops || !ops->hold || !ops->retain || !ops->drop || !ops->state_alloc || !ops->state_release || page_tokens <= 0) return nullptr;
  auto* t = new ling_b200_prefix;
  t->budget = budget_bytes, t->state_bytes = state_bytes, t->pt = page_tokens, t->ops = *ops;
  return t;
}

void ling_b200_prefix_destroy(ling_b200_prefix* t) {
  if (!t) return;
  t->clear();
  delete t;
}

int ling_b200_prefix_match(const ling_b200_prefix* t, const int* prompt, int n, uint64_t scope, int* path, int cap, int* n_path) {
  if (!t || (n > 0 && !prompt)) return 0;
  const Walk w = t->walk(prompt, std::max(n, 0), scope);
  const int count = static_cast<int>(w.path.size());
  if (n_path) *n_path = count;
  for (int i = 0; i < std::min(count, path ? cap : 0); ++i) path[i] = w.path[size_t(i)];
  return w.len;
}

int ling_b200_prefix_best_state(const ling_b200_prefix* t, const int* path, int n_path, int len, int limit, void** state) {
  int best = 0;
  if (state) *state = nullptr;
  if (!t) return 0;
  for (int i = 0; i < n_path; ++i) {
    if (!t->alive(path[i])) break;
    const Run& r = t->runs[size_t(path[i])];
    if (r.last > len || r.last > limit) break;
    if (r.state) {
      best = r.last;
      if (state) *state = r.state;
    }
  }
  return best;
}

int ling_b200_prefix_pages(const ling_b200_prefix* t, const int* path, int n_path, int n, int* pages, int cap) {
  if (!t || n < 0) return -1;
  const int count = (n + t->pt - 1) / t->pt;
  if (count > cap) return -1;
  std::fill(pages, pages + count, 0);
  // Shallow to deep: where two nodes hold the same page index, the deeper one's page is the one this prompt wrote last.
  for (int i = 0; i < n_path; ++i) {
    if (!t->alive(path[i])) break;
    const Run& r = t->runs[size_t(path[i])];
    if (r.first >= n) break;
    const int lo = t->page_of(r.first), hi = std::min(t->page_of(r.last - 1), count - 1);
    for (int j = lo; j <= hi; ++j) pages[j] = r.held[size_t(j - lo)];
  }
  return count;
}

void ling_b200_prefix_touch(ling_b200_prefix* t, const int* path, int n_path, uint64_t epoch) {
  if (t) t->touch(path, n_path, epoch);
}

int ling_b200_prefix_insert(ling_b200_prefix* t, const int* prompt, int n, int q, const int* cuts, int n_cuts, uint64_t epoch,
                            uint64_t scope, int* want_node, int* want_pos, int cap) {
  if (!t || !prompt) return 0;
  q = std::min(q, n);
  if (q <= 0) return 0;
  // Every boundary inside what the tree already holds becomes a node end: where the match stops, and each cut.
  Walk w = t->walk(prompt, q, scope);
  if (!w.path.empty() && t->runs[size_t(w.path.back())].last > w.len) t->cut(w.path.back(), w.len);
  for (int i = 0; i < n_cuts; ++i) {
    const int c = cuts[i];
    if (c <= 0 || c >= w.len) continue;
    for (int id : t->walk(prompt, q, scope).path)
      if (t->runs[size_t(id)].first < c && c < t->runs[size_t(id)].last) {
        t->cut(id, c);
        break;
      }
  }
  w = t->walk(prompt, q, scope);
  t->touch(w.path.data(), static_cast<int>(w.path.size()), epoch);
  if (w.len < q) {
    // The rest stays in the session's pages: a chain of new nodes, one per cut and one to q, each holding the pages under it.
    int parent = w.path.empty() ? 0 : w.path.back();
    int from = w.len;
    std::vector<int> ends;
    for (int i = 0; i < n_cuts; ++i)
      if (cuts[i] > w.len && cuts[i] < q) ends.push_back(cuts[i]);
    ends.push_back(q);
    for (int e : ends) {
      if (e <= from) continue;
      const int want = t->page_of(e - 1) - t->page_of(from) + 1;
      std::vector<int> got(size_t(want), 0);
      const int n_got = t->ops.hold(t->ops.user, from, e, got.data(), want);
      const bool whole = n_got == want && std::find(got.begin(), got.end(), 0) == got.end();
      if (!whole) {
        for (int j = 0; j < std::min(std::max(n_got, 0), want); ++j)
          if (got[size_t(j)] != 0) t->ops.drop(t->ops.user, got[size_t(j)]);
        break;
      }
      const int id = t->fresh();
      Run& r = t->runs[size_t(id)];
      r.up = parent;
      r.first = from, r.last = e;
      r.toks.assign(prompt + from, prompt + e);
      r.held = std::move(got);
      r.scope = scope, r.stamp = epoch;
      t->runs[size_t(parent)].below[t->key(parent, scope, r.toks[0])] = id;
      parent = id;
      from = e;
    }
    w = t->walk(prompt, q, scope);
  }
  int n_want = 0;
  for (int i = 0; i < n_cuts; ++i)
    for (int id : w.path)
      if (t->runs[size_t(id)].last == cuts[i] && cuts[i] <= w.len) {
        if (!t->runs[size_t(id)].state) {
          if (n_want < cap && want_node && want_pos) want_node[n_want] = id, want_pos[n_want] = cuts[i];
          ++n_want;
        }
        break;
      }
  return n_want;
}

void* ling_b200_prefix_add_state(ling_b200_prefix* t, int node, uint64_t epoch) {
  if (!t || !t->alive(node) || t->runs[size_t(node)].state) return nullptr;
  if (!t->make_room(t->state_bytes, epoch)) return nullptr;
  if (!t->alive(node)) return nullptr;  // a node stamped before `epoch` may itself have been what made the room
  void* p = t->ops.state_alloc(t->ops.user, t->state_bytes);
  if (!p) return nullptr;
  Run& r = t->runs[size_t(node)];
  r.state = p;
  r.stamp = std::max(r.stamp, epoch);
  t->bytes += t->state_bytes;
  return p;
}

int ling_b200_prefix_evict_lru_leaf(ling_b200_prefix* t, const int* keep, int n_keep) {
  if (!t) return 0;
  const int v = t->oldest_leaf([&](int id, const Run&) { return std::find(keep, keep + n_keep, id) != keep + n_keep; });
  if (v < 0) return 0;
  t->remove_leaf(v);
  return 1;
}

void ling_b200_prefix_clear(ling_b200_prefix* t) {
  if (t) t->clear();
}
size_t ling_b200_prefix_bytes(const ling_b200_prefix* t) { return t ? t->bytes : 0; }
size_t ling_b200_prefix_budget(const ling_b200_prefix* t) { return t ? t->budget : 0; }
int ling_b200_prefix_nodes(const ling_b200_prefix* t) {
  return t ? static_cast<int>(std::count_if(t->runs.begin() + 1, t->runs.end(), [](const Run& r) { return r.live; })) : 0;
}
int ling_b200_prefix_states(const ling_b200_prefix* t) {
  return t ? static_cast<int>(std::count_if(t->runs.begin() + 1, t->runs.end(), [](const Run& r) { return r.live && r.state; })) : 0;
}
int ling_b200_prefix_pages_held(const ling_b200_prefix* t) {
  int n = 0;
  if (t)
    for (size_t i = 1; i < t->runs.size(); ++i)
      if (t->runs[i].live) n += static_cast<int>(t->runs[i].held.size());
  return n;
}

int ling_b200_prefix_page_lists(const ling_b200_prefix* t, const int* skip, int n_skip, int* pages, int cap_pages, int* lens,
                                int cap_lists) {
  if (!t) return 0;
  int lists = 0, used = 0;
  for (int i = 1; i < static_cast<int>(t->runs.size()); ++i) {
    const Run& r = t->runs[size_t(i)];
    if (!r.live || r.held.empty() || std::find(skip, skip + n_skip, i) != skip + n_skip) continue;
    if (lists >= cap_lists || used + static_cast<int>(r.held.size()) > cap_pages) return -1;
    std::copy(r.held.begin(), r.held.end(), pages + used);
    used += static_cast<int>(r.held.size());
    lens[lists++] = static_cast<int>(r.held.size());
  }
  return lists;
}

}  // extern "C"
