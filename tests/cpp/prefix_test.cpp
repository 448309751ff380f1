// prefix_test.cpp -- the prefix KV store through the C++ facade (ling-engine_b200/csrc/host/ling_engine.hpp).
//   prefix_test host   PrefixKvTree and ArenaAlloc as classes over a KvPool, the way the reference's own test drives its
//                      (tests/prefix_kv_tests.cpp, paged mode): page references, copy-on-write of a page two prompts share
//   prefix_test gpu    the real Engine on the toy configuration, prefill by the verify pass over linear chains: a prompt that
//                      resumes from the store (pages mapped by reference, the state restored, the shared page copied before
//                      it is written) ends with the same state bits and the same tokens as the same prompt prefilled from
//                      nothing on an engine without a store, and the conversation whose pages are shared is not disturbed
#include <cstdio>
#include <cstring>
#include <map>

#include "ling_scheduler.hpp"

static int failures = 0;
#define EXPECT(cond)                                                \
  do {                                                              \
    if (!(cond)) {                                                  \
      std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); \
      ++failures;                                                   \
    }                                                               \
  } while (0)

static std::vector<int> prompt_of(const std::vector<int>& shared, int salt, int n) {
  std::vector<int> p = shared;
  unsigned x = unsigned(salt) * 2654435761u + 1u;
  for (int i = 0; i < n; ++i) {
    x = x * 1664525u + 1013904223u;
    p.push_back(100 + int((x >> 8) % 3900u));
  }
  return p;
}

// ---------------------------------------------------------------------------------------------- host
namespace {
constexpr int PT = 64;
constexpr size_t kState = 1 << 16;
struct Paged {  // a pool, one active session's table, each page's contents: a hash of the whole prompt up to each position
  ling::KvPool pool{400, PT};
  std::map<int, std::vector<uint64_t>> mem;
  std::vector<int> table;
  int states = 0;
  static uint64_t kv_at(const std::vector<int>& p, int pos) {
    uint64_t h = 1469598103934665603ull;
    for (int i = 0; i <= pos; ++i) h = (h ^ uint64_t(p[size_t(i)] + 7)) * 1099511628211ull;
    return h;
  }
  ling::PrefixKvTree::Ops ops() {
    ling::PrefixKvTree::Ops o;
    o.alloc = [this](size_t n) { return ++states, std::malloc(n); };
    o.release = [this](void* p) { --states, std::free(p); };
    o.hold = [this](int from, int to) {
      std::vector<int> out;
      for (int i = from / PT; i <= (to - 1) / PT; ++i) {
        const int pg = i < int(table.size()) ? table[size_t(i)] : 0;
        if (pg) pool.retain(pg);
        out.push_back(pg);
      }
      return out;
    };
    o.retain = [this](int pg) { pool.retain(pg); };
    o.drop = [this](int pg) { pool.release(pg); };
    return o;
  }
  void end_session() {
    for (int pg : table)
      if (pg) pool.release(pg);
    table.clear();
  }
  void run(const std::vector<int>& p, const std::vector<int>& from_store, int n) {
    end_session();
    for (int pg : from_store) pool.retain(pg), table.push_back(pg);
    std::vector<ling::KvPool::Copy> copies;
    EXPECT(pool.ensure(table, n, int(p.size()), &copies));
    for (const auto& c : copies) mem[c.dst] = mem[c.src];
    for (int pos = n; pos < int(p.size()); ++pos) {
      const int pg = table[size_t(pos / PT)];
      EXPECT(pool.refs(pg) == 1);  // a shared page is never written
      mem[pg].resize(PT, 0);
      mem[pg][size_t(pos % PT)] = kv_at(p, pos);
    }
  }
  int live_pages() const {
    int n = 0;
    for (int pg = 1; pg < pool.capacity(); ++pg) n += pool.refs(pg) > 0;
    return n;
  }
};
}  // namespace

static void host_checks() {
  {  // the arena: first fit, merging
    ling::ArenaAlloc a(1000, 64);
    size_t x = 0, y = 0, z = 0;
    EXPECT(a.size() == 960 && a.alloc(100, &x) && a.alloc(100, &y) && a.alloc(700, &z) && x == 0 && y == 128 && z == 256);
    EXPECT(a.in_use() == 960 && !a.alloc(1, &x));
    a.release(128);
    a.release(0);
    EXPECT(a.alloc(200, &x) && x == 0 && a.in_use() == 960);
  }
  {  // two prompts that diverge inside a page: the second maps the first's pages and copies the straddling one
    Paged h;
    ling::PrefixKvTree t(2 * kState, 0, kState, h.ops(), PT);
    std::vector<int> sys;
    for (int i = 0; i < 100; ++i) sys.push_back(i);
    const std::vector<int> a = prompt_of(sys, 1, 60), b = prompt_of(sys, 2, 60);
    h.run(a, {}, 0);
    auto want = t.insert(a, 160, {96}, 1);
    EXPECT(t.nodes() == 2 && want.size() == 1 && want[0].second == 96 && t.add_state(want[0].first, 1) && t.states() == 1);
    const auto mb = t.match(b);
    const void* st = nullptr;
    EXPECT(mb.len == 100 && t.best_state(mb, 99, &st) == 96 && st != nullptr);
    h.run(b, t.pages(mb, 96), 96);
    t.insert(b, 160, {96}, 2);
    EXPECT(t.nodes() == 4);  // [0,96) [96,100) and the two tails
    for (const auto& p : {a, b}) {
      const auto m = t.match(p);
      const std::vector<int> pg = t.pages(m, 160);
      bool same = m.len == 160;
      for (int pos = 0; pos < 160 && same; ++pos) same = h.mem[pg[size_t(pos / PT)]][size_t(pos % PT)] == Paged::kv_at(p, pos);
      EXPECT(same);
    }
    EXPECT(t.pages(t.match(a), 160)[0] == t.pages(t.match(b), 160)[0] && t.pages(t.match(a), 160)[1] != t.pages(t.match(b), 160)[1]);
    EXPECT(t.page_lists().size() == 4 && t.pages_held() >= 6);
    EXPECT(t.evict_lru_leaf(t.match(b).path) && t.match(a).len == 100 && t.match(b).len == 160);
    h.end_session();
    t.clear();
    EXPECT(h.live_pages() == 0 && h.states == 0 && t.bytes() == 0);
  }
  {  // an Ops without its callbacks is refused
    bool threw = false;
    try {
      ling::PrefixKvTree t(0, 0, kState, ling::PrefixKvTree::Ops{}, PT);
    } catch (const std::invalid_argument&) {
      threw = true;
    }
    EXPECT(threw);
  }
}

// ---------------------------------------------------------------------------------------------- the real engine
static ling::ModelConfig toy_config() {
  ling::ModelConfig c{};
  c.hidden = 256, c.intermediate = 704, c.layers = 4, c.vocab = 4096;
  c.heads = 4, c.kv_heads = 1, c.head_dim = 64, c.rotary_dim = 16, c.rope_theta = 1e6f, c.eps = 1e-6f;
  c.lin_k_heads = 2, c.lin_v_heads = 4, c.lin_k_dim = 64, c.lin_v_dim = 64, c.conv_kernel = 4;
  c.full_attention[3] = 1;
  return c;
}
static ling::DraftTree chain_tree(int anchor, int rows, int seed) {
  ling::DraftTree t;
  t.E = rows - 1;
  for (int r = 0; r < rows; ++r) {
    t.parent.push_back(r - 1);
    t.depth.push_back(r);
    t.token.push_back(r == 0 ? anchor : (seed * 7919 + r * 104729) % 4096);
    t.pick.push_back(0);
  }
  t.children.assign(t.parent.size(), {});
  for (int r = 1; r < rows; ++r) t.children[size_t(r - 1)].push_back(r);
  return t;
}
static void setup(ling::Engine& e) {
  ling_b200_synth_weights(e.handle(), 0);
  e.set_tree_source([](int, int anchor, const std::vector<int>& history) { return chain_tree(anchor, 6, anchor + int(history.size())); });
  e.use_chain_prefill();
}
// Prefill, then `steps` decode passes; the tokens, and the state's hash right after the prefill.
struct Served {
  std::vector<int> tokens;
  uint64_t hash_after_prefill = 0;
};
static Served serve(ling::Engine& e, int session, const std::vector<int>& prompt, int steps) {
  Served out;
  static const ling::SamplingParams greedy{0.f};
  e.activate_session(session, "", true);
  int anchor = e.begin_prefill(session, prompt);
  e.select_session(session);
  out.hash_after_prefill = e.state_hash();
  out.tokens.push_back(anchor);
  for (int i = 0; i < steps; ++i) {
    const std::vector<int> got = e.speculate(anchor, greedy);
    out.tokens.insert(out.tokens.end(), got.begin(), got.end());
    anchor = got.back();
  }
  return out;
}
static void decode_more(ling::Engine& e, int session, Served& s, int steps) {
  static const ling::SamplingParams greedy{0.f};
  e.select_session(session);
  int anchor = s.tokens.back();
  for (int i = 0; i < steps; ++i) {
    const std::vector<int> got = e.speculate(anchor, greedy);
    s.tokens.insert(s.tokens.end(), got.begin(), got.end());
    anchor = got.back();
  }
}

static void gpu_checks() {
  constexpr int kBoundary = 7;
  ling::EngineOptions o;
  o.max_context = 1024, o.sessions = 3, o.max_seqs = 2, o.max_rows = 64, o.page_tokens = 64, o.boundary_token = kBoundary;
  o.kv_pool_pages = 3 * 16;
  ling::EngineOptions with_store = o;
  with_store.prefix_kv_mb = 8;

  // A system message of 110 tokens after the boundary token, then the user's: the store keeps [0, 96) (the end of the second
  // message boundary at position 111, aligned down to 96), which is inside page 1 of 64-token pages.
  std::vector<int> sys{kBoundary};
  for (int i = 0; i < 110; ++i) sys.push_back(1000 + i * 3);
  sys.push_back(kBoundary);
  const std::vector<int> p1 = prompt_of(sys, 11, 50), p2 = prompt_of(sys, 22, 70), p3 = prompt_of(sys, 33, 20);

  // What each prompt gives on an engine without a store, prefilled from nothing.
  Served alone1, alone2, alone3;
  {
    ling::Engine plain(toy_config(), o);
    setup(plain);
    alone1 = serve(plain, 0, p1, 6);
    alone2 = serve(plain, 1, p2, 6);
    alone3 = serve(plain, 2, p3, 4);
    EXPECT(plain.last_prefill().reused_tokens == 0 && !plain.kv_store_on());
  }

  ling::Engine eng(toy_config(), with_store);
  setup(eng);
  EXPECT(eng.kv_store_on() && eng.kv_store()->nodes() == 0);
  const int cold2 = eng.kv_admit_need(1, p2, 0);
  Served s1 = serve(eng, 0, p1, 3);
  EXPECT(s1.hash_after_prefill == alone1.hash_after_prefill);
  EXPECT(eng.last_prefill().reused_tokens == 0 && eng.last_prefill().chunks == 2);  // [0, 96) and the rest
  EXPECT(eng.kv_store()->nodes() == 1 && eng.kv_store()->states() == 1 && eng.kv_store()->pages_held() == 2);
  const std::vector<int> shared = eng.book().at(0).table;
  EXPECT(eng.book().pool().refs(shared[0]) == 2 && eng.book().pool().refs(shared[1]) == 2 && eng.book().pool().refs(shared[2]) == 1);

  // The second conversation resumes from the store: two pages by reference, one of them copied before it is written.
  const int warm2 = eng.kv_admit_need(1, p2, 0);
  EXPECT(warm2 == cold2 - 1);  // page 0 is not taken again; page 1 is, as a copy
  EXPECT(eng.kv_store_path(1, p2, 0).size() == 1 && eng.kv_store_path(1, p2, 0) == eng.kv_store()->match(p2).path);
  Served s2 = serve(eng, 1, p2, 6);
  EXPECT(eng.last_prefill().store_tokens == 96 && eng.last_prefill().reused_tokens == 96 && eng.last_prefill().prefill_tokens == int(p2.size()) - 96);
  EXPECT(s2.hash_after_prefill == alone2.hash_after_prefill);
  EXPECT(s2.tokens == alone2.tokens);
  const std::vector<int>& t1 = eng.book().at(1).table;
  EXPECT(t1[0] == shared[0] && t1[1] != shared[1]);
  EXPECT(eng.book().pool().refs(shared[0]) == 3 && eng.book().pool().refs(shared[1]) == 2 && eng.book().pool().refs(t1[1]) == 1);
  EXPECT(eng.kv_store()->nodes() == 1);  // nothing new to keep: the same beginning

  // The first conversation goes on undisturbed.
  decode_more(eng, 0, s1, 3);
  EXPECT(s1.tokens == alone1.tokens);

  // A third prompt, with the first conversation's session evicted: the store still holds the beginning.
  eng.kv_evict(0);
  eng.kv_retire(true);
  EXPECT(eng.book().pool().refs(shared[0]) == 2 && eng.book().pool().refs(shared[1]) == 1);
  Served s3 = serve(eng, 2, p3, 4);
  EXPECT(eng.last_prefill().store_tokens == 96 && s3.hash_after_prefill == alone3.hash_after_prefill && s3.tokens == alone3.tokens);

  // The same prompt again in its own session, extended: resumes from its own history, not from the store.
  std::vector<int> p2b = p2;
  p2b.insert(p2b.end(), s2.tokens.begin(), s2.tokens.end() - 1);
  EXPECT(eng.book().at(1).history == p2b);
  p2b.push_back(kBoundary), p2b.push_back(1234), p2b.push_back(2345);
  eng.activate_session(1, "", false);
  eng.begin_prefill(1, p2b);
  EXPECT(eng.last_prefill().reused_tokens == int(p2b.size()) - 3 && eng.last_prefill().store_tokens == 0);

  // from_scratch ignores both and still gives the same state.
  eng.activate_session(2, "", true);
  eng.begin_prefill(2, p3, 0, true);
  eng.select_session(2);
  EXPECT(eng.last_prefill().reused_tokens == 0 && eng.state_hash() == alone3.hash_after_prefill);

  // The store's pages are the pool's first reclaimable memory.
  EXPECT(eng.kv_store_pages() >= 0 && eng.kv_store_evict() && !eng.kv_store_evict() && eng.kv_store()->nodes() == 0);
  EXPECT(eng.kv_store()->bytes() == 0 && eng.kv_store_pages() == 0);
  std::printf("prefix store: resumed %d of %zu tokens from the store, state and tokens equal to a prefill from nothing\n", 96, p2.size());

  // Under the scheduler: conversations over three system messages queue up for two session slots and a pool of 11 pages
  // (two running requests take up to 5 each), so the store's entries have to be given up for pages now and then.  Whatever
  // is resumed, evicted or prefilled again, every request produces what it produces alone on an engine without a store.
  std::vector<std::vector<int>> systems;
  for (int k = 0; k < 3; ++k) {
    std::vector<int> m{kBoundary};
    for (int i = 0; i < 110; ++i) m.push_back(500 + 700 * k + i * 5);
    m.push_back(kBoundary);
    systems.push_back(m);
  }
  std::vector<ling::serve::Request> reqs;
  const int order[8] = {0, 1, 0, 2, 1, 0, 2, 1};
  for (int i = 0; i < 8; ++i) {
    ling::serve::Request r;
    r.prompt = prompt_of(systems[size_t(order[i])], 100 + i, 30 + 9 * i);
    r.max_tokens = 8 + i;
    r.sampling.temperature = 0.f;
    reqs.push_back(r);
  }
  ling::EngineOptions small = o;
  small.sessions = 2, small.kv_pool_pages = 11;
  std::map<size_t, std::vector<int>> alone;  // by prompt length (all different)
  {
    ling::Engine plain(toy_config(), small);
    setup(plain);
    ling::serve::Scheduler sch(plain, 1);
    for (const ling::serve::Request& r : reqs) {
      sch.submit(r);
      sch.run_until_idle();
      const std::vector<ling::serve::Finished> f = sch.take_finished();
      EXPECT(f.size() == 1 && f[0].finish == "length" && int(f[0].tokens.size()) == r.max_tokens);
      alone[r.prompt.size()] = f[0].tokens;
    }
  }
  small.prefix_kv_mb = 8;
  ling::Engine shared_eng(toy_config(), small);
  setup(shared_eng);
  ling::serve::Scheduler sch(shared_eng, 2);
  std::map<long, size_t> len_of;
  for (const ling::serve::Request& r : reqs) len_of[sch.submit(r)] = r.prompt.size();
  sch.run_until_idle();
  const std::vector<ling::serve::Finished> done = sch.take_finished();
  EXPECT(done.size() == 8);
  for (const ling::serve::Finished& f : done) EXPECT(f.finish == "length" && f.tokens == alone[len_of[f.id]]);
  EXPECT(sch.stats().kv_store_evictions > 0 && sch.stats().batched_steps > 0);
  std::printf("scheduler with the store: %ld store entries and %ld idle sessions evicted for pages, %ld decode passes (%ld shared)\n",
              sch.stats().kv_store_evictions, sch.stats().kv_evictions, sch.stats().decode_passes, sch.stats().batched_steps);
}

int main(int argc, char** argv) {
  host_checks();
  if (argc > 1 && std::strcmp(argv[1], "gpu") == 0) {
    if (ling_b200_device_count() < 1) {
      std::printf("no CUDA device\n");
      return 2;
    }
    gpu_checks();
  }
  std::printf(failures ? "%d check(s) failed\n" : "all checks passed\n", failures);
  return failures ? 1 : 0;
}
