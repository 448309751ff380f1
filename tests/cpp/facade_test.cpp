// facade_test.cpp -- a caller written against the reference's C++ names (ling::Engine::speculate_batch, ling::KvPool,
// ling::describe_tree, ling::serve::select_batch ...) compiled against the facade header and linked to libling_b200.so.
//   facade_test host   host logic only (no GPU)
//   facade_test gpu    also drives two sessions through Engine::speculate_batch on the toy configuration
#include <cstdio>
#include <cstring>
#include <numeric>

#include "ling_engine.hpp"

static int failures = 0;
#define EXPECT(cond)                                         \
  do {                                                       \
    if (!(cond)) {                                           \
      std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); \
      ++failures;                                            \
    }                                                        \
  } while (0)

static ling::DraftTree two_branch(int anchor, int chain_rows, int branch_rows, int seed) {
  ling::DraftTree t;
  t.E = chain_rows - 1;
  for (int r = 0; r < chain_rows + branch_rows; ++r) {
    t.parent.push_back(r == 0 ? -1 : r < chain_rows ? r - 1 : r == chain_rows ? 0 : r - 1);
    t.depth.push_back(r == 0 ? 0 : t.depth[t.parent[r]] + 1);
    t.token.push_back(r == 0 ? anchor : (seed * 7919 + r * 104729) % 4096);
    t.pick.push_back(0);
  }
  t.children.assign(t.parent.size(), {});
  for (int r = 1; r < t.rows(); ++r) t.children[t.parent[r]].push_back(r);
  return t;
}

static void host_checks() {
  // the tree description of a 16-row chain plus a 4-row branch off the anchor: two variants, two DeltaNet paths
  ling::kernels::TreeDesc d;
  const ling::DraftTree t = two_branch(1000, 16, 4, 1);
  EXPECT(ling::describe_tree(t, d) == 2 && d.nvar == 2 && d.n == 20);
  EXPECT(d.gdn_len[0] == 17 && d.gdn_len[1] == 5 && d.gdn_step[1][0] == 0);
  EXPECT(d.gdn_step[0][15] == (15 | ling::kernels::TreeDesc::kLeaf | ling::kernels::TreeDesc::kWrite));
  std::vector<int> argmax(20, -1);
  argmax[0] = t.token[16], argmax[16] = t.token[17], argmax[17] = 4242;
  int next = 0;
  const std::vector<int> path = ling::accept_tree_greedy(t, argmax.data(), next);
  EXPECT((path == std::vector<int>{0, 16, 17}) && next == 4242);
  const ling::LookupProposal p = ling::lookup_propose({1, 2, 3, 4, 5, 9, 1, 2, 3}, 2);
  EXPECT((p.tokens == std::vector<int>{4, 5}) && p.match == 3);
  // page bookkeeping with 16-position pages: copy-on-write and deferred frees
  ling::KvPool pool(8, 16);
  std::vector<int> a, b;
  std::vector<ling::KvPool::Copy> copies;
  EXPECT(pool.ensure(a, 0, 40, &copies) && (a == std::vector<int>{1, 2, 3}) && copies.empty());
  pool.share(b, a, 20);
  EXPECT((b == std::vector<int>{1, 2}) && pool.refs(2) == 2 && pool.needed(b, 18, 19) == 1);
  EXPECT(pool.ensure(b, 18, 19, &copies) && (b == std::vector<int>{1, 4}) && copies.size() == 1 && copies[0].src == 2);
  EXPECT(!pool.ensure(b, 32, 128, &copies) && pool.free_pages() == 3);
  pool.truncate(a, 16);
  EXPECT(pool.pending_pages() == 2 && pool.free_pages() == 3);
  pool.retire();
  EXPECT(pool.free_pages() == 5);
  // pairing and pool policy
  using namespace ling::serve;
  const std::vector<PairCandidate> c = {{true, 3, 9}, {true, 1, 4}, {false, 0, 0}, {true, 1, 2}};
  EXPECT((select_batch(c, 0, 2, true) == std::vector<size_t>{0, 3}) && (select_batch(c, 0, 2, false) == std::vector<size_t>{0, 1}));
  EXPECT(select_batch(c, 2, 2, true).empty());
  EXPECT(kv_verdict(3, {4, 0, 0}) == KvVerdict::Go && kv_verdict(5, {4, 2, 0}) == KvVerdict::Retire &&
         kv_verdict(9, {4, 2, 5}) == KvVerdict::Reclaim && kv_verdict(99, {4, 2, 5}) == KvVerdict::Wait);
  EXPECT(kv_last_resort({{1, true, 50}, {7, true, 60}}, {1, 1, 1}) == 1 && kv_last_resort({{1, true, 50}, {7, false, 60}}, {1, 1, 1}) == -1);
  {
    // kv_reclaim with the reference's std::function arguments: two idle sessions of 3 pages each; the unit needs 5
    int need = 5, have = 1, idle_left = 2, source_left = 1;
    const std::vector<KvEvictNext> kept = {[&] { return idle_left > 0 ? (--idle_left, have += 3, true) : false; }};
    const std::vector<KvEvictNext> source = {[&] { return source_left > 0 ? (--source_left, have += 9, need += 2, true) : false; }};
    EXPECT(kv_reclaim([&] { return need; }, [&] { return have; }, kept, 5, 7, source, 7, 16, false) && idle_left == 0 && source_left == 1);
    need = 20, have = 1, idle_left = 2;
    EXPECT(!kv_reclaim([&] { return need; }, [&] { return have; }, kept, 20, 7, source, 22, 16, false) && idle_left == 2);   // nothing evicted
    EXPECT(refuse_request(9000, 8192).empty() && refuse_request(-1, 8192).empty());
    EXPECT(refuse_request(100, 8192) == "host memory low: 100 MB available, below the 8192 MB this server keeps free; the request was not started (retry later)");
  }
  StepRecord rec;
  rec.t = 1.5, rec.pass = 12, rec.turn = 1, rec.sessions = {0, 2}, rec.rows = {12, 12}, rec.tokens = {5, 7}, rec.left = {0, 0};
  rec.cand = {{0, 3, 1, 2, 11}}, rec.ms = 121.75, rec.side = false;
  EXPECT(format_step(rec) == "{\"t\":1.500000,\"pass\":12,\"kind\":\"decode\",\"turn\":1,\"sessions\":[0,2],\"rows\":[12,12],"
                            "\"tokens\":[5,7],\"left\":[0,0],\"cand\":[[0,3,1,2,11]],\"ms\":121.750,\"side\":false}");
  PassWindow w;
  for (long p2 = 1; p2 <= 20; ++p2) w.record(p2);
  EXPECT(w.count(20) == 16 && w.last() == 20);
}

static ling::ModelConfig toy_config() {
  ling::ModelConfig c{};
  c.hidden = 256, c.intermediate = 704, c.layers = 4, c.vocab = 4096, c.heads = 4, c.kv_heads = 1, c.head_dim = 64, c.rotary_dim = 16;
  c.rope_theta = 1e7f, c.eps = 1e-6f, c.lin_k_heads = 2, c.lin_v_heads = 4, c.lin_k_dim = 64, c.lin_v_dim = 64, c.conv_kernel = 4;
  c.full_attention[3] = 1;
  return c;
}

static void gpu_checks() {
  ling::EngineOptions o;
  o.max_context = 2048, o.sessions = 3, o.max_seqs = 3, o.max_rows = 96;
  ling::SamplingParams greedy;
  greedy.temperature = 0.f;
  auto make = [&](ling::Engine& e) {
    ling_b200_synth_weights(e.handle(), 0);
    for (int s = 0; s < 3; ++s) {
      std::vector<int> ctx(40 + 100 * s);
      std::iota(ctx.begin(), ctx.end(), 5);
      e.adopt_context(s, ctx);
      ling_b200_synth_kv(e.handle(), s, int(ctx.size()), 3);
      ling_b200_synth_state(e.handle(), s, 3);
    }
    e.set_tree_source([](int session, int anchor, const std::vector<int>& history) {
      return two_branch(anchor, 16, 4, session + int(history.size()));
    });
  };
  ling::Engine batch(toy_config(), o), alone(toy_config(), o);
  make(batch), make(alone);
  EXPECT(batch.can_batch(0, greedy) && batch.kv_pages_total() == 3 * 128 && batch.kv_step_need(0, true) >= 1);
  std::vector<int> anchor = {11, 22, 33};
  for (int step = 0; step < 4; ++step) {
    std::vector<ling::Engine::SeqStep> q(3);
    for (int s = 0; s < 3; ++s) q[s].session = s, q[s].anchor = anchor[s], q[s].params = &greedy;
    batch.speculate_batch(q);
    for (int s = 0; s < 3; ++s) {
      EXPECT(!q[s].error && !q[s].out.empty());
      alone.select_session(s);
      const uint64_t before = alone.state_hash();
      const std::vector<int> out = alone.speculate(anchor[s], greedy);  // each sequence's step alone: the same tokens
      EXPECT(out == q[s].out && alone.state_hash() != before);
      batch.select_session(s);
      EXPECT(batch.state_hash() == alone.state_hash() && batch.position(s) == alone.position(s));
      EXPECT(int(batch.history().size()) == batch.position(s));
      anchor[s] = q[s].out.back();
    }
  }
  // a session twice in one batch is refused before anything runs
  std::vector<ling::Engine::SeqStep> bad(2);
  bad[0].session = bad[1].session = 1, bad[0].params = bad[1].params = &greedy;
  bool threw = false;
  try {
    batch.speculate_batch(bad);
  } catch (const std::runtime_error&) {
    threw = true;
  }
  EXPECT(threw);
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
