// scheduler_test.cpp -- the headless scheduler (ling-engine_b200/csrc/host/ling_scheduler.hpp) driven the way the
// reference's server drives its own: jobs in, turns, finished requests out.
//   scheduler_test host   against a host-only engine (the session book and the page pool are the library's, a step accepts a
//                         scripted number of tokens): admission, turn order, batching, pairing, page pressure, last resort
//   scheduler_test gpu    the real Engine on the toy configuration: every request's tokens under continuous batching equal
//                         the tokens of the same request served alone
#include <cstdio>
#include <cstring>
#include <map>
#include <numeric>
#include <random>

#include "ling_scheduler.hpp"

static int failures = 0;
#define EXPECT(cond)                                                \
  do {                                                              \
    if (!(cond)) {                                                  \
      std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); \
      ++failures;                                                   \
    }                                                               \
  } while (0)

using ling::serve::Finished;
using ling::serve::Request;

// The scheduler's view of an engine without a device: sessions and pages are the library's, a step accepts accept(session, pos)
// tokens (the anchor included) whose values are a function of the session's position.
struct HostEngine {
  struct SeqStep {
    int session = -1, anchor = 0;
    const ling::SamplingParams* params = nullptr;
    std::vector<int> out;
    std::exception_ptr error;
  };
  ling::SessionBook book;
  int max_batch_;
  double now = 0;
  std::function<int(int, int)> accept = [](int, int) { return 3; };
  std::vector<std::vector<int>> passes;  // the sessions of every verify pass, in order
  long evictions = 0, kv_evictions_ = 0;
  HostEngine(int sessions, int pool_pages, int max_context, int max_batch) : book(sessions, pool_pages, 16, max_context), max_batch_(max_batch) {
    book.clock = [this] { return now; };
  }
  int sessions() const { return book.sessions(); }
  int max_context() const { return book.max_context(); }
  int max_batch() const { return max_batch_; }
  int match_session(const std::vector<int>& p, const std::string& k, uint64_t s) const { return book.match_session(p, k, s); }
  int free_session(double protect, const std::vector<bool>& pinned) const { return book.free_session(protect, pinned); }
  void activate_session(int i, const std::string& k, bool fresh, uint64_t scope) {
    if (book.activate(i, k, fresh, scope)) ++evictions;
  }
  void touch_session(int i) { book.touch(i); }
  int kv_admit_pages(size_t n) const { return book.kv_admit_pages(n); }
  int kv_pages_total() const { return book.pool().capacity(); }
  int kv_pages_free() { return book.pool().free_pages(); }
  int kv_pages_pending() const { return book.pool().pending_pages(); }
  int kv_admit_need(int s, const std::vector<int>& p, uint64_t scope, bool scratch = false) const { return book.kv_admit_need(s, p, scope, scratch); }
  int kv_step_need(int s, bool spec) const { return book.kv_step_need(s, spec); }
  int kv_lru_idle(const std::vector<bool>& busy) const { return book.kv_lru_idle(busy); }
  int kv_reclaimable(const std::vector<int>& s) const { return book.kv_reclaimable(s); }
  void kv_evict(int s) {
    if (book.evict(s)) ++kv_evictions_;
  }
  bool kv_retire(bool) {
    book.pool().retire();
    return book.pool().pending_pages() == 0;
  }
  bool can_batch(int s, const ling::SamplingParams& p) const {
    return p.temperature <= 0.f && book.at(s).pos + ling::kernels::kMaxStreamRows <= book.max_context();
  }
  int begin_prefill(int session, const std::vector<int>& prompt, uint64_t scope) {
    ling::Session& s = book.at(session);
    const int L = int(prompt.size()), reuse = book.resume_reuse(session, prompt, scope, false);
    const int target = std::min(L + 2 * 16, book.max_context());
    if (book.kv_admit_need(session, prompt, scope) > book.pool().free_pages()) book.pool().retire();
    if (book.kv_admit_need(session, prompt, scope) > book.pool().free_pages()) throw ling::KvPoolExhausted("prefill");
    book.pool().truncate(s.table, book.pool().pages_for(target) * 16);
    if (!book.pool().ensure(s.table, reuse, target, nullptr)) throw ling::KvPoolExhausted("prefill");
    s.history = prompt, s.prompt_len = s.turn_start = s.pos = L;
    return 7000 + L % 100;
  }
  void speculate_batch(std::span<SeqStep> seqs) {
    int need = 0;
    for (const SeqStep& q : seqs) need += book.kv_step_need(q.session, true);
    if (need > book.pool().free_pages()) book.pool().retire();
    if (need > book.pool().free_pages()) throw ling::KvPoolExhausted("step");
    passes.emplace_back();
    for (SeqStep& q : seqs) {
      ling::Session& s = book.at(q.session);
      passes.back().push_back(q.session);
      book.pool().ensure(s.table, s.pos, s.pos + book.kv_step_rows(s, true), nullptr);
      const int n = std::max(1, accept(q.session, s.pos));
      s.history.push_back(q.anchor);
      q.out.clear();
      for (int j = 0; j < n; ++j) q.out.push_back(100000 + q.session * 1000 + (s.pos + j) % 1000);
      for (int j = 0; j + 1 < n; ++j) s.history.push_back(q.out[size_t(j)]);
      s.pos += n;
    }
    book.pool().retire();
  }
};
using HostScheduler = ling::serve::SchedulerT<HostEngine>;

static Request request(int len, int first, int max_tokens, const std::string& key = "") {
  Request r;
  r.prompt.resize(size_t(len));
  std::iota(r.prompt.begin(), r.prompt.end(), first);
  r.max_tokens = max_tokens, r.session_key = key;
  r.sampling.temperature = 0.f;
  return r;
}
static std::map<long, Finished> by_id(std::vector<Finished> v) {
  std::map<long, Finished> m;
  for (Finished& f : v) m[f.id] = std::move(f);
  return m;
}

static void host_checks() {
  {  // two requests share every verify pass once both have prefilled; a third waits for a place in the batch
    HostEngine eng(4, 64, 2048, 4);
    HostScheduler sch(eng, 2);
    const long a = sch.submit(request(40, 1, 9)), b = sch.submit(request(70, 500, 6)), c = sch.submit(request(20, 900, 3));
    EXPECT(sch.turn() && sch.running() == 1 && sch.queued() == 2);  // a admitted, its prefill is the unit
    EXPECT(sch.turn() && sch.running() == 2);                       // b admitted; the turn is a's again or b's prefill
    sch.run_until_idle();
    auto done = by_id(sch.take_finished());
    EXPECT(done.size() == 3 && done[a].tokens.size() == 9 && done[b].tokens.size() == 6 && done[c].tokens.size() == 3);
    EXPECT(done[a].finish == "length" && done[a].tokens[0] == 7040 && done[b].tokens[0] == 7070);
    EXPECT(done[a].batched >= 1 && done[b].batched >= 1 && done[c].admitted == 3);
    bool together = false, c_early = false;
    for (const auto& p : eng.passes) {
      together = together || p.size() == 2;
      EXPECT(p.size() <= 2);
    }
    for (size_t i = 0; i + 1 < eng.passes.size() && i < 2; ++i)
      for (int s : eng.passes[i]) c_early = c_early || s == done[c].session;
    EXPECT(together && !c_early && sch.stats().batched_steps >= 1 && sch.queued() == 0 && sch.running() == 0);
  }
  {  // a follow-up that extends a finished conversation is bound to its resident session and reuses its pages
    HostEngine eng(3, 64, 2048, 4);
    HostScheduler sch(eng, 2);
    Request first = request(50, 1, 4, "conv");
    const long a = sch.submit(first);
    sch.run_until_idle();
    Finished fa = by_id(sch.take_finished())[a];
    Request next = first;
    next.prompt.insert(next.prompt.end(), fa.tokens.begin(), fa.tokens.end() - 1);  // what the session has processed
    for (int t = 0; t < 10; ++t) next.prompt.push_back(9000 + t);
    const int need_cold = eng.kv_admit_need(1, next.prompt, 0), need_warm = eng.kv_admit_need(fa.session, next.prompt, 0);
    EXPECT(eng.match_session(next.prompt, "conv", 0) == fa.session && need_warm < need_cold);
    const long b = sch.submit(next), c = sch.submit(request(30, 4000, 2, "other"));
    sch.run_until_idle();
    auto done = by_id(sch.take_finished());
    EXPECT(done[b].session == fa.session && done[c].session != fa.session && eng.evictions == 0 && eng.book.resident() == 2);
    // two jobs that continue the same session run one after the other
    Request again = next;
    again.prompt.push_back(1), again.max_tokens = 2;
    Request again2 = again;
    const long d = sch.submit(again), e = sch.submit(again2);
    EXPECT(sch.turn() && sch.running() == 1 && sch.queued() == 1);
    sch.run_until_idle();
    done = by_id(sch.take_finished());
    EXPECT(done.size() == 2 && done[d].session == done[e].session && done[d].admitted < done[e].admitted);
  }
  {  // a prompt as long as the context, or longer than the pool, is answered at once
    HostEngine eng(2, 8, 256, 2);
    HostScheduler sch(eng, 2);
    const long a = sch.submit(request(256, 1, 4)), b = sch.submit(request(200, 1, 4)), c = sch.submit(request(20, 1, 2));
    sch.run_until_idle();
    auto done = by_id(sch.take_finished());
    EXPECT(done[a].finish == "error" && done[a].code == "context_length_exceeded" &&
           done[a].error.rfind("This model's maximum context length is 256 tokens.", 0) == 0);
    EXPECT(done[b].finish == "error" && done[b].code == "context_length_exceeded");  // 13 + 2 pages > 8
    EXPECT(done[c].finish == "length" && done[c].tokens.size() == 2);
  }
  {  // the end-of-sequence token stops a request and is not counted
    HostEngine eng(2, 64, 2048, 2);
    HostScheduler sch(eng, 1);
    Request r = request(10, 1, 50);
    r.eos_token = 100000 + 0 * 1000 + 14;  // the fifth token the first session's steps produce (positions 10 .. 14)
    const long a = sch.submit(r);
    sch.run_until_idle();
    Finished f = by_id(sch.take_finished())[a];
    EXPECT(f.finish == "stop" && f.tokens.size() == 5 && f.tokens.back() == 100013);
  }
  {  // page pressure: idle sessions are evicted least recently used first to admit a prompt
    HostEngine eng(4, 24, 2048, 2);
    HostScheduler sch(eng, 1);
    for (int i = 0; i < 3; ++i) {
      eng.now = 10.0 * (i + 1);
      sch.submit(request(60, 1000 * (i + 1), 2, "k" + std::to_string(i)));  // 4 + 2 pages each, 6 or 7 held after the steps
      sch.run_until_idle();
    }
    EXPECT(sch.take_finished().size() == 3 && eng.book.resident() == 3 && eng.kv_pages_free() <= 6);
    eng.now = 50;
    const long d = sch.submit(request(250, 7000, 2, "big"));  // 16 + 2 pages: two idle sessions must go
    sch.run_until_idle();
    auto done = by_id(sch.take_finished());
    EXPECT(done[d].finish == "length" && sch.stats().kv_evictions == 2 && eng.kv_evictions_ == 2);
    EXPECT(!eng.book.at(0).owned && !eng.book.at(1).owned && eng.book.at(2).owned);  // the two least recently used went
  }
  {  // every running request waits for a page: the one admitted last ends at "length", the other goes on
    HostEngine eng(2, 10, 2048, 2);
    eng.accept = [](int, int) { return 8; };
    HostScheduler sch(eng, 2);
    const long a = sch.submit(request(30, 1, 400)), b = sch.submit(request(30, 500, 400));  // 2 + 2 pages each, 2 more a step
    sch.run_until_idle(2000);
    auto done = by_id(sch.take_finished());
    EXPECT(sch.stats().kv_pool_exhausted >= 1 && done.count(b) == 1 && done[b].finish == "length" && done[b].tokens.size() < 400);
    EXPECT(done.count(a) == 1 && done[a].tokens.size() > done[b].tokens.size());
  }
  {  // pairing: with room for two in a pass and three decoding, running order always takes the first partner;
     // fair pairing takes the one with the fewest recent passes, so everybody steps about as often
    for (int fair = 0; fair < 2; ++fair) {
      HostEngine eng(3, 96, 2048, 2);
      eng.accept = [](int, int) { return 1; };
      HostScheduler sch(eng, 3, 0, fair != 0);
      for (int i = 0; i < 3; ++i) sch.submit(request(20, 100 * i, 30));
      sch.run_until_idle();
      std::map<int, int> count;
      size_t last_full = 0;
      for (size_t i = 0; i < eng.passes.size(); ++i)
        if (eng.passes[i].size() == 2) last_full = i;
      for (size_t i = 0; i < 30 && i < last_full; ++i)
        for (int s : eng.passes[i]) ++count[s];
      const int lo = std::min({count[0], count[1], count[2]}), hi = std::max({count[0], count[1], count[2]});
      if (fair) EXPECT(hi - lo <= 2);
      else EXPECT(hi - lo >= 5);
      EXPECT(sch.take_finished().size() == 3);
    }
  }
  {  // keyed sessions are protected for a while: a new conversation waits, and is admitted once the protection has run out
    HostEngine eng(2, 64, 2048, 2);
    HostScheduler sch(eng, 2, 30.0);
    eng.now = 100;
    sch.submit(request(20, 1, 2, "a")), sch.submit(request(20, 300, 2, "b"));
    sch.run_until_idle();
    EXPECT(sch.take_finished().size() == 2);
    eng.now = 110;
    const long c = sch.submit(request(20, 600, 2, "c"));
    sch.run_until_idle();
    EXPECT(sch.queued() == 1 && sch.take_finished().empty());
    eng.now = 140;
    sch.poke();
    sch.run_until_idle();
    auto done = by_id(sch.take_finished());
    EXPECT(done.count(c) == 1 && done[c].finish == "length" && eng.evictions == 1);
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
  e.set_tree_source([](int, int anchor, const std::vector<int>& history) { return chain_tree(anchor, 12, anchor + int(history.size())); });
  e.set_prefill_fill([](ling_b200_ctx* ctx, int session, int, int to) {
    // stand-in for the prefill pass: the KV of [0, to) and the DeltaNet state written from host values that are a function of
    // the length alone (the library's synthetic fills are keyed by the slot), so that a request has the same context
    // whichever slot and company it runs in
    const ling::ModelConfig c = toy_config();
    std::mt19937 rng{unsigned(to) * 2654435761u + 17u};
    std::normal_distribution<float> nd(0.f, 1.f);
    std::vector<float> k(size_t(to) * c.kv_heads * c.head_dim), v(k.size());
    for (float& x : k) x = nd(rng);
    for (float& x : v) x = nd(rng);
    ling_b200_kv_write(ctx, session, 0, 0, to, k.data(), v.data());
    const int C = 2 * c.lin_k_heads * c.lin_k_dim + c.lin_v_heads * c.lin_v_dim;
    std::vector<float> st(size_t(c.lin_v_heads) * c.lin_k_dim * c.lin_v_dim), conv(size_t(C) * 3);
    for (int gl = 0; gl < 3; ++gl) {
      for (float& x : st) x = 0.1f * nd(rng);
      for (float& x : conv) x = nd(rng);
      ling_b200_state_write(ctx, session, gl, st.data(), conv.data());
    }
    return (to * 37) % 4096;
  });
}
static void gpu_checks() {
  ling::EngineOptions o;
  o.max_context = 1024, o.sessions = 4, o.max_seqs = 4, o.max_rows = 128, o.kv_pool_pages = 4 * 64;
  std::vector<Request> reqs;
  const int lens[6] = {37, 120, 64, 300, 90, 15};
  for (int i = 0; i < 6; ++i) reqs.push_back(request(lens[i], 10 * i, 10 + 3 * i));
  std::map<int, std::vector<int>> alone;  // by prompt length
  {
    ling::Engine eng(toy_config(), o);
    setup(eng);
    ling::serve::Scheduler sch(eng, 1);
    for (const Request& r : reqs) {
      sch.submit(r);
      sch.run_until_idle();
      std::vector<Finished> f = sch.take_finished();
      EXPECT(f.size() == 1 && f[0].finish == "length" && int(f[0].tokens.size()) == r.max_tokens && f[0].batched == 0);
      alone[int(r.prompt.size())] = f[0].tokens;
    }
  }
  ling::Engine eng(toy_config(), o);
  setup(eng);
  ling::serve::Scheduler sch(eng, 4);
  std::map<long, int> len_of;
  for (const Request& r : reqs) len_of[sch.submit(r)] = int(r.prompt.size());
  sch.run_until_idle();
  std::vector<Finished> done = sch.take_finished();
  EXPECT(done.size() == 6 && sch.stats().batched_steps > 0);
  int batched = 0;
  for (const Finished& f : done) {
    EXPECT(f.finish == "length" && f.tokens == alone[len_of[f.id]]);
    batched += f.batched;
  }
  EXPECT(batched > 0);
  std::printf("continuous batching: %ld decode passes, %ld of them shared, %.2f sequences a pass\n", sch.stats().decode_passes,
              sch.stats().batched_steps, double(sch.stats().rows) / double(sch.stats().decode_passes));
  // The same requests through a page pool that cannot keep every finished session resident: admission evicts idle sessions,
  // and what the running requests produce does not change.
  ling::EngineOptions tight = o;
  tight.kv_pool_pages = 44;
  ling::Engine eng2(toy_config(), tight);
  setup(eng2);
  ling::serve::Scheduler sch2(eng2, 2);
  std::map<long, int> len2;
  for (const Request& r : reqs) len2[sch2.submit(r)] = int(r.prompt.size());
  sch2.run_until_idle();
  std::vector<Finished> done2 = sch2.take_finished();
  EXPECT(done2.size() == 6 && sch2.stats().kv_evictions > 0);
  for (const Finished& f : done2) {
    EXPECT(f.finish == "length" && f.tokens == alone[len2[f.id]]);
    if (f.tokens != alone[len2[f.id]]) {
      std::printf("request %ld (prompt %d) in session %d: finish %s %s, %zu tokens, passes %d (%d shared):", f.id, len2[f.id], f.session,
                  f.finish.c_str(), f.error.c_str(), f.tokens.size(), f.passes, f.batched);
      for (size_t i = 0; i < f.tokens.size() && i < alone[len2[f.id]].size(); ++i)
        if (f.tokens[i] != alone[len2[f.id]][i]) {
          std::printf(" first difference at token %zu (%d vs %d)", i, f.tokens[i], alone[len2[f.id]][i]);
          break;
        }
      std::printf("\n");
    }
  }
  std::printf("tight pool (44 pages): %ld idle sessions evicted, %ld page waits, %ld ended by the last resort\n", sch2.stats().kv_evictions,
              sch2.stats().kv_waits, sch2.stats().kv_pool_exhausted);
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
