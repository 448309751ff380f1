// ling_scheduler.hpp -- the loop that calls the verify step: the reference server's Scheduler (src/serve/main.cpp:357-860 of
// dreamference/ling-engine) as a headless driver, without the HTTP server, the tokenizer, streaming text and metrics.
//
// What it keeps: jobs queue up; a job is admitted when a session slot can be bound (the resident session it continues, else
// a free or evictable one) and, with the KV page pool, when its prompt's pages and the growth reserve can be made free;
// the running requests take turns, one unit each -- the prompt's prefill, then decode steps; when the request whose turn
// it is can step speculatively and others can too, they take ONE verify pass together (Engine::speculate_batch) as far as
// the pass's capacity and the pool's free pages allow, partners chosen by serve::pair_order; a decode step whose pages are
// not there waits while others run, and when every request waits the last resort ends the one admitted last at "length".
// Policy decisions are the library's exported functions (select order, kv_reclaim, kv_last_resort), pinned to the
// reference's by golden vectors; this file is the control flow around them.
//
// What differs, by design of this build: a prompt's prefill is one unit (the prefill pass is outside this build: the
// engine's fill hook stands in for it), there is no side stream and no donor session (a prompt resumes from its own session
// or from the prefix KV store, whose least recently used entries are the first thing given up for pages), and a pass takes
// up to the engine's max_batch() sequences (the reference: kMaxStreamRows / draft_block = 2).  The loop is single-threaded
// and step-driven (turn() runs one admission attempt and one unit), so tests and the benchmark replay it deterministically.
#pragma once

#include <list>
#include <optional>
#include <utility>

#include "ling_engine.hpp"

namespace ling::serve {

// src/serve/api.cpp:116-124
inline bool exceeds_context(size_t prompt_tokens, int max_context) { return prompt_tokens >= size_t(std::max(max_context, 0)); }
inline std::string context_overflow_message(size_t prompt_tokens, int max_context) {
  return "This model's maximum context length is " + std::to_string(max_context) + " tokens. However, your request has " +
         std::to_string(prompt_tokens) + " input tokens. Please reduce the length of the messages.";
}
inline constexpr const char* kContextLengthExceeded = "context_length_exceeded";

struct Request {
  std::vector<int> prompt;
  std::string session_key;
  uint64_t share_scope = 0;
  int max_tokens = 16;
  int eos_token = -1;
  SamplingParams sampling;  // temperature 0: greedy, the only mode the verify path accepts
};
struct Finished {
  long id = 0;
  int session = -1;
  std::vector<int> tokens;       // produced tokens (the stop token excluded)
  std::string finish = "length"; // "length", "stop", or "error"
  std::string error, code;
  int passes = 0, batched = 0;   // decode passes taken, and how many of them with another request
  long admitted = 0;
};
struct SchedulerStats {
  long turns = 0, decode_passes = 0, batched_steps = 0, kv_evictions = 0, kv_pool_exhausted = 0, kv_waits = 0;
  long kv_store_evictions = 0;  // prefix KV store entries given up for pages
  long rows = 0;  // sequences summed over the decode passes
};

template <class E>
class SchedulerT {
 public:
  SchedulerT(E& engine, int batch, double protect_seconds = 0, bool fair_pairing = false)
      : eng_(engine), batch_(batch), protect_seconds_(protect_seconds), fair_pairing_(fair_pairing) {}

  long submit(Request req) {
    queue_.push_back(Job{++ids_, std::move(req), -1, false});
    dirty_ = true;
    return ids_;
  }
  size_t queued() const { return queue_.size(); }
  size_t running() const { return running_.size(); }
  const SchedulerStats& stats() const { return stats_; }
  std::vector<Finished> take_finished() { return std::exchange(finished_, {}); }
  // Sessions of the requests that took the last decode pass (empty: the last unit was not a decode pass).
  const std::vector<int>& last_pass() const { return last_pass_; }

  // One iteration of the reference's run(): at most one admission, then one unit of the request whose turn it is.
  // False when nothing runs and nothing queued can be admitted now.
  bool turn() {
    ++stats_.turns;
    last_pass_.clear();
    const bool admitted = admit();
    if (running_.empty()) return admitted;  // a job answered at once (its prompt cannot run) still was a turn
    const size_t k = turn_++ % running_.size();
    Running& r = *at(k);
    std::vector<Running*> ended;
    const bool kv_blocked = !r.prefilling && !kv_room(r);  // main.cpp:577-579
    r.kv_wait = kv_blocked;
    if (kv_blocked) {
      ++stats_.kv_waits;
      kv_stalled(ended);
    } else {
      const std::vector<Running*> batch = batch_with(r);
      if (batch.size() >= 2) {
        batch_step(batch, ended);
      } else {
        bool done = false;
        try {
          done = unit(r);
        } catch (const std::exception& e) {
          fail(r, e.what(), "server_error");
          done = true;
        }
        if (done) ended.push_back(&r);
      }
    }
    for (Running* e : ended) {
      eng_.touch_session(e->out.session);  // the session's clock restarts however the request ended
      if (!e->requeued) finished_.push_back(std::move(e->out));
      running_.remove_if([&](const Running& x) { return &x == e; });
      dirty_ = true;  // its session may be what a queued job waits for
    }
    return true;
  }
  // A queued job that could not be placed is looked at again when something changed; the reference also looks once a
  // second (a protection expires).  A caller whose clock moved says so here.
  void poke() { dirty_ = true; }
  // Turns until everything submitted has finished or nothing can move (a second look after an idle turn finds nothing);
  // returns the turns taken.
  long run_until_idle(long max_turns = 1000000) {
    long n = 0;
    for (int idle = 0; n < max_turns && !(queue_.empty() && running_.empty()); ++n) {
      if (turn()) {
        idle = 0;
      } else {
        poke();
        if (++idle > 1) break;
      }
    }
    return n;
  }

 private:
  struct Job {
    long id;
    Request req;
    int session;
    bool fresh;
  };
  struct Running {
    Job job;
    bool prefilling = true, kv_wait = false, requeued = false;
    std::vector<int> pending;  // chosen tokens not yet emitted
    int produced = 0;
    long admitted = 0;
    PassWindow window;
    Finished out;
  };
  using Iter = typename std::list<Running>::iterator;
  Iter at(size_t k) {
    Iter it = running_.begin();
    std::advance(it, k);
    return it;
  }

  // ---- admission (main.cpp:386-445 pick, 447-478 admit, 481-527 start)
  bool admit() {
    if (static_cast<int>(running_.size()) >= batch_ || queue_.empty() || !(dirty_ || kv_wait_)) return false;
    dirty_ = false;
    std::optional<Job> job = pick();
    if (!job) return false;
    start(std::move(*job));
    // the reference looks at the rest of the queue again when something changes or a second has passed; without a clock
    // of its own this loop looks again at its next turn
    dirty_ = !queue_.empty();
    return true;
  }
  std::optional<Job> pick() {
    kv_wait_ = false;
    std::vector<bool> busy(size_t(eng_.sessions()), false);
    for (const Running& r : running_) busy[size_t(r.job.session)] = true;
    std::vector<bool> pinned = busy;
    std::vector<int> match(queue_.size());
    for (size_t j = 0; j < queue_.size(); ++j) {
      match[j] = eng_.match_session(queue_[j].req.prompt, queue_[j].req.session_key, queue_[j].req.share_scope);
      if (match[j] >= 0) pinned[size_t(match[j])] = true;
    }
    for (size_t j = 0; j < queue_.size(); ++j) {
      int s = match[j];
      if (s >= 0 && busy[size_t(s)]) continue;  // one request per session at a time
      const bool fresh = s < 0;
      if (fresh) s = eng_.free_session(protect_seconds_, pinned);
      if (s < 0) continue;
      const Request& q = queue_[j].req;
      // a prompt the whole pool could never hold is admitted to be answered at once (start)
      if (eng_.kv_admit_pages(q.prompt.size()) <= eng_.kv_pages_total()) {
        bool evicted = false;
        if (!kv_admit_room(s, q, &evicted)) {
          kv_wait_ = true;
          if (evicted) return std::nullopt;  // the matches above may name emptied sessions: look again from the start
          continue;
        }
      }
      Job out = std::move(queue_[j]);
      out.session = s, out.fresh = fresh;
      queue_.erase(queue_.begin() + long(j));
      return out;
    }
    return std::nullopt;
  }
  void start(Job job) {
    Running r;
    r.job = std::move(job);
    r.admitted = ++admitted_;
    r.out.id = r.job.id, r.out.session = r.job.session, r.out.admitted = r.admitted;
    const Request& q = r.job.req;
    const int session = r.job.session;
    if (exceeds_context(q.prompt.size(), eng_.max_context())) {
      fail(r, context_overflow_message(q.prompt.size(), eng_.max_context()), kContextLengthExceeded);
    } else if (eng_.kv_admit_pages(q.prompt.size()) > eng_.kv_pages_total()) {
      fail(r, "the KV page pool (" + std::to_string(eng_.kv_pages_total()) + " pages) cannot hold a prompt of " +
                  std::to_string(q.prompt.size()) + " tokens", kContextLengthExceeded);
    } else {
      eng_.activate_session(session, q.session_key, r.job.fresh, q.share_scope);
      running_.push_back(std::move(r));
      return;
    }
    eng_.touch_session(session);
    finished_.push_back(std::move(r.out));
  }
  void fail(Running& r, const std::string& what, const char* code) {
    r.out.finish = "error", r.out.error = what, r.out.code = code;
  }

  // ---- one unit of one request (main.cpp:913-988): the prompt's prefill, then one decode step alone
  bool unit(Running& r) {
    if (r.prefilling) {
      int first;
      try {
        first = eng_.begin_prefill(r.job.session, r.job.req.prompt, r.job.req.share_scope);
      } catch (const KvPoolExhausted& e) {
        // admission's count was short after all (nothing changed): while others run the job goes back to the front of the
        // queue and is admitted again once one ends; alone, room is made once more and the prefill tried again
        if (running_.size() > 1) {
          queue_.push_front(std::move(r.job));
          r.requeued = true;
          return true;
        }
        kv_admit_room(r.job.session, r.job.req, nullptr);
        first = eng_.begin_prefill(r.job.session, r.job.req.prompt, r.job.req.share_scope);
      }
      r.prefilling = false;
      r.pending = {first};
      return emit(r);
    }
    ++r.out.passes;
    ++stats_.decode_passes, ++stats_.rows;
    r.window.record(stats_.decode_passes);
    std::vector<typename E::SeqStep> q(1);
    q[0].session = r.job.session, q[0].anchor = r.pending.back(), q[0].params = &r.job.req.sampling;
    eng_.speculate_batch(std::span<typename E::SeqStep>(q));
    last_pass_ = {r.job.session};
    if (q[0].error) std::rethrow_exception(q[0].error);
    r.pending = std::move(q[0].out);
    return emit(r);
  }
  // main.cpp:1020-1078 without text, stop strings and logprobs: tokens one by one; the end-of-sequence token stops the
  // request and is not counted; the limit ends it at "length".
  bool emit(Running& r) {
    for (int t : r.pending) {
      if (t == r.job.req.eos_token) {
        r.out.finish = "stop";
        return true;
      }
      ++r.produced;
      r.out.tokens.push_back(t);
      if (r.produced >= r.job.req.max_tokens) return true;
    }
    return false;
  }

  // ---- batching (main.cpp:619-668)
  bool batchable(const Running& r) const { return !r.prefilling && eng_.can_batch(r.job.session, r.job.req.sampling); }
  std::vector<Running*> batch_with(Running& r) {
    std::vector<Running*> b;
    if (!batchable(r)) return b;
    b.push_back(&r);
    int kv_need = eng_.kv_step_need(r.job.session, true);
    const int kv_free = eng_.kv_pages_free(), fit = eng_.max_batch();
    constexpr bool kSlots = requires(E& e) { e.attn_slot_need(0); e.attn_slot_capacity(); };  // a pass's attention partial slots
    long slots = 0, slot_cap = 0;
    if constexpr (kSlots) slots = eng_.attn_slot_need(r.job.session), slot_cap = eng_.attn_slot_capacity();
    std::vector<PairCandidate> c;
    std::vector<Running*> by_index;
    for (Running& o : running_) {
      c.push_back(fair_pairing_ ? PairCandidate{false, o.window.count(stats_.decode_passes), o.window.last()} : PairCandidate{});
      by_index.push_back(&o);
    }
    for (size_t i : pair_order(c, fair_pairing_)) {
      Running* o = by_index[i];
      if (o == &r || static_cast<int>(b.size()) >= fit || !batchable(*o)) continue;
      const int n = eng_.kv_step_need(o->job.session, true);
      if (kv_need + n > kv_free) continue;  // only requests whose step's pages are free join
      if constexpr (kSlots) {
        const long need = eng_.attn_slot_need(o->job.session);
        if (slots + need > slot_cap) continue;  // the pass's contexts would not fit the attention's partial buffers
        slots += need;
      }
      kv_need += n;
      b.push_back(o);
    }
    return b;
  }
  // main.cpp:845-900: one verify pass over the batch; a non-finite row fails only its own request.
  void batch_step(const std::vector<Running*>& batch, std::vector<Running*>& ended) {
    std::vector<typename E::SeqStep> steps(batch.size());
    ++stats_.decode_passes, ++stats_.batched_steps;
    stats_.rows += long(batch.size());
    for (size_t i = 0; i < batch.size(); ++i) {
      Running& r = *batch[i];
      ++r.out.passes, ++r.out.batched;
      r.kv_wait = false;
      r.window.record(stats_.decode_passes);
      steps[i].session = r.job.session, steps[i].anchor = r.pending.back(), steps[i].params = &r.job.req.sampling;
      last_pass_.push_back(r.job.session);
    }
    try {
      eng_.speculate_batch(std::span<typename E::SeqStep>(steps));
    } catch (const std::exception& e) {  // not one sequence's rows: the step itself failed
      for (Running* r : batch) fail(*r, e.what(), "server_error"), ended.push_back(r);
      return;
    }
    for (size_t i = 0; i < batch.size(); ++i) {
      Running& r = *batch[i];
      bool done = false;
      try {
        if (steps[i].error) std::rethrow_exception(steps[i].error);
        r.pending = std::move(steps[i].out);
        done = emit(r);
      } catch (const std::exception& e) {
        fail(r, e.what(), "server_error");
        done = true;
      }
      if (done) ended.push_back(&r);
    }
  }

  // ---- the KV page pool (main.cpp:676-843)
  // Whether the engine has a prefix KV store (the real Engine; a host-only test engine need not).
  static constexpr bool kStore = requires(E& e, const std::vector<int>& v) {
    e.kv_store_evict(v);
    e.kv_reclaimable(v, true, v);
    e.kv_store_path(0, v, uint64_t(0));
  };
  // The pool as a unit of session `keep` sees it: free, pending, and what the idle sessions and the store's nodes outside
  // `store_keep` would free together.
  KvPoolView kv_view(int keep, std::vector<int>* idle = nullptr, const std::vector<int>& store_keep = {}) {
    std::vector<bool> excl = running_sessions(keep);
    KvPoolView v;
    v.free = eng_.kv_pages_free(), v.pending = eng_.kv_pages_pending();
    std::vector<int> lru;
    for (int s; (s = eng_.kv_lru_idle(excl)) >= 0;) lru.push_back(s), excl[size_t(s)] = true;
    if constexpr (kStore) v.idle = eng_.kv_reclaimable(lru, true, store_keep);
    else v.idle = eng_.kv_reclaimable(lru);
    if (idle) *idle = std::move(lru);
    return v;
  }
  std::vector<bool> running_sessions(int keep) const {
    std::vector<bool> excl(size_t(eng_.sessions()), false);
    for (const Running& r : running_) excl[size_t(r.job.session)] = true;
    if (keep >= 0) excl[size_t(keep)] = true;
    return excl;
  }
  // Whether the pages of a unit of session `keep` are free now, making room as kv_reclaim says (main.cpp:709-756): first the
  // holders that may go without moving the unit's resume point -- the store's least recently used leaves outside the path
  // the unit resumes from (`source`), then idle sessions least recently used first (protection does not hold against the
  // pool's need) -- and, only when those cannot be enough but everything can (or nothing else will ever free a page), the
  // unit's own source too, after which it needs `need_cold` pages.  Sessions are never a unit's source in this build.
  bool kv_make_room(const std::function<int()>& need, int keep, int need_cold, bool* evicted, const std::vector<int>& source = {}) {
    if (need() > eng_.kv_pages_free() + eng_.kv_pages_pending()) {
      const KvPoolView kept = kv_view(keep, nullptr, source), all = kv_view(keep);
      const std::vector<bool> excl = running_sessions(keep);
      const KvEvictNext session = [&] {
        const int s = eng_.kv_lru_idle(excl);
        if (s < 0) return false;
        if (evicted) *evicted = true;
        eng_.kv_evict(s);
        ++stats_.kv_evictions;
        return true;
      };
      std::vector<KvEvictNext> kept_order, source_order;
      if constexpr (kStore) {
        const auto store = [&](const std::vector<int>& keep_nodes) {
          return [this, evicted, &keep_nodes] {
            if (!eng_.kv_store_evict(keep_nodes)) return false;
            if (evicted) *evicted = true;
            ++stats_.kv_store_evictions;
            return true;
          };
        };
        static const std::vector<int> no_nodes;
        kept_order.push_back(store(source));
        source_order.push_back(store(no_nodes));
      }
      kept_order.push_back(session);
      source_order.push_back(session);
      kv_reclaim(need, [&] { return eng_.kv_pages_free() + eng_.kv_pages_pending(); }, kept_order, need(),
                 kept.free + kept.pending + kept.idle, source_order, std::max(need_cold, need()), all.free + all.pending + all.idle,
                 running_.empty() && need_cold > 0);
    }
    if (running_.empty()) eng_.kv_retire(true);
    return need() <= eng_.kv_pages_free();
  }
  bool kv_admit_room(int s, const Request& q, bool* evicted) {
    const int cold = eng_.kv_admit_need(s, q.prompt, q.share_scope, true);
    std::vector<int> source;
    if constexpr (kStore) source = eng_.kv_store_path(s, q.prompt, q.share_scope);
    return kv_make_room([&] { return eng_.kv_admit_need(s, q.prompt, q.share_scope); }, s, cold, evicted, source);
  }
  bool kv_room(Running& r) {
    return kv_make_room([&] { return eng_.kv_step_need(r.job.session, true); }, r.job.session, 0, nullptr);
  }
  // main.cpp:791-822: a decode turn waited for pages.  While someone still makes progress, or released pages are on their
  // way, nothing; else the last resort ends the request admitted last as if it had reached the context limit.
  void kv_stalled(std::vector<Running*>& ended) {
    std::vector<KvRunner> rs;
    std::vector<Running*> by_index;
    for (Running& o : running_) {
      if (o.prefilling || !o.kv_wait) return;
      rs.push_back({o.admitted, true, eng_.kv_step_need(o.job.session, true)});
      by_index.push_back(&o);
    }
    const KvPoolView v = kv_view(-1);
    if (v.pending > 0) {
      eng_.kv_retire(true);
      return;
    }
    const int i = kv_last_resort(rs, v);
    if (i < 0) return;
    Running& victim = *by_index[size_t(i)];
    victim.out.finish = "length";
    eng_.kv_evict(victim.job.session);
    ++stats_.kv_pool_exhausted;
    ended.push_back(&victim);
  }

  E& eng_;
  int batch_;
  double protect_seconds_;
  bool fair_pairing_;
  std::deque<Job> queue_;
  std::list<Running> running_;
  std::vector<Finished> finished_;
  std::vector<int> last_pass_;
  SchedulerStats stats_;
  size_t turn_ = 0;
  long ids_ = 0, admitted_ = 0;
  bool dirty_ = false, kv_wait_ = false;
};

using Scheduler = SchedulerT<Engine>;

}  // namespace ling::serve
