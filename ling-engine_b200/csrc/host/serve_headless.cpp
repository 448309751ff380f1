// serve_headless.cpp -- the serving loop without the server: the reference's ling-serve admits requests over HTTP and its
// Scheduler (src/serve/main.cpp:357-860) drives Engine::speculate_batch; this program feeds the same loop
// (ling_scheduler.hpp) from a seeded request generator instead and reports what the loop did and how fast the verify passes
// ran.  It is how the 64-sequence continuous-batching workload is produced by the scheduler's own policy rather than by a
// script: requests arrive in a queue, are admitted into session slots and the KV page pool, share verify passes, finish,
// and give their pages back to the ones behind them.
//
//   ling_serve_headless [--layers 64] [--requests 96] [--sessions 64] [--batch 64] [--max-context 131072] [--pool-pages 0]
//                       [--median 6000] [--max-tokens 32] [--seed 1] [--fair 0] [--toy]
//                       [--systems 0] [--system-tokens 3000] [--prefix-kv-mb 0]
// Prompts: lengths lognormal around --median (at most max-context - 64), token ids uniform.  With --systems K every prompt
// begins with one of K system messages of --system-tokens tokens (boundary token, message, boundary token), the way
// conversations of a few agents share their instructions; --prefix-kv-mb > 0 turns the engine's prefix KV store on, which
// then keeps each system message's pages and state once and lets later prompts resume behind it.  The prefill pass is outside this
// build: an admitted prompt's KV and DeltaNet state are filled synthetically on the device.  Draft trees: a chain plus a lookup
// branch off the anchor, 1-32 rows, random tokens (so a pass accepts what the random-weight model happens to agree with:
// nearly always the anchor alone).  One JSON line on stdout.
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>

#include "ling_scheduler.hpp"

namespace {

ling::ModelConfig model(bool toy, int layers) {
  ling::ModelConfig c{};
  if (toy) {
    c.hidden = 256, c.intermediate = 704, c.layers = 4, c.vocab = 4096;
    c.heads = 4, c.kv_heads = 1, c.head_dim = 64, c.rotary_dim = 16;
    c.lin_k_heads = 2, c.lin_v_heads = 4, c.lin_k_dim = 64, c.lin_v_dim = 64;
    c.full_attention[3] = 1;
  } else {
    c.hidden = 5120, c.intermediate = 17408, c.layers = layers, c.vocab = 248320;
    c.heads = 24, c.kv_heads = 4, c.head_dim = 256, c.rotary_dim = 64;
    c.lin_k_heads = 16, c.lin_v_heads = 48, c.lin_k_dim = 128, c.lin_v_dim = 128;
    for (int l = 0; l < layers; ++l) c.full_attention[l] = (l % 4) == 3;
  }
  c.rope_theta = 1e6f, c.eps = 1e-6f, c.conv_kernel = 4;
  return c;
}

ling::DraftTree chain_plus_branch(int anchor, int rows, std::mt19937& rng, int vocab) {
  const int chain_rows = std::max(1, (2 * rows + 2) / 3);
  ling::DraftTree t;
  t.E = chain_rows - 1;
  for (int r = 0; r < rows; ++r) {
    t.parent.push_back(r == 0 ? -1 : r < chain_rows ? r - 1 : r == chain_rows ? 0 : r - 1);
    t.depth.push_back(r == 0 ? 0 : t.depth[size_t(t.parent[size_t(r)])] + 1);
    t.token.push_back(r == 0 ? anchor : int(rng() % unsigned(vocab)));
    t.pick.push_back(0);
  }
  t.children.assign(t.parent.size(), {});
  for (int r = 1; r < rows; ++r) t.children[size_t(t.parent[size_t(r)])].push_back(r);
  return t;
}

int arg(int argc, char** argv, const char* name, int def) {
  for (int i = 1; i + 1 < argc; ++i)
    if (!std::strcmp(argv[i], name)) return std::atoi(argv[i + 1]);
  return def;
}
bool flag(int argc, char** argv, const char* name) {
  for (int i = 1; i < argc; ++i)
    if (!std::strcmp(argv[i], name)) return true;
  return false;
}

}  // namespace

int main(int argc, char** argv) {
  const bool toy = flag(argc, argv, "--toy");
  const int layers = arg(argc, argv, "--layers", 64), n_req = arg(argc, argv, "--requests", 96), sessions = arg(argc, argv, "--sessions", 64);
  const int batch = arg(argc, argv, "--batch", sessions), max_context = arg(argc, argv, "--max-context", toy ? 4096 : 131072);
  const int median = arg(argc, argv, "--median", toy ? 300 : 6000), max_tokens = arg(argc, argv, "--max-tokens", 32);
  const int seed = arg(argc, argv, "--seed", 1), device = arg(argc, argv, "--device", 0);
  int pool_pages = arg(argc, argv, "--pool-pages", 0);
  if (ling_b200_device_count() < 1) {
    std::fprintf(stderr, "ling_serve_headless: no CUDA device (there is no CPU path)\n");
    return 2;
  }
  std::mt19937 rng{unsigned(seed)};
  std::lognormal_distribution<double> len(std::log(double(median)), 1.0);
  std::vector<ling::serve::Request> reqs{};
  reqs.resize(size_t(n_req));
  const ling::ModelConfig cfg = model(toy, layers);
  long prompt_tokens = 0;
  constexpr int kBoundary = 1;
  const int n_sys = arg(argc, argv, "--systems", 0), sys_tokens = arg(argc, argv, "--system-tokens", toy ? 150 : 3000);
  const int prefix_kv_mb = arg(argc, argv, "--prefix-kv-mb", 0);
  std::vector<std::vector<int>> systems(size_t(std::max(n_sys, 0)));
  for (auto& m : systems) {
    m.push_back(kBoundary);
    for (int i = 0; i < sys_tokens; ++i) m.push_back(2 + int(rng() % unsigned(cfg.vocab - 2)));
    m.push_back(kBoundary);
  }
  for (auto& r : reqs) {
    const int L = std::clamp(int(len(rng)), 16, max_context - 64 - (n_sys > 0 ? sys_tokens + 2 : 0));
    if (n_sys > 0) r.prompt = systems[size_t(rng() % unsigned(n_sys))];
    const size_t head = r.prompt.size();
    r.prompt.resize(head + size_t(L));
    for (size_t i = head; i < r.prompt.size(); ++i) r.prompt[i] = 2 + int(rng() % unsigned(cfg.vocab - 2));
    // a later message of the conversation's own: its last message then starts past what it shares with the others, so it is
    // a conversation of its own to match_session and not the next turn of another one with the same system message
    if (n_sys > 0 && L >= 4) r.prompt[head + size_t(L) / 2] = kBoundary;
    r.max_tokens = 1 + int(rng() % unsigned(max_tokens));
    r.sampling.temperature = 0.f;
    prompt_tokens += long(r.prompt.size());
  }
  ling::EngineOptions o;
  o.max_context = max_context, o.sessions = sessions, o.max_seqs = std::min(batch, ling::kernels::kMaxSeqs), o.max_rows = 32 * o.max_seqs;
  o.page_tokens = 16, o.device = device, o.pdl = true;
  o.boundary_token = kBoundary, o.prefix_kv_mb = prefix_kv_mb;
  if (pool_pages <= 0) {  // room for the resident sessions at the workload's mean length, plus a quarter: long prompts force evictions
    pool_pages = int(double(prompt_tokens) / n_req / 16.0 * sessions * 1.25) + 8 * sessions;
    pool_pages = std::max(pool_pages, (max_context + 15) / 16 + 8);
  }
  o.kv_pool_pages = pool_pages;
  try {
    ling::Engine eng(cfg, o);
    if (ling_b200_synth_weights(eng.handle(), 0) != LING_B200_OK) throw std::runtime_error(ling_b200_last_error());
    long tree_rows = 0;
    eng.set_tree_source([&](int, int anchor, const std::vector<int>&) {
      const int rows = 1 + int(rng() % 32u);
      tree_rows += rows;
      return chain_plus_branch(anchor, rows, rng, cfg.vocab);
    });
    double fill_s = 0;
    long filled_tokens = 0;
    eng.set_prefill_fill([&](ling_b200_ctx* ctx, int session, int from, int to) {
      const auto t0 = std::chrono::steady_clock::now();
      filled_tokens += to - from;
      ling_b200_synth_kv_range(ctx, session, from, to - from, uint64_t(to));  // only what this prompt does not share
      ling_b200_synth_state(ctx, session, uint64_t(to));
      ling_b200_sync(ctx);
      fill_s += std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
      return to % cfg.vocab;
    });
    ling::serve::Scheduler sch(eng, batch, 0.0, flag(argc, argv, "--fair"));
    for (auto& r : reqs) sch.submit(r);
    const auto t0 = std::chrono::steady_clock::now();
    double pass_s = 0;
    long turns = 0, max_seqs_in_pass = 0;
    while (!(sch.queued() == 0 && sch.running() == 0) && turns < 10000000) {
      const auto a = std::chrono::steady_clock::now();
      const bool moved = sch.turn();
      ++turns;
      if (!sch.last_pass().empty()) {
        pass_s += std::chrono::duration<double>(std::chrono::steady_clock::now() - a).count();
        max_seqs_in_pass = std::max<long>(max_seqs_in_pass, long(sch.last_pass().size()));
      }
      if (!moved) {
        sch.poke();
        if (!sch.turn()) break;
      }
    }
    const double wall = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    std::vector<ling::serve::Finished> done = sch.take_finished();
    long produced = 0, errors = 0, at_length = 0;
    for (const auto& f : done) {
      produced += long(f.tokens.size());
      if (f.finish == "error" && errors < 3) std::fprintf(stderr, "ling_serve_headless: request %ld ended in error: %s\n", f.id, f.error.c_str());
      errors += f.finish == "error";
      at_length += f.finish == "length";
    }
    const ling::serve::SchedulerStats& st = sch.stats();
    std::printf(
        "{\"driver\": \"ling_serve_headless\", \"model\": \"%s\", \"requests\": %d, \"finished\": %zu, \"errors\": %ld, \"sessions\": %d, "
        "\"batch\": %d, \"pool_pages\": %d, \"prompt_tokens\": %ld, \"produced_tokens\": %ld, \"turns\": %ld, \"decode_passes\": %ld, "
        "\"shared_passes\": %ld, \"sequences_per_pass\": %.2f, \"max_sequences_in_pass\": %ld, \"rows_per_pass\": %.1f, "
        "\"kv_evictions\": %ld, \"kv_waits\": %ld, \"kv_pool_exhausted\": %ld, \"session_evictions\": %ld, \"pass_seconds\": %.4f, "
        "\"ms_per_pass\": %.3f, \"rows_per_s\": %.1f, \"tokens_per_s\": %.1f, \"prefill_fill_seconds\": %.3f, \"wall_seconds\": %.3f, "
        "\"not_finished\": %zu, \"launches_last_pass\": %d, \"systems\": %d, \"prefix_kv_mb\": %d, \"prefilled_tokens\": %ld, "
        "\"store_evictions\": %ld, \"store_nodes\": %d, \"store_states\": %d, \"store_pages_held\": %d}\n",
        toy ? "toy" : "27B-class", n_req, done.size(), errors, sessions, batch, pool_pages, prompt_tokens, produced, turns, st.decode_passes,
        st.batched_steps, st.decode_passes ? double(st.rows) / double(st.decode_passes) : 0.0, max_seqs_in_pass,
        st.decode_passes ? double(tree_rows) / double(st.decode_passes) : 0.0, st.kv_evictions, st.kv_waits, st.kv_pool_exhausted,
        eng.session_evictions(), pass_s, st.decode_passes ? pass_s / double(st.decode_passes) * 1e3 : 0.0,
        pass_s > 0 ? double(tree_rows) / pass_s : 0.0, pass_s > 0 ? double(produced) / pass_s : 0.0, fill_s, wall, sch.queued() + sch.running(), ling_b200_step_launch_count(eng.handle()),
        n_sys, prefix_kv_mb, filled_tokens, st.kv_store_evictions, eng.kv_store_on() ? eng.kv_store()->nodes() : 0,
        eng.kv_store_on() ? eng.kv_store()->states() : 0, eng.kv_store_on() ? eng.kv_store()->pages_held() : 0);
    return done.size() == size_t(n_req) ? 0 : 1;
  } catch (const std::exception& e) {
    std::fprintf(stderr, "ling_serve_headless: %s\n", e.what());
    return 1;
  }
}
