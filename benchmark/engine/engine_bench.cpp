// Engine benchmark: scenarios over the continuous-batching engine, driven through the C API / C++ owners only (no Python on the
// host side), with the acceptance gates of the reference's engine benchmark (benchmark/engine/docs/benchmark-requirements.md:
// cancellation latency p95 <= 500 ms; decode inter-token latency p95 during another request's prefill <= 1.5 x the steady
// baseline; every admitted request completes).  Scenarios: decode_baseline, mixed (decodes + one long prefill), cancellation,
// continuation.  Prints one JSON object; exit code 1 when a gate fails.
//
//   engine_bench --model DIR --vocab N --scenario mixed --concurrency 8 --prompt_len 512 --long_prompt_len 32768 --new_tokens 128
#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <random>
#include <string>
#include <vector>

#include "ogb_genai.hpp"

using Clock = std::chrono::steady_clock;
static double Ms(Clock::time_point a, Clock::time_point b) { return std::chrono::duration<double, std::milli>(b - a).count(); }

struct Args {
  std::string model, scenario = "decode_baseline";
  int vocab = 0, concurrency = 4, prompt_len = 512, long_prompt_len = 8192, new_tokens = 64, trials = 8, turns = 3, seed = 1;
  double cancel_gate_ms = 500.0, itl_gate_ratio = 1.5;
};

static double Percentile(std::vector<double> v, double p) {
  if (v.empty()) return 0.0;
  std::sort(v.begin(), v.end());
  size_t i = static_cast<size_t>(p * (v.size() - 1) + 0.5);
  return v[std::min(i, v.size() - 1)];
}

struct Tracked {
  std::unique_ptr<ogb::Request> req;
  Clock::time_point added, last;
  bool first_seen = false;
  double ttft_ms = 0;
  std::vector<double> itl_ms;
  std::vector<Clock::time_point> stamps;
  size_t tokens = 0;
};

struct Bench {
  const Args& a;
  ogb::Model model;
  ogb::Engine engine;
  std::mt19937 rng;
  std::vector<std::unique_ptr<Tracked>> all;
  std::map<void*, Tracked*> by_tag;

  explicit Bench(const Args& args) : a(args), model(args.model), engine(model), rng(args.seed) {}

  std::vector<int32_t> Prompt(int n) {
    std::uniform_int_distribution<int> d(3, std::max(4, a.vocab - 1));
    std::vector<int32_t> t(n);
    for (auto& x : t) x = d(rng);
    return t;
  }

  Tracked* Add(int prompt_len, int new_tokens) {
    ogb::GeneratorParams params(model);
    params.SetSearchOption("max_length", prompt_len + new_tokens);
    params.SetSearchOptionBool("do_sample", false);
    auto t = std::make_unique<Tracked>();
    t->req = std::make_unique<ogb::Request>(params);
    t->req->AddTokens(Prompt(prompt_len));
    t->req->SetOpaqueData(t.get());
    t->added = t->last = Clock::now();
    engine.Add(*t->req);
    Tracked* raw = t.get();
    by_tag[raw] = raw;
    all.push_back(std::move(t));
    return raw;
  }

  void Drain(Tracked* t) {
    while (t->req->HasUnseenTokens()) {
      t->req->GetUnseenToken();
      auto now = Clock::now();
      if (!t->first_seen) {
        t->first_seen = true;
        t->ttft_ms = Ms(t->added, now);
      } else {
        t->itl_ms.push_back(Ms(t->last, now));
      }
      t->stamps.push_back(now);
      t->last = now;
      ++t->tokens;
    }
  }

  // One engine step; every tracked request's new tokens are time-stamped.
  void Step() {
    ogb::Request ready = engine.Step();
    for (auto& t : all)
      if (t->req) Drain(t.get());
  }

  void Remove(Tracked* t) {
    engine.Remove(*t->req);
    t->req.reset();
  }
};

static void Json(const char* key, const std::vector<double>& v, bool last = false) {
  printf("  \"%s_p50\": %.3f, \"%s_p95\": %.3f, \"%s_n\": %zu%s\n", key, Percentile(v, 0.5), key, Percentile(v, 0.95), key, v.size(), last ? "" : ",");
}

static int DecodeBaseline(const Args& a) {
  Bench b(a);
  std::vector<Tracked*> rs;
  auto t0 = Clock::now();
  for (int i = 0; i < a.concurrency; ++i) rs.push_back(b.Add(a.prompt_len, a.new_tokens));
  int guard = 0;
  while (b.engine.HasPendingRequests() && guard++ < 1000000) b.Step();
  auto t1 = Clock::now();
  std::vector<double> itl, ttft;
  size_t tokens = 0;
  bool complete = true;
  for (auto* r : rs) {
    itl.insert(itl.end(), r->itl_ms.begin(), r->itl_ms.end());
    ttft.push_back(r->ttft_ms);
    tokens += r->tokens;
    complete = complete && r->req->IsTurnComplete();
    b.Remove(r);
  }
  printf("{\n  \"scenario\": \"decode_baseline\", \"concurrency\": %d, \"prompt_len\": %d, \"new_tokens\": %d,\n", a.concurrency, a.prompt_len, a.new_tokens);
  Json("itl_ms", itl);
  Json("ttft_ms", ttft);
  printf("  \"tokens\": %zu, \"tokens_per_s\": %.1f, \"all_complete\": %s, \"gates_passed\": %s\n}\n", tokens, tokens / (Ms(t0, t1) / 1e3),
         complete ? "true" : "false", complete ? "true" : "false");
  return complete ? 0 : 1;
}

static int Mixed(const Args& a) {
  Bench b(a);
  std::vector<Tracked*> rs;
  const int long_new = 4;
  // decodes that outlive the long request's whole prefill
  for (int i = 0; i < a.concurrency; ++i) rs.push_back(b.Add(a.prompt_len, a.new_tokens + a.long_prompt_len / 8 + 64));
  int guard = 0;
  auto warm = [&] { for (auto* r : rs) if (r->tokens < size_t(a.new_tokens)) return false; return true; };
  while (!warm() && guard++ < 1000000) b.Step();
  std::vector<double> base;
  for (auto* r : rs) base.insert(base.end(), r->itl_ms.begin() + std::min<size_t>(2, r->itl_ms.size()), r->itl_ms.end());
  std::vector<size_t> mark;
  for (auto* r : rs) mark.push_back(r->itl_ms.size());
  Tracked* big = b.Add(a.long_prompt_len, long_new);
  double max_gap = 0;
  while (!big->first_seen && guard++ < 1000000) b.Step();
  std::vector<double> during;
  for (size_t i = 0; i < rs.size(); ++i) {
    during.insert(during.end(), rs[i]->itl_ms.begin() + mark[i], rs[i]->itl_ms.end());
    for (size_t k = mark[i]; k < rs[i]->itl_ms.size(); ++k) max_gap = std::max(max_gap, rs[i]->itl_ms[k]);
  }
  const double ratio = Percentile(base, 0.95) > 0 ? Percentile(during, 0.95) / Percentile(base, 0.95) : 0.0;
  bool starved = false;
  for (size_t i = 0; i < rs.size(); ++i) starved = starved || rs[i]->itl_ms.size() == mark[i];   // a decode that never ran during the prefill
  b.Remove(big);
  for (auto* r : rs) b.Remove(r);
  const bool ok = ratio <= a.itl_gate_ratio && !starved;
  printf("{\n  \"scenario\": \"mixed\", \"concurrency\": %d, \"prompt_len\": %d, \"long_prompt_len\": %d,\n", a.concurrency, a.prompt_len, a.long_prompt_len);
  Json("baseline_itl_ms", base);
  Json("itl_during_prefill_ms", during);
  printf("  \"long_request_ttft_ms\": %.3f, \"max_scheduling_delay_ms\": %.3f, \"itl_p95_ratio\": %.3f, \"itl_gate_ratio\": %.2f, \"starved\": %s, \"gates_passed\": %s\n}\n",
         big->ttft_ms, max_gap, ratio, a.itl_gate_ratio, starved ? "true" : "false", ok ? "true" : "false");
  return ok ? 0 : 1;
}

static int Cancellation(const Args& a) {
  Bench b(a);
  std::vector<Tracked*> rs;
  for (int i = 0; i < a.concurrency; ++i) rs.push_back(b.Add(a.prompt_len, a.trials * 40 + a.new_tokens));
  for (int i = 0; i < 4; ++i) b.Step();
  std::vector<double> lat;
  for (int k = 0; k < a.trials; ++k) {
    Tracked* big = b.Add(a.long_prompt_len, 4);
    b.Step();
    b.Step();       // the long prompt is in the middle of its chunked prefill
    auto t0 = Clock::now();
    b.Remove(big);
    b.Step();       // the next step runs without it: the cancellation is in effect
    lat.push_back(Ms(t0, Clock::now()));
  }
  bool alive = true;
  for (auto* r : rs) {
    alive = alive && r->tokens > 0;
    b.Remove(r);
  }
  const double p95 = Percentile(lat, 0.95);
  const bool ok = p95 <= a.cancel_gate_ms && alive;
  printf("{\n  \"scenario\": \"cancellation\", \"concurrency\": %d, \"long_prompt_len\": %d, \"trials\": %d,\n", a.concurrency, a.long_prompt_len, a.trials);
  Json("cancel_latency_ms", lat);
  printf("  \"gate_ms\": %.1f, \"other_requests_progressed\": %s, \"gates_passed\": %s\n}\n", a.cancel_gate_ms, alive ? "true" : "false", ok ? "true" : "false");
  return ok ? 0 : 1;
}

static int Continuation(const Args& a) {
  Bench b(a);
  std::vector<Tracked*> rs;
  // every turn ends at the request's max_length and the next one is continued with a larger limit
  const int appended = 16;
  for (int i = 0; i < a.concurrency; ++i) {
    ogb::GeneratorParams params(b.model);
    params.SetSearchOption("max_length", a.prompt_len + a.new_tokens);
    params.SetSearchOptionBool("do_sample", false);
    auto t = std::make_unique<Tracked>();
    t->req = std::make_unique<ogb::Request>(params);
    t->req->AddTokens(b.Prompt(a.prompt_len));
    t->added = t->last = Clock::now();
    b.engine.Add(*t->req);
    rs.push_back(t.get());
    b.all.push_back(std::move(t));
  }
  std::vector<std::vector<double>> ttft(a.turns);
  bool ok = true;
  for (int turn = 0; turn < a.turns; ++turn) {
    std::vector<size_t> start;
    for (auto* r : rs) start.push_back(r->tokens);
    int guard = 0;
    auto done = [&] { for (size_t i = 0; i < rs.size(); ++i) if (rs[i]->tokens < start[i] + size_t(a.new_tokens)) return false; return true; };
    while (!done() && guard++ < 1000000) b.Step();
    ok = ok && done();
    for (size_t i = 0; i < rs.size(); ++i) ttft[turn].push_back(Ms(rs[i]->added, rs[i]->stamps[start[i]]));
    if (turn + 1 < a.turns) {
      for (auto* r : rs) {
        // the turn ends when the caller says so: cut it by continuing with new input (valid once the turn is complete)
        int spin = 0;
        while (!r->req->IsTurnComplete() && spin++ < 100000) b.Step();
        r->added = Clock::now();
        r->req->Continue(b.Prompt(appended), size_t(a.prompt_len + (turn + 2) * a.new_tokens + (turn + 1) * appended));
      }
    }
  }
  for (auto* r : rs) b.Remove(r);
  printf("{\n  \"scenario\": \"continuation\", \"concurrency\": %d, \"prompt_len\": %d, \"turns\": %d,\n", a.concurrency, a.prompt_len, a.turns);
  for (int t = 0; t < a.turns; ++t) {
    char key[64];
    snprintf(key, sizeof key, "turn%d_ttft_ms", t);
    Json(key, ttft[t]);
  }
  printf("  \"gates_passed\": %s\n}\n", ok ? "true" : "false");
  return ok ? 0 : 1;
}

int main(int argc, char** argv) {
  Args a;
  for (int i = 1; i + 1 < argc; i += 2) {
    std::string k = argv[i];
    const char* v = argv[i + 1];
    if (k == "--model") a.model = v;
    else if (k == "--scenario") a.scenario = v;
    else if (k == "--vocab") a.vocab = atoi(v);
    else if (k == "--concurrency") a.concurrency = atoi(v);
    else if (k == "--prompt_len") a.prompt_len = atoi(v);
    else if (k == "--long_prompt_len") a.long_prompt_len = atoi(v);
    else if (k == "--new_tokens") a.new_tokens = atoi(v);
    else if (k == "--trials") a.trials = atoi(v);
    else if (k == "--turns") a.turns = atoi(v);
    else if (k == "--seed") a.seed = atoi(v);
    else if (k == "--cancel_gate_ms") a.cancel_gate_ms = atof(v);
    else if (k == "--itl_gate_ratio") a.itl_gate_ratio = atof(v);
    else { fprintf(stderr, "unknown option %s\n", k.c_str()); return 2; }
  }
  if (a.model.empty() || a.vocab <= 0) { fprintf(stderr, "usage: engine_bench --model DIR --vocab N --scenario decode_baseline|mixed|cancellation|continuation ...\n"); return 2; }
  ogb::ShutdownGuard guard;
  try {
    if (a.scenario == "decode_baseline") return DecodeBaseline(a);
    if (a.scenario == "mixed") return Mixed(a);
    if (a.scenario == "cancellation") return Cancellation(a);
    if (a.scenario == "continuation") return Continuation(a);
    fprintf(stderr, "unknown scenario %s\n", a.scenario.c_str());
    return 2;
  } catch (const std::exception& e) {
    fprintf(stderr, "engine_bench: %s\n", e.what());
    return 3;
  }
}
