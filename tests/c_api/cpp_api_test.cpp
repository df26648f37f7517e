// The C++ owners over the C API: exceptions for errors, moves, a generation loop and an engine loop.
#include <cstdio>
#include <map>

#include "ogb_genai.hpp"

static void Print(const char* key, const std::vector<int32_t>& t) {
  printf("%s:", key);
  for (int32_t v : t) printf(" %d", v);
  printf("\n");
}

int main(int argc, char** argv) {
  if (argc < 2) return 2;
  ogb::ShutdownGuard guard;
  try {
    ogb::Model("/nonexistent/model/dir");
    printf("bad_model_error: no\n");
  } catch (const std::exception&) {
    printf("bad_model_error: yes\n");
  }
  ogb::Model model(argv[1]);
  ogb::Tokenizer tok(model);
  ogb::GeneratorParams params(model);
  params.SetSearchOption("max_length", 24);
  params.SetSearchOptionBool("do_sample", false);
  auto prompt = tok.Encode("hello world");
  {
    ogb::Generator gen(model, params);
    gen.AppendTokens(prompt);
    while (!gen.IsDone()) gen.GenerateNextToken();
    ogb::Generator moved = std::move(gen);
    Print("greedy", moved.GetSequence(0));
    auto logits = moved.GetLogits();
    printf("logits_rank: %zu\n", logits.Shape().size());
  }
  ogb::Engine engine(model);
  std::vector<ogb::Request> reqs;
  std::map<void*, std::vector<int32_t>> out;
  for (int i = 0; i < 3; ++i) {
    reqs.emplace_back(params);
    reqs.back().AddTokens(prompt);
    reqs.back().SetOpaqueData(reqs.back().get());
    engine.Add(reqs.back());
  }
  for (int guard_n = 0; engine.HasPendingRequests() && guard_n < 1000; ++guard_n) {
    ogb::Request ready = engine.Step();
    while (ready && ready.HasUnseenTokens()) out[ready.GetOpaqueData()].push_back(ready.GetUnseenToken());
  }
  for (auto& r : reqs) {
    while (r.HasUnseenTokens()) out[r.GetOpaqueData()].push_back(r.GetUnseenToken());
    engine.Remove(r);
  }
  Print("engine_0", out[reqs[0].get()]);
  printf("engine_rows_equal: %s\n", out[reqs[0].get()] == out[reqs[1].get()] && out[reqs[1].get()] == out[reqs[2].get()] ? "yes" : "no");
  return 0;
}
