// pybind11 bindings of the native runtime core (module name: _og_native).
#include <pybind11/functional.h>
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "config.h"
#include "engine_core.h"
#include "search.h"
#include "speculative.h"
#include "tracing.h"

namespace py = pybind11;
using namespace ogb;
using namespace ogb::engine;

using IntArray = py::array_t<int32_t, py::array::c_style | py::array::forcecast>;
using FloatArray = py::array_t<float, py::array::c_style | py::array::forcecast>;

static py::dict SearchToDict(const SearchConfig& s) {
  py::dict d;
  d["do_sample"] = s.do_sample; d["min_length"] = s.min_length; d["max_length"] = s.max_length;
  d["batch_size"] = s.batch_size; d["num_beams"] = s.num_beams; d["num_return_sequences"] = s.num_return_sequences;
  d["repetition_penalty"] = s.repetition_penalty; d["top_k"] = s.top_k; d["top_p"] = s.top_p;
  d["temperature"] = s.temperature; d["early_stopping"] = s.early_stopping;
  d["no_repeat_ngram_size"] = s.no_repeat_ngram_size; d["diversity_penalty"] = s.diversity_penalty;
  d["length_penalty"] = s.length_penalty; d["past_present_share_buffer"] = s.past_present_share_buffer;
  d["random_seed"] = s.random_seed; d["blank_penalty"] = s.blank_penalty;
  d["chunk_size"] = s.chunk_size ? py::cast(*s.chunk_size) : py::cast(0);
  return d;
}

static py::dict SpecToDict(const SpeculativeConfig& s) {
  py::dict d;
  d["max_draft_tokens"] = s.max_draft_tokens; d["ngram_size"] = s.ngram_size;
  d["ngram_chained_lookup"] = s.ngram_chained_lookup; d["min_adaptive_k"] = s.min_adaptive_k; d["cooldown"] = s.cooldown;
  return d;
}

static py::dict DecoderToDict(const DecoderConfig& d) {
  py::dict o;
  o["filename"] = d.filename; o["hidden_size"] = d.hidden_size; o["num_attention_heads"] = d.num_attention_heads;
  o["num_key_value_heads"] = d.num_key_value_heads; o["num_hidden_layers"] = d.num_hidden_layers; o["head_size"] = d.head_size;
  py::dict in, out;
  for (auto& p : d.inputs) in[py::str(p.first)] = p.second;
  for (auto& p : d.outputs) out[py::str(p.first)] = p.second;
  o["inputs"] = in; o["outputs"] = out;
  if (d.sliding_window) {
    py::dict w;
    w["window_size"] = d.sliding_window->window_size; w["pad_value"] = d.sliding_window->pad_value;
    w["alignment"] = d.sliding_window->alignment; w["slide_key_value_cache"] = d.sliding_window->slide_key_value_cache;
    w["slide_inputs"] = d.sliding_window->slide_inputs; w["layers"] = d.sliding_window->layers;
    w["cache_slack"] = d.sliding_window->cache_slack;
    o["sliding_window"] = w;
  } else o["sliding_window"] = py::none();
  py::list provs;
  for (auto& p : d.session_options.provider_options) {
    py::dict opts;
    for (auto& kv : p.options) opts[py::str(kv.first)] = kv.second;
    provs.append(py::make_tuple(p.name, opts));
  }
  o["provider_options"] = provs;
  o["graph_capture"] = IsGraphCaptureEnabled(d.session_options);
  return o;
}

PYBIND11_MODULE(_og_native, m) {
  m.doc() = "native runtime core: config, search, sampling math, speculative helpers, engine scheduler";

  // ------------------------------------------------------------------ config
  py::class_<Config>(m, "Config")
      .def(py::init<const std::string&, std::string_view>(), py::arg("dir"), py::arg("overlay") = "")
      .def_static("from_json", &Config::FromJson, py::arg("text"), py::arg("overlay") = "")
      .def("overlay", &Config::Overlay)
      .def("to_json", &Config::ToJson, py::arg("indent") = 2)
      .def("clear_providers", &Config::ClearProviders)
      .def("append_provider", &Config::AppendProvider)
      .def("set_provider_option", &Config::SetProviderOption)
      .def_readonly("config_path", &Config::config_path)
      .def_property_readonly("model_type", [](const Config& c) { return c.model.type; })
      .def_property_readonly("vocab_size", [](const Config& c) { return c.model.vocab_size; })
      .def_property_readonly("context_length", [](const Config& c) { return c.model.context_length; })
      .def_property_readonly("pad_token_id", [](const Config& c) { return c.model.pad_token_id; })
      .def_property_readonly("bos_token_id", [](const Config& c) { return c.model.bos_token_id; })
      .def_property_readonly("eos_token_ids", [](const Config& c) { return c.model.eos_token_id; })
      .def_property_readonly("tokenizer_dir", [](const Config& c) { return c.model.tokenizer_dir; })
      .def_property_readonly("decoder", [](const Config& c) { return DecoderToDict(c.model.decoder); })
      .def_property_readonly("draft", [](const Config& c) -> py::object {
        if (!c.model.draft) return py::none();
        return DecoderToDict(*c.model.draft);
      })
      .def_property_readonly("search", [](const Config& c) { return SearchToDict(c.search); })
      .def_property_readonly("speculative", [](const Config& c) { return SpecToDict(c.speculative); })
      .def_property_readonly("engine", [](const Config& c) {
        py::dict d;
        if (c.engine.dynamic_batching) {
          py::dict x;
          auto& e = *c.engine.dynamic_batching;
          x["block_size"] = e.block_size; x["max_batch_size"] = e.max_batch_size;
          x["max_scheduled_tokens"] = e.max_scheduled_tokens;
          x["num_blocks"] = e.num_blocks ? py::cast(*e.num_blocks) : py::none();
          x["gpu_utilization_factor"] = e.gpu_utilization_factor ? py::cast(*e.gpu_utilization_factor) : py::none();
          d["dynamic_batching"] = x;
        }
        if (c.engine.static_batching) {
          py::dict x;
          x["max_batch_size"] = c.engine.static_batching->max_batch_size;
          d["static_batching"] = x;
        }
        return d;
      });
  m.def("validate_config_path", [](const std::string& p, const std::string& ctx) { ValidateConfigPath(p, ctx); },
        py::arg("path"), py::arg("context") = "");
  m.def("validate_search_option", [](const std::string& name, py::object v) {
    SearchConfig s;
    if (py::isinstance<py::bool_>(v)) SetSearchBool(s, name, v.cast<bool>());
    else SetSearchNumber(s, name, v.cast<double>());
  });
  m.def("validate_speculative_option", [](const std::string& name, py::object v) {
    SpeculativeConfig s;
    if (py::isinstance<py::bool_>(v)) SetSpeculativeBool(s, name, v.cast<bool>());
    else SetSpeculativeNumber(s, name, v.cast<double>());
  });

  // ------------------------------------------------------------------ search
  py::class_<SearchParams>(m, "SearchParams")
      .def(py::init<>())
      .def_readwrite("batch_size", &SearchParams::batch_size)
      .def_readwrite("num_beams", &SearchParams::num_beams)
      .def_readwrite("num_return_sequences", &SearchParams::num_return_sequences)
      .def_readwrite("max_length", &SearchParams::max_length)
      .def_readwrite("min_length", &SearchParams::min_length)
      .def_readwrite("vocab_size", &SearchParams::vocab_size)
      .def_readwrite("pad_token_id", &SearchParams::pad_token_id)
      .def_readwrite("eos_token_ids", &SearchParams::eos_token_ids)
      .def_readwrite("repetition_penalty", &SearchParams::repetition_penalty)
      .def_readwrite("no_repeat_ngram_size", &SearchParams::no_repeat_ngram_size)
      .def_readwrite("length_penalty", &SearchParams::length_penalty)
      .def_readwrite("early_stopping", &SearchParams::early_stopping)
      .def_readwrite("random_seed", &SearchParams::random_seed);

  py::class_<SearchCheckpoint>(m, "SearchCheckpoint");

  py::class_<Search>(m, "Search")
      .def(py::init([](const SearchParams& p) { return MakeSearch(p); }))
      .def_property_readonly("length", &Search::Length)
      .def_property_readonly("is_done", &Search::IsDone)
      .def_property_readonly("is_beam", &Search::IsBeam)
      .def("append_tokens", [](Search& s, IntArray ids) {
        if (ids.ndim() == 1) s.AppendTokens(ids.data(), 1, int(ids.shape(0)));
        else if (ids.ndim() == 2) s.AppendTokens(ids.data(), int(ids.shape(0)), int(ids.shape(1)));
        else throw std::runtime_error("append_tokens expects a 1-D or 2-D int32 array");
      })
      .def("rewind_to", &Search::RewindTo)
      .def("next_tokens", [](Search& s) { return IntArray(s.NextTokens().size(), s.NextTokens().data()); })
      .def("sequence", [](Search& s, int row) {
        if (row < 0 || row >= s.Seqs().Rows()) throw std::out_of_range("sequence index out of range");
        return IntArray(size_t(s.Length()), s.Seqs().Row(row));
      })
      // Host scoring: logits [rows, vocab] float32, modified in place by the processors.
      .def("score", [](Search& s, py::array_t<float, py::array::c_style> logits, const std::string& method, int k, float p, float t) {
        auto& P = s.Params();
        if (logits.size() != ssize_t(P.BatchBeam()) * P.vocab_size) throw std::runtime_error("logits must be [batch*beams, vocab]");
        s.SetLogits(logits.mutable_data());
        if (P.min_length > 0) s.ApplyMinLength();
        if (P.repetition_penalty != 1.f) s.ApplyRepetitionPenalty();
        if (P.no_repeat_ngram_size > 0) s.ApplyNoRepeatNgram();
        if (method == "greedy" || method == "beam") s.SelectTop();
        else if (method == "top_k") s.SampleTopK(k, t);
        else if (method == "top_p") s.SampleTopP(p, t);
        else if (method == "top_k_top_p") s.SampleTopKTopP(k, p, t);
        else throw std::runtime_error("unknown sampling method " + method);
        s.SetLogits(nullptr);
      }, py::arg("logits"), py::arg("method"), py::arg("top_k") = 0, py::arg("top_p") = 0.f, py::arg("temperature") = 1.f)
      .def("apply_processors", [](Search& s, py::array_t<float, py::array::c_style> logits) {
        auto& P = s.Params();
        s.SetLogits(logits.mutable_data());
        if (P.min_length > 0) s.ApplyMinLength();
        if (P.repetition_penalty != 1.f) s.ApplyRepetitionPenalty();
        if (P.no_repeat_ngram_size > 0) s.ApplyNoRepeatNgram();
        s.SetLogits(nullptr);
      })
      .def("commit_tokens", [](Search& s, IntArray toks) {
        if (toks.size() != s.Params().BatchBeam()) throw std::runtime_error("commit_tokens: one token per row required");
        s.CommitTokens(toks.data());
      })
      .def("commit_beam_step", [](Search& s, FloatArray cs, IntArray ct, IntArray cb) {
        auto* b = dynamic_cast<BeamSearch*>(&s);
        if (!b) throw std::runtime_error("not a beam search");
        ssize_t want = ssize_t(s.Params().batch_size) * 2 * s.Params().num_beams;
        if (cs.size() != want || ct.size() != want || cb.size() != want) throw std::runtime_error("beam candidates must be [batch, 2*num_beams]");
        b->CommitBeamStep(cs.data(), ct.data(), cb.data());
      })
      .def("commit_beam_result", [](Search& s, IntArray toks, IntArray rows, bool all_done) {
        auto* b = dynamic_cast<BeamSearch*>(&s);
        if (!b) throw std::runtime_error("not a beam search");
        if (toks.size() != s.Params().BatchBeam() || rows.size() != s.Params().BatchBeam())
          throw std::runtime_error("commit_beam_result: one token and one source row per row required");
        b->CommitBeamResult(toks.data(), rows.data(), all_done);
      })
      .def("set_hypothesis", [](Search& s, int batch, int rank, IntArray toks, float score) {
        auto* b = dynamic_cast<BeamSearch*>(&s);
        if (!b) throw std::runtime_error("not a beam search");
        b->SetHypothesis(batch, rank, toks.data(), int(toks.size()), score);
      })
      .def("beam_rows", [](Search& s) {
        auto* b = dynamic_cast<BeamSearch*>(&s);
        if (!b) throw std::runtime_error("not a beam search");
        return IntArray(b->NextRows().size(), b->NextRows().data());
      })
      .def("beam_scores", [](Search& s) {
        auto* b = dynamic_cast<BeamSearch*>(&s);
        if (!b) throw std::runtime_error("not a beam search");
        return FloatArray(b->BeamScores().size(), b->BeamScores().data());
      })
      .def("finalize", [](Search& s) { if (auto* b = dynamic_cast<BeamSearch*>(&s)) b->Finalize(); })
      .def("hypothesis", [](Search& s, int batch, int rank) {
        auto* b = dynamic_cast<BeamSearch*>(&s);
        if (!b) throw std::runtime_error("not a beam search");
        auto& h = b->Hypothesis(batch, rank);
        return py::make_tuple(IntArray(h.tokens.size(), h.tokens.data()), h.score);
      })
      .def("save", &Search::Save)
      .def("restore", &Search::Restore)
      .def("uniform", [](Search& s) { return std::uniform_real_distribution<float>(0.f, 1.f)(s.Rng()); });

  // ------------------------------------------------------------------ sampling math (tests, speculative)
  m.def("sampled_distribution", [](FloatArray logits, int k, float p, float t) {
    SparseDist d;
    std::vector<int32_t> scratch;
    BuildSampledDistribution(logits.data(), int(logits.size()), k, p, t, d, scratch);
    return py::make_tuple(IntArray(d.ids.size(), d.ids.data()), FloatArray(d.probs.size(), d.probs.data()));
  });
  m.def("apply_repetition_penalty", [](py::array_t<float, py::array::c_style> logits, IntArray prefix, float penalty) {
    std::vector<uint8_t> seen;
    ApplyRepetitionPenalty(logits.mutable_data(), int(logits.size()), prefix.data(), size_t(prefix.size()), penalty, seen);
  });
  m.def("apply_no_repeat_ngram", [](py::array_t<float, py::array::c_style> logits, IntArray prefix, int n) {
    ApplyNoRepeatNgram(logits.mutable_data(), int(logits.size()), prefix.data(), size_t(prefix.size()), n);
  });
  m.def("apply_min_length", [](py::array_t<float, py::array::c_style> logits, int cur, int min_len, std::vector<int32_t> eos) {
    ApplyMinLength(logits.mutable_data(), int(logits.size()), cur, min_len, eos);
  });
  m.def("no_repeat_ngram_banned", [](IntArray prefix, int n, int vocab) {
    // Tokens that would complete a repeated n-gram (used to build device edit lists).
    std::vector<float> tmp(size_t(vocab), 0.f);
    ApplyNoRepeatNgram(tmp.data(), vocab, prefix.data(), size_t(prefix.size()), n);
    std::vector<int32_t> out;
    for (int v = 0; v < vocab; ++v) if (tmp[size_t(v)] != 0.f) out.push_back(v);
    return out;
  });
  m.def("accept_probability", &AcceptProbability);

  // ------------------------------------------------------------------ speculative helpers
  py::class_<NGramIndex>(m, "NGramIndex")
      .def(py::init<int>())
      .def("append", [](NGramIndex& n, IntArray t) { n.Append(t.data(), size_t(t.size())); })
      .def("reset", [](NGramIndex& n, IntArray t) { n.Reset(t.data(), size_t(t.size())); })
      .def("propose", &NGramIndex::Propose, py::arg("max_tokens"), py::arg("chained") = false)
      .def_property_readonly("history_size", &NGramIndex::HistorySize)
      .def_property_readonly("hits", &NGramIndex::Hits)
      .def_property_readonly("misses", &NGramIndex::Misses)
      .def_property_readonly("ngram_size", &NGramIndex::NGramSize);
  py::class_<AdaptiveK>(m, "AdaptiveK")
      .def(py::init<int, int>())
      .def_property_readonly("k", &AdaptiveK::K)
      .def_property_readonly("min_k", &AdaptiveK::MinK)
      .def_property_readonly("increases", &AdaptiveK::Increases)
      .def_property_readonly("decreases", &AdaptiveK::Decreases)
      .def_property_readonly("probes", &AdaptiveK::Probes)
      .def("record", &AdaptiveK::Record)
      .def("reset", &AdaptiveK::Reset);
  py::class_<ZeroAcceptCooldown>(m, "ZeroAcceptCooldown")
      .def(py::init<bool>())
      .def("should_skip_round", &ZeroAcceptCooldown::ShouldSkipRound)
      .def("record", &ZeroAcceptCooldown::Record)
      .def_property_readonly("skips", &ZeroAcceptCooldown::Skips);
  m.def("verify_greedy", [](IntArray draft, FloatArray target_logits) {
    int k = int(draft.size());
    if (target_logits.ndim() != 2 || target_logits.shape(0) != k + 1) throw std::runtime_error("target logits must be [K+1, vocab]");
    auto r = VerifyGreedy(draft.data(), k, target_logits.data(), int(target_logits.shape(1)));
    return py::make_tuple(r.accepted, r.commit, r.bonus);
  });
  m.def("verify_sampled", [](IntArray draft, py::list draft_dists, FloatArray target_logits, int top_k, float top_p,
                             float temperature, Search& search) {
    // draft_dists: list of (ids, probs) pairs or None (deterministic proposal -> one-hot).
    int k = int(draft.size());
    if (target_logits.ndim() != 2 || target_logits.shape(0) != k + 1) throw std::runtime_error("target logits must be [K+1, vocab]");
    int vocab = int(target_logits.shape(1));
    std::vector<SparseDist> dd(static_cast<size_t>(k)), td(static_cast<size_t>(k) + 1);
    std::vector<int32_t> scratch;
    for (int i = 0; i <= k; ++i)
      BuildSampledDistribution(target_logits.data() + size_t(i) * vocab, vocab, top_k, top_p, temperature, td[size_t(i)], scratch);
    for (int i = 0; i < k; ++i) {
      if (size_t(i) >= draft_dists.size() || draft_dists[size_t(i)].is_none()) {
        dd[size_t(i)].ids = {draft.data()[i]};
        dd[size_t(i)].probs = {1.f};
      } else {
        auto tup = draft_dists[size_t(i)].cast<py::tuple>();
        auto ids = tup[0].cast<IntArray>();
        auto pr = tup[1].cast<FloatArray>();
        dd[size_t(i)].ids.assign(ids.data(), ids.data() + ids.size());
        dd[size_t(i)].probs.assign(pr.data(), pr.data() + pr.size());
      }
    }
    auto r = VerifySampled(draft.data(), k, dd, td, search.Rng());
    return py::make_tuple(r.accepted, r.commit, r.bonus);
  });

  // ------------------------------------------------------------------ engine
  py::enum_<RequestStatus>(m, "RequestStatus")
      .value("Unassigned", RequestStatus::kUnassigned).value("Assigned", RequestStatus::kAssigned)
      .value("Active", RequestStatus::kActive).value("TurnComplete", RequestStatus::kTurnComplete)
      .value("Closed", RequestStatus::kClosed);
  py::enum_<StepOutcome>(m, "StepOutcome")
      .value("NoWork", StepOutcome::kNoWork).value("CapacityDeferred", StepOutcome::kCapacityDeferred)
      .value("UnserviceableRequest", StepOutcome::kUnserviceableRequest).value("Committed", StepOutcome::kCommitted)
      .value("RetryableBatchAbort", StepOutcome::kRetryableBatchAbort)
      .value("ExecutionCapacityExceeded", StepOutcome::kExecutionCapacityExceeded)
      .value("ExecutionContractFailure", StepOutcome::kExecutionContractFailure)
      .value("FatalExecutionFailure", StepOutcome::kFatalExecutionFailure).value("Planned", StepOutcome::kPlanned);
  py::enum_<FailureKind>(m, "FailureKind")
      .value("RetryableBeforeExecution", FailureKind::kRetryableBeforeExecution)
      .value("RetryableDuringExecution", FailureKind::kRetryableDuringExecution)
      .value("CapacityExceeded", FailureKind::kCapacityExceeded).value("Fatal", FailureKind::kFatal)
      .value("PostProcessing", FailureKind::kPostProcessing);

  py::class_<RequestOptions>(m, "RequestOptions")
      .def(py::init<>())
      .def_readwrite("max_length", &RequestOptions::max_length).def_readwrite("min_length", &RequestOptions::min_length)
      .def_readwrite("do_sample", &RequestOptions::do_sample).def_readwrite("top_k", &RequestOptions::top_k)
      .def_readwrite("top_p", &RequestOptions::top_p).def_readwrite("temperature", &RequestOptions::temperature)
      .def_readwrite("repetition_penalty", &RequestOptions::repetition_penalty)
      .def_readwrite("no_repeat_ngram_size", &RequestOptions::no_repeat_ngram_size)
      .def_readwrite("random_seed", &RequestOptions::random_seed).def_readwrite("chunk_size", &RequestOptions::chunk_size)
      .def_readwrite("num_beams", &RequestOptions::num_beams).def_readwrite("batch_size", &RequestOptions::batch_size)
      .def("resolve", [](const RequestOptions& o) { auto a = o.Resolve(); return py::make_tuple(a.top_k, a.top_p, a.temperature); });

  py::class_<Request, std::shared_ptr<Request>>(m, "Request")
      .def_property_readonly("id", &Request::Id)
      .def_property_readonly("status", &Request::Status)
      .def_property_readonly("options", &Request::Options)
      .def_property_readonly("processed", &Request::Processed)
      .def_property_readonly("pending", &Request::Pending)
      .def_property_readonly("is_prefill", &Request::IsPrefill)
      .def_property_readonly("seed", &Request::Seed)
      .def("tokens", [](const Request& r) { return IntArray(r.Tokens().size(), r.Tokens().data()); })
      .def_property_readonly("num_tokens", [](const Request& r) { return r.Tokens().size(); })
      .def("add_tokens", [](Request& r, IntArray ids) { r.AddTokens(ids.data(), size_t(ids.size())); })
      .def("continue_with", [](Request& r, IntArray ids, int new_max_length) { r.ContinueWith(ids.data(), size_t(ids.size()), new_max_length); },
           py::arg("ids"), py::arg("new_max_length") = 0)
      .def("has_unseen_tokens", &Request::HasUnseen)
      .def("get_unseen_token", &Request::PopUnseen)
      .def("is_turn_complete", &Request::TurnComplete)
      .def("set_draft", [](Request& r, IntArray ids) { return r.SetDraft(ids.data(), size_t(ids.size())); })
      .def_property_readonly("draft_count", &Request::DraftCount)
      .def("blocks", [](const Request& r) { return r.Blocks(); })
      .def("window_blocks", [](const Request& r) { return r.WindowBlocks(); });

  py::class_<PlanEntry>(m, "PlanEntry")
      .def_readonly("request", &PlanEntry::request).def_readonly("num_tokens", &PlanEntry::num_tokens)
      .def_readonly("packed_offset", &PlanEntry::packed_offset).def_readonly("logits_row", &PlanEntry::logits_row)
      .def_readonly("processed_before", &PlanEntry::processed_before).def_readonly("is_prefill", &PlanEntry::is_prefill)
      .def_readonly("samples", &PlanEntry::samples).def_readonly("newly_admitted", &PlanEntry::newly_admitted);
  py::class_<StepPlan>(m, "StepPlan")
      .def_readonly("outcome", &StepPlan::outcome).def_readonly("entries", &StepPlan::entries)
      .def_readonly("token_count", &StepPlan::token_count).def_readonly("max_query_len", &StepPlan::max_query_len)
      .def_readonly("max_kv_len", &StepPlan::max_kv_len).def_readonly("block_table_columns", &StepPlan::block_table_columns)
      .def_readonly("graph_eligible", &StepPlan::graph_eligible).def_readonly("unserviceable", &StepPlan::unserviceable)
      .def_readonly("deferred", &StepPlan::deferred).def_readonly("lookahead_ok", &StepPlan::lookahead_ok)
      .def_readonly("signature", &StepPlan::signature).def_readonly("next_signature", &StepPlan::next_signature)
      .def_property_readonly("batch", [](const StepPlan& p) { return p.entries.size(); });

  py::class_<EngineOptions>(m, "EngineOptions")
      .def(py::init<>())
      .def_readwrite("block_size", &EngineOptions::block_size).def_readwrite("num_blocks", &EngineOptions::num_blocks)
      .def_readwrite("max_batch_size", &EngineOptions::max_batch_size)
      .def_readwrite("static_batching", &EngineOptions::static_batching)
      .def_readwrite("max_scheduled_tokens", &EngineOptions::max_scheduled_tokens)
      .def_readwrite("window_size", &EngineOptions::window_size).def_readwrite("lookahead", &EngineOptions::lookahead)
      .def_readwrite("lookahead_execution", &EngineOptions::lookahead_execution)
      .def_readwrite("num_window_blocks", &EngineOptions::num_window_blocks)
      .def_readwrite("vocab_size", &EngineOptions::vocab_size).def_readwrite("pad_token_id", &EngineOptions::pad_token_id)
      .def_readwrite("eos_ids", &EngineOptions::eos_ids);

  py::class_<EngineCore>(m, "EngineCore")
      .def(py::init<EngineOptions>())
      .def("create_request", &EngineCore::CreateRequest)
      .def("add_request", &EngineCore::AddRequest)
      .def("remove_request", &EngineCore::RemoveRequest)
      .def("has_pending_requests", &EngineCore::HasPendingRequests)
      .def_property_readonly("healthy", &EngineCore::Healthy)
      .def("plan", &EngineCore::Plan, py::return_value_policy::reference_internal)
      // Buffer addresses are raw host pointers (pinned torch tensors): a dict name -> address.
      .def("pack", [](EngineCore& e, py::dict a, int max_tokens, int max_batch, int table_columns) {
        auto P = [&](const char* k) -> uintptr_t { return a.contains(k) ? a[k].cast<uintptr_t>() : 0; };
        PackBuffers b;
        b.input_ids = reinterpret_cast<int32_t*>(P("input_ids")); b.positions = reinterpret_cast<int32_t*>(P("positions"));
        b.token_row = reinterpret_cast<int32_t*>(P("token_row")); b.slot_mapping = reinterpret_cast<int32_t*>(P("slot_mapping"));
        b.slot_mapping_w = reinterpret_cast<int32_t*>(P("slot_mapping_w")); b.cu_seqlens = reinterpret_cast<int32_t*>(P("cu_seqlens"));
        b.past_lens = reinterpret_cast<int32_t*>(P("past_lens")); b.logits_rows = reinterpret_cast<int32_t*>(P("logits_rows"));
        b.block_table = reinterpret_cast<int32_t*>(P("block_table")); b.block_table_w = reinterpret_cast<int32_t*>(P("block_table_w"));
        b.top_k = reinterpret_cast<int32_t*>(P("top_k")); b.top_p = reinterpret_cast<float*>(P("top_p"));
        b.temperature = reinterpret_cast<float*>(P("temperature")); b.seeds = reinterpret_cast<uint64_t*>(P("seeds"));
        b.sample_pos = reinterpret_cast<int32_t*>(P("sample_pos"));
        b.max_tokens = max_tokens; b.max_batch = max_batch; b.table_columns = table_columns;
        for (void* p : {(void*)b.input_ids, (void*)b.positions, (void*)b.token_row, (void*)b.slot_mapping, (void*)b.cu_seqlens,
                        (void*)b.past_lens, (void*)b.logits_rows, (void*)b.block_table, (void*)b.top_k, (void*)b.top_p,
                        (void*)b.temperature, (void*)b.seeds, (void*)b.sample_pos})
          if (!p) throw std::runtime_error("pack: a required staging buffer is missing");
        e.Pack(b);
      })
      .def("commit", [](EngineCore& e, IntArray toks) { return e.Commit(toks.data(), size_t(toks.size())); })
      .def("commit_speculative", [](EngineCore& e, IntArray accepted, IntArray toks) {
        if (accepted.size() != toks.size()) throw std::invalid_argument("commit_speculative: arrays of different lengths");
        return e.CommitSpeculative(accepted.data(), toks.data(), size_t(toks.size()));
      })
      .def("abort", &EngineCore::Abort, py::arg("kind"), py::arg("what") = "")
      .def_property_readonly("transaction_open", &EngineCore::TransactionOpen)
      .def("next_ready", &EngineCore::NextReady)
      .def("check_invariants", &EngineCore::CheckInvariants)
      .def_property_readonly("free_blocks", &EngineCore::FreeBlocks)
      .def_property_readonly("free_window_blocks", &EngineCore::FreeWindowBlocks)
      .def_property_readonly("ring_blocks_per_request", &EngineCore::RingBlocksPerRequest)
      .def_property_readonly("metrics", [](const EngineCore& e) {
        auto& x = e.Metrics();
        py::dict d;
        d["steps_committed"] = x.steps_committed; d["steps_aborted"] = x.steps_aborted; d["steps_deferred"] = x.steps_deferred;
        d["requests_admitted"] = x.requests_admitted; d["requests_completed"] = x.requests_completed;
        d["tokens_scheduled"] = x.tokens_scheduled; d["tokens_generated"] = x.tokens_generated; d["unserviceable"] = x.unserviceable;
        return d;
      });

  py::class_<BlockPool>(m, "BlockPool")
      .def(py::init<int>())
      .def_property_readonly("total", &BlockPool::Total)
      .def_property_readonly("free_count", &BlockPool::FreeCount)
      .def("reserve", [](BlockPool& p, int n) -> py::object {
        std::vector<int> out;
        if (!p.Reserve(n, out)) return py::none();
        return py::cast(out);
      })
      .def("commit", &BlockPool::Commit).def("release", &BlockPool::Release).def("free", &BlockPool::Free);

  // ------------------------------------------------------------------ tracing / logging
  m.def("trace_enable", [](const std::string& path) { Tracer::Get().Enable(path); }, py::arg("path") = "");
  m.def("trace_disable", [] { Tracer::Get().Disable(); });
  m.def("trace_enabled", [] { return Tracer::Get().Enabled(); });
  m.def("trace_now_us", &Tracer::NowUs);
  m.def("trace_complete", [](const std::string& cat, const std::string& name, int64_t t0, int64_t dur) {
    static std::vector<std::string> cats;  // category strings must outlive the call
    Tracer::Get().Complete(cat == "model" ? "model" : cat == "engine" ? "engine" : "generator", name, t0, dur);
  });
  m.def("log_set_bool", [](const std::string& n, bool v) { Log::Get().SetBool(n, v); });
  m.def("log_set_string", [](const std::string& n, const std::string& v) { Log::Get().SetString(n, v); });
  m.def("log_flag", [](const std::string& n) { return Log::Get().Flag(n); });
  m.def("log_set_callback", [](py::object cb) {
    if (cb.is_none()) Log::Get().SetCallback(nullptr);
    else Log::Get().SetCallback([cb](const std::string& s) { py::gil_scoped_acquire g; cb(s); });
  });
  m.def("log_write", [](const std::string& label, const std::string& text) { Log::Get().Write(label, text); });
}
