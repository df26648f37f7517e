// genai_config.json: strict, schema-validated configuration.
//
// Behavioural contract taken from the reference (src/config.h:142-549, src/config.cpp:1497-1671,
// 1931-2148): root keys model/search/speculative/engine; an unknown key anywhere is an error that
// names its path; a JSON overlay can be applied after load; search.max_length defaults to
// model.context_length; eos_token_id may be a scalar or a list and defaults to pad_token_id;
// speculative and engine options are range checked; dynamic and static batching are mutually
// exclusive (the later one wins); file names must stay inside the model directory.
//
// Design: the document is parsed to a tree, validated against a declarative schema table and then
// projected into the typed structs below.  Sections the B200 runtime does not execute (vision,
// speech, encoder ...) are still validated so that a reference config loads unchanged.
#pragma once
#include <optional>
#include <string>
#include <string_view>
#include <utility>
#include <vector>

#include "json.h"

namespace ogb {

struct ProviderOptions {
  std::string name;
  std::vector<std::pair<std::string, std::string>> options;
};

struct SessionOptions {
  std::optional<std::string> log_id;
  std::optional<std::string> enable_profiling;
  std::vector<ProviderOptions> provider_options;
  std::vector<std::string> providers;  // runtime list, mirrors provider_options order
};

struct SlidingWindow {
  int window_size{};
  int pad_value{};
  std::string alignment{"right"};
  bool slide_key_value_cache{true};
  bool slide_inputs{true};
  std::vector<int> layers;
  int cache_slack{0};
};

struct DecoderConfig {
  std::string filename;
  SessionOptions session_options;
  int hidden_size{};
  int num_attention_heads{};
  int num_key_value_heads{};
  int num_hidden_layers{};
  int head_size{};
  std::optional<SlidingWindow> sliding_window;
  std::vector<std::pair<std::string, std::string>> inputs;   // nominal name -> graph name
  std::vector<std::pair<std::string, std::string>> outputs;  // nominal name -> graph name
  std::string Input(std::string_view nominal) const;
  std::string Output(std::string_view nominal) const;
};

struct ModelConfig {
  std::string type;
  std::string tokenizer_dir;
  int pad_token_id{};
  std::vector<int> eos_token_id;
  int bos_token_id{};
  int vocab_size{};
  int context_length{};
  DecoderConfig decoder;
  std::optional<DecoderConfig> draft;
};

struct SearchConfig {
  bool do_sample{};
  int min_length{};
  int max_length{};
  int batch_size{1};
  int num_beams{1};
  int num_return_sequences{1};
  float repetition_penalty{1.0f};
  int top_k{50};
  float top_p{};
  float temperature{1.0f};
  bool early_stopping{true};
  int no_repeat_ngram_size{};
  float diversity_penalty{};
  float length_penalty{1.0f};
  bool past_present_share_buffer{};
  int random_seed{-1};
  std::optional<size_t> chunk_size;
  float blank_penalty{};
};

struct SpeculativeConfig {
  int max_draft_tokens{4};
  int ngram_size{};
  bool ngram_chained_lookup{};
  int min_adaptive_k{};
  bool cooldown{};
};

struct DynamicBatching {
  size_t block_size{256};
  std::optional<size_t> num_blocks;
  std::optional<float> gpu_utilization_factor;
  size_t max_batch_size{16};
  size_t max_scheduled_tokens{2048};
};
struct StaticBatching {
  size_t max_batch_size{4};
};
struct EngineConfig {
  std::optional<DynamicBatching> dynamic_batching;
  std::optional<StaticBatching> static_batching;
};

struct Config {
  Config() = default;
  // Loads <dir>/genai_config.json, applies the optional overlay, validates and fills defaults.
  Config(const std::string& dir, std::string_view json_overlay = {});
  static Config FromJson(std::string_view json_text, std::string_view json_overlay = {});

  void Overlay(std::string_view json_text);  // merge + revalidate + reproject
  std::string ToJson(int indent = 2) const;  // merged tree

  // Provider management (reference: src/python/python.cpp:543-587).
  void ClearProviders();
  void AppendProvider(std::string_view name);
  void SetProviderOption(std::string_view provider, std::string_view key, std::string_view value);

  std::string config_path;
  ModelConfig model;
  SearchConfig search;
  SpeculativeConfig speculative;
  EngineConfig engine;
  json::Value tree;

 private:
  void Finish();   // validate + project + defaults
  void Project();  // tree -> typed structs
};

void SetSearchNumber(SearchConfig& s, std::string_view name, double value);
void SetSearchBool(SearchConfig& s, std::string_view name, bool value);
void SetSpeculativeNumber(SpeculativeConfig& s, std::string_view name, double value);
void SetSpeculativeBool(SpeculativeConfig& s, std::string_view name, bool value);
int SafeDoubleToInt(double x, std::string_view name);
std::string NormalizeProviderName(std::string_view name);
bool IsGraphCaptureEnabled(const SessionOptions& so);
// Throws if the path is absolute or contains a ".." component; empty is allowed.
void ValidateConfigPath(const std::string& path, std::string_view context = {});

}  // namespace ogb
