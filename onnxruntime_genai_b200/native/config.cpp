#include "config.h"

#include <algorithm>
#include <cctype>
#include <cmath>
#include <fstream>
#include <sstream>
#include <stdexcept>

namespace ogb {
namespace {

// ---------------------------------------------------------------------------------------------
// Schema table.  One letter per node:
//   n number   i integer   b bool   s string
//   I integer or array of integers       A array of integers    S array of strings   F array of numbers
//   o object with listed children        f free-form object (string -> scalar)
//   a array of objects (children describe one element)
//   P provider_options array: [{"<provider>": {"k": "v", ...}}, ...]
//   X session_options: known keys typed, provider_options as P, everything else scalar config entries
//   M map string -> string
struct Schema {
  char t;
  std::vector<std::pair<const char*, Schema>> kids;
};

Schema Leaf(char t) { return Schema{t, {}}; }
Schema Obj(std::vector<std::pair<const char*, Schema>> kids) { return Schema{'o', std::move(kids)}; }
Schema Arr(std::vector<std::pair<const char*, Schema>> kids) { return Schema{'a', std::move(kids)}; }

std::vector<std::pair<const char*, Schema>> Strings(std::initializer_list<const char*> names) {
  std::vector<std::pair<const char*, Schema>> v;
  for (auto* n : names) v.emplace_back(n, Leaf('s'));
  return v;
}

Schema SubModel(std::vector<std::pair<const char*, Schema>> extra, std::initializer_list<const char*> in,
                std::initializer_list<const char*> out) {
  std::vector<std::pair<const char*, Schema>> kids = {
      {"filename", Leaf('s')}, {"session_options", Leaf('X')}, {"run_options", Leaf('f')}};
  for (auto& e : extra) kids.push_back(e);
  kids.emplace_back("inputs", Obj(Strings(in)));
  kids.emplace_back("outputs", Obj(Strings(out)));
  return Obj(std::move(kids));
}

Schema DecoderSchema() {
  Schema shared_init = Arr({{"name", Leaf('s')}, {"data_file", Leaf('s')}, {"offset", Leaf('s')}, {"length", Leaf('s')},
                            {"data_type", Leaf('i')}, {"shape", Leaf('A')}});
  Schema sliding = Obj({{"window_size", Leaf('i')}, {"pad_value", Leaf('i')}, {"alignment", Leaf('s')},
                        {"slide_key_value_cache", Leaf('b')}, {"slide_inputs", Leaf('b')}, {"layers", Leaf('A')},
                        {"cache_slack", Leaf('i')}});
  Schema pipeline_elem = Obj({{"filename", Leaf('s')}, {"session_options", Leaf('X')}, {"run_options", Leaf('f')},
                              {"model_id", Leaf('s')}, {"inputs", Leaf('S')}, {"outputs", Leaf('S')},
                              {"output_names_forwarder", Leaf('M')}, {"run_on_prompt", Leaf('b')},
                              {"run_on_token_gen", Leaf('b')}, {"is_lm_head", Leaf('b')},
                              {"inherit_session_options", Leaf('b')}, {"reset_session_idx", Leaf('i')}});
  // pipeline: [{"<model_id>": {...}}, ...]
  Schema pipeline{'p', {{"*", pipeline_elem}}};
  return SubModel(
      {{"shared_initializers", shared_init}, {"hidden_size", Leaf('i')}, {"num_attention_heads", Leaf('i')},
       {"num_key_value_heads", Leaf('i')}, {"num_hidden_layers", Leaf('i')}, {"head_size", Leaf('i')},
       {"layer_types", Leaf('S')}, {"conv_cache_size", Leaf('i')}, {"sliding_window", sliding}, {"pipeline", pipeline}},
      {"input_ids", "inputs_embeds", "attention_mask", "position_ids", "past_key_names", "past_value_names", "past_names",
       "cross_past_key_names", "cross_past_value_names", "past_key_values_length", "past_sequence_length",
       "current_sequence_length", "total_sequence_length", "cache_indirection", "encoder_hidden_states",
       "rnn_states_prev", "encoder_attention_mask", "cumulative_sequence_lengths", "past_sequence_lengths",
       "block_table", "block_table_windowed", "attention_metadata", "past_conv_names", "hidden_states", "targets",
       "lstm_hidden_state", "lstm_cell_state", "per_layer_inputs", "targets_length"},
      {"logits", "present_key_names", "present_value_names", "present_names", "output_cross_qk_names", "rnn_states",
       "present_conv_names", "hidden_states", "outputs", "lstm_hidden_state", "lstm_cell_state", "outputs_length"});
}

const Schema& Root() {
  static const Schema root = [] {
    Schema encoder = SubModel(
        {{"hidden_size", Leaf('i')}, {"num_attention_heads", Leaf('i')}, {"num_hidden_layers", Leaf('i')},
         {"num_key_value_heads", Leaf('i')}, {"head_size", Leaf('i')}},
        {"input_ids", "inputs_embeds", "attention_mask", "position_ids", "audio_features", "length", "cache_last_channel",
         "cache_last_time", "cache_last_channel_len", "lang_id"},
        {"encoder_outputs", "encoder_hidden_states", "cross_present_key_names", "cross_present_value_names",
         "encoded_lengths", "cache_last_channel_next", "cache_last_time_next", "cache_last_channel_len_next"});
    Schema embedding = SubModel({}, {"input_ids", "image_features", "audio_features"}, {"inputs_embeds", "per_layer_inputs"});
    Schema vision_stage = Arr({{"filename", Leaf('s')}, {"session_options", Leaf('X')}, {"run_options", Leaf('f')},
                               {"model_id", Leaf('s')}, {"inputs", Leaf('S')}, {"outputs", Leaf('S')}, {"run_on_cpu", Leaf('b')}});
    Schema vision = SubModel(
        {{"spatial_merge_size", Leaf('i')}, {"tokens_per_second", Leaf('n')}, {"num_visual_tokens", Leaf('i')},
         {"patch_size", Leaf('i')}, {"window_size", Leaf('i')}, {"config_filename", Leaf('s')},
         {"adapter_filename", Leaf('s')}, {"pipeline", vision_stage}},
        {"pixel_values", "pixel_position_ids", "image_sizes", "image_grid_thw", "attention_mask"}, {"image_features"});
    Schema speech = SubModel({{"config_filename", Leaf('s')}, {"adapter_filename", Leaf('s')}},
                             {"audio_embeds", "attention_mask", "audio_sizes", "audio_projection_mode"}, {"audio_features"});
    Schema joiner = SubModel({}, {"encoder_outputs", "decoder_outputs"}, {"logits"});
    Schema vad = Obj({{"filename", Leaf('s')}, {"threshold", Leaf('n')}, {"silence_duration_ms", Leaf('i')},
                      {"prefix_padding_ms", Leaf('i')}, {"session_options", Leaf('X')}, {"run_options", Leaf('f')}});
    Schema mtp = SubModel(
        {{"shared_initializers", Arr({{"name", Leaf('s')}, {"data_file", Leaf('s')}, {"offset", Leaf('s')},
                                      {"length", Leaf('s')}, {"data_type", Leaf('i')}, {"shape", Leaf('A')}})},
         {"num_hidden_layers", Leaf('i')}, {"num_key_value_heads", Leaf('i')}, {"head_size", Leaf('i')},
         {"main_hidden_states", Leaf('s')}},
        {"input_ids", "hidden_states", "attention_mask", "position_ids", "past_key_names", "past_value_names"},
        {"logits", "hidden_states", "present_key_names", "present_value_names"});

    std::vector<std::pair<const char*, Schema>> model = {
        {"type", Leaf('s')}, {"tokenizer_dir", Leaf('s')}, {"pad_token_id", Leaf('i')}, {"eos_token_id", Leaf('I')},
        {"bos_token_id", Leaf('i')}, {"sep_token_id", Leaf('i')}, {"decoder_start_token_id", Leaf('i')},
        {"image_token_id", Leaf('i')}, {"audio_token_id", Leaf('i')}, {"boa_token_id", Leaf('i')},
        {"video_token_id", Leaf('i')}, {"vision_start_token_id", Leaf('i')}, {"bot_token_id", Leaf('i')},
        {"eot_token_id", Leaf('i')}, {"bor_token_id", Leaf('i')}, {"eor_token_id", Leaf('i')},
        {"vocab_size", Leaf('i')}, {"context_length", Leaf('i')}, {"num_mels", Leaf('i')}, {"fft_size", Leaf('i')},
        {"hop_length", Leaf('i')}, {"win_length", Leaf('i')}, {"preemph", Leaf('n')}, {"log_eps", Leaf('n')},
        {"norm_eps", Leaf('n')}, {"subsampling_factor", Leaf('i')}, {"left_context", Leaf('i')},
        {"conv_context", Leaf('i')}, {"pre_encode_cache_size", Leaf('i')}, {"sample_rate", Leaf('i')},
        {"chunk_samples", Leaf('i')}, {"blank_id", Leaf('i')}, {"max_symbols_per_step", Leaf('i')},
        {"left_context_samples", Leaf('i')}, {"right_context_samples", Leaf('i')}, {"tdt_durations", Leaf('A')},
        {"encoder", encoder}, {"embedding", embedding}, {"vision", vision}, {"speech", speech}, {"joiner", joiner},
        {"vad", vad}, {"decoder", DecoderSchema()}, {"mtp", mtp}, {"draft", DecoderSchema()}};

    Schema search = Obj({{"do_sample", Leaf('b')}, {"min_length", Leaf('i')}, {"max_length", Leaf('i')},
                         {"batch_size", Leaf('i')}, {"num_beams", Leaf('i')}, {"num_return_sequences", Leaf('i')},
                         {"repetition_penalty", Leaf('n')}, {"top_k", Leaf('i')}, {"top_p", Leaf('n')},
                         {"temperature", Leaf('n')}, {"early_stopping", Leaf('b')}, {"no_repeat_ngram_size", Leaf('i')},
                         {"diversity_penalty", Leaf('n')}, {"length_penalty", Leaf('n')},
                         {"past_present_share_buffer", Leaf('b')}, {"random_seed", Leaf('i')}, {"chunk_size", Leaf('n')},
                         {"blank_penalty", Leaf('n')}});
    Schema speculative = Obj({{"max_draft_tokens", Leaf('i')}, {"ngram_size", Leaf('i')}, {"ngram_chained_lookup", Leaf('b')},
                              {"min_adaptive_k", Leaf('i')}, {"cooldown", Leaf('b')}});
    Schema engine = Obj({{"dynamic_batching", Obj({{"block_size", Leaf('i')}, {"num_blocks", Leaf('i')},
                                                   {"gpu_utilization_factor", Leaf('n')}, {"max_batch_size", Leaf('i')},
                                                   {"max_scheduled_tokens", Leaf('i')}})},
                         {"static_batching", Obj({{"max_batch_size", Leaf('i')}})}});
    return Obj({{"model", Obj(model)}, {"search", search}, {"speculative", speculative}, {"engine", engine}});
  }();
  return root;
}

[[noreturn]] void TypeError(const std::string& path, const char* want, const json::Value& v) {
  throw std::runtime_error("genai_config: '" + path + "' must be " + want + ", got " + v.kind_name());
}

bool IsScalar(const json::Value& v) { return v.is_bool() || v.is_number() || v.is_string() || v.is_null(); }

void CheckInteger(const json::Value& v, const std::string& path) {
  if (!v.is_number()) TypeError(path, "an integer", v);
  SafeDoubleToInt(v.num, path);
}

void Validate(const json::Value& v, const Schema& s, const std::string& path) {
  switch (s.t) {
    case 'n': if (!v.is_number()) TypeError(path, "a number", v); return;
    case 'i': CheckInteger(v, path); return;
    case 'b': if (!v.is_bool()) TypeError(path, "a bool", v); return;
    case 's': if (!v.is_string()) TypeError(path, "a string", v); return;
    case 'I':
      if (v.is_number()) { CheckInteger(v, path); return; }
      [[fallthrough]];
    case 'A':
      if (!v.is_array()) TypeError(path, "an array of integers", v);
      for (auto& e : *v.arr) CheckInteger(e, path + "[]");
      return;
    case 'F':
      if (!v.is_array()) TypeError(path, "an array of numbers", v);
      for (auto& e : *v.arr) if (!e.is_number()) TypeError(path + "[]", "a number", e);
      return;
    case 'S':
      if (!v.is_array()) TypeError(path, "an array of strings", v);
      for (auto& e : *v.arr) if (!e.is_string()) TypeError(path + "[]", "a string", e);
      return;
    case 'M':
    case 'f':
      if (!v.is_object()) TypeError(path, "an object", v);
      for (auto& m : *v.obj) if (!IsScalar(m.second)) TypeError(path + "." + m.first, "a scalar", m.second);
      return;
    case 'P':
      if (!v.is_array()) TypeError(path, "an array of {provider: {options}} objects", v);
      for (auto& e : *v.arr) {
        if (!e.is_object()) TypeError(path + "[]", "an object", e);
        for (auto& prov : *e.obj) {
          if (!prov.second.is_object()) TypeError(path + "." + prov.first, "an object", prov.second);
          for (auto& opt : *prov.second.obj)
            if (!IsScalar(opt.second)) TypeError(path + "." + prov.first + "." + opt.first, "a scalar", opt.second);
        }
      }
      return;
    case 'X':
      if (!v.is_object()) TypeError(path, "an object", v);
      for (auto& m : *v.obj) {
        if (m.first == "provider_options") Validate(m.second, Leaf('P'), path + ".provider_options");
        else if (m.first == "config_entries") Validate(m.second, Leaf('f'), path + ".config_entries");
        else if (!IsScalar(m.second)) TypeError(path + "." + m.first, "a scalar", m.second);
      }
      return;
    case 'p':
      if (!v.is_array()) TypeError(path, "an array", v);
      for (auto& e : *v.arr) {
        if (!e.is_object()) TypeError(path + "[]", "an object", e);
        for (auto& stage : *e.obj) Validate(stage.second, s.kids[0].second, path + "." + stage.first);
      }
      return;
    case 'a':
      if (!v.is_array()) TypeError(path, "an array of objects", v);
      for (auto& e : *v.arr) Validate(e, Schema{'o', s.kids}, path + "[]");
      return;
    case 'o': {
      if (!v.is_object()) TypeError(path, "an object", v);
      for (auto& m : *v.obj) {
        const Schema* child = nullptr;
        for (auto& k : s.kids)
          if (m.first == k.first) { child = &k.second; break; }
        if (!child) {
          throw std::runtime_error("genai_config: unknown value \"" + m.first + "\" at " +
                                   (path.empty() ? std::string("the document root") : ("'" + path + "'")));
        }
        Validate(m.second, *child, path.empty() ? m.first : path + "." + m.first);
      }
      return;
    }
  }
}

// Deep merge: objects merge member-wise, everything else replaces.
void Merge(json::Value& dst, const json::Value& src) {
  if (dst.is_object() && src.is_object()) {
    for (auto& m : *src.obj) {
      if (auto* d = dst.find(m.first)) Merge(*d, m.second);
      else dst.obj->emplace_back(m.first, m.second);
    }
  } else {
    dst = src;
  }
}

json::Value DeepCopy(const json::Value& v) { return json::Parse(json::Dump(v)); }

int GetInt(const json::Value& o, const char* k, int dflt) {
  auto* p = o.find(k);
  return p ? SafeDoubleToInt(p->num, k) : dflt;
}
bool GetBool(const json::Value& o, const char* k, bool dflt) {
  auto* p = o.find(k);
  return p ? p->b : dflt;
}
std::string GetStr(const json::Value& o, const char* k, std::string dflt = {}) {
  auto* p = o.find(k);
  return p ? p->str : dflt;
}
std::string ScalarToString(const json::Value& v) {
  if (v.is_string()) return v.str;
  if (v.is_bool()) return v.b ? "1" : "0";
  if (v.is_number()) return json::Dump(v);
  return "";
}

SessionOptions ProjectSession(const json::Value* so) {
  SessionOptions out;
  if (!so) return out;
  if (auto* p = so->find("log_id")) out.log_id = ScalarToString(*p);
  if (auto* p = so->find("enable_profiling")) out.enable_profiling = ScalarToString(*p);
  if (auto* po = so->find("provider_options")) {
    for (auto& e : *po->arr)
      for (auto& prov : *e.obj) {
        ProviderOptions p;
        p.name = NormalizeProviderName(prov.first);
        for (auto& opt : *prov.second.obj) p.options.emplace_back(opt.first, ScalarToString(opt.second));
        out.provider_options.push_back(std::move(p));
      }
  }
  for (auto& p : out.provider_options) out.providers.push_back(p.name);
  return out;
}

DecoderConfig ProjectDecoder(const json::Value& d) {
  static const std::pair<const char*, const char*> kInputDefaults[] = {
      {"input_ids", "input_ids"}, {"inputs_embeds", "inputs_embeds"}, {"attention_mask", "attention_mask"},
      {"position_ids", "position_ids"}, {"past_key_names", "past_key_values.%d.key"},
      {"past_value_names", "past_key_values.%d.value"}, {"cumulative_sequence_lengths", "cumulative_sequence_lengths"},
      {"past_sequence_lengths", "past_sequence_lengths"}, {"block_table", "block_table"},
      {"block_table_windowed", "block_table_windowed"}, {"attention_metadata", "attention_metadata"}};
  static const std::pair<const char*, const char*> kOutputDefaults[] = {
      {"logits", "logits"}, {"present_key_names", "present.%d.key"}, {"present_value_names", "present.%d.value"}};
  DecoderConfig out;
  out.filename = GetStr(d, "filename");
  out.session_options = ProjectSession(d.find("session_options"));
  out.hidden_size = GetInt(d, "hidden_size", 0);
  out.num_attention_heads = GetInt(d, "num_attention_heads", 0);
  out.num_key_value_heads = GetInt(d, "num_key_value_heads", 0);
  out.num_hidden_layers = GetInt(d, "num_hidden_layers", 0);
  out.head_size = GetInt(d, "head_size", 0);
  if (auto* sw = d.find("sliding_window")) {
    SlidingWindow w;
    w.window_size = GetInt(*sw, "window_size", 0);
    w.pad_value = GetInt(*sw, "pad_value", 0);
    w.alignment = GetStr(*sw, "alignment", "right");
    w.slide_key_value_cache = GetBool(*sw, "slide_key_value_cache", true);
    w.slide_inputs = GetBool(*sw, "slide_inputs", true);
    w.cache_slack = GetInt(*sw, "cache_slack", 0);
    if (auto* l = sw->find("layers"))
      for (auto& e : *l->arr) w.layers.push_back(SafeDoubleToInt(e.num, "layers"));
    if (w.alignment != "left" && w.alignment != "right")
      throw std::runtime_error("genai_config: sliding_window.alignment must be \"left\" or \"right\"");
    out.sliding_window = w;
  }
  for (auto& kv : kInputDefaults) out.inputs.emplace_back(kv.first, kv.second);
  for (auto& kv : kOutputDefaults) out.outputs.emplace_back(kv.first, kv.second);
  auto overlay = [](std::vector<std::pair<std::string, std::string>>& dst, const json::Value* src) {
    if (!src) return;
    for (auto& m : *src->obj) {
      auto it = std::find_if(dst.begin(), dst.end(), [&](auto& p) { return p.first == m.first; });
      if (it != dst.end()) it->second = m.second.str;
      else dst.emplace_back(m.first, m.second.str);
    }
  };
  overlay(out.inputs, d.find("inputs"));
  overlay(out.outputs, d.find("outputs"));
  return out;
}

}  // namespace

std::string DecoderConfig::Input(std::string_view nominal) const {
  for (auto& p : inputs) if (p.first == nominal) return p.second;
  return {};
}
std::string DecoderConfig::Output(std::string_view nominal) const {
  for (auto& p : outputs) if (p.first == nominal) return p.second;
  return {};
}

int SafeDoubleToInt(double x, std::string_view name) {
  if (!std::isfinite(x) || x != std::floor(x) || x < -2147483648.0 || x > 2147483647.0) {
    std::ostringstream ss;
    ss << "Field '" << name << "' value " << x << " is not an integer";
    throw std::runtime_error(ss.str());
  }
  return static_cast<int>(x);
}

std::string NormalizeProviderName(std::string_view name) {
  std::string low;
  for (char c : name) low.push_back(char(std::tolower((unsigned char)c)));
  if (low == "cuda" || low == "cudaexecutionprovider") return "cuda";
  if (low == "cpu" || low == "cpuexecutionprovider") return "cpu";
  return std::string(name);
}

bool IsGraphCaptureEnabled(const SessionOptions& so) {
  for (auto& provider : so.providers) {
    for (auto& po : so.provider_options) {
      if (po.name != provider) continue;
      if (po.name == "cuda") {
        for (auto& kv : po.options)
          if (kv.first == "enable_cuda_graph" && kv.second == "1") return true;
        return false;
      }
    }
  }
  return false;
}

void ValidateConfigPath(const std::string& path, std::string_view context) {
  if (path.empty()) return;
  auto err = [&](const std::string& msg) {
    return context.empty() ? msg : std::string(context) + ": " + msg;
  };
  if (path[0] == '/' || path[0] == '\\' ||
      (path.size() >= 2 && std::isalpha((unsigned char)path[0]) && path[1] == ':'))
    throw std::runtime_error(err("Config path must be a relative path under the model directory, got: " + path));
  std::string comp;
  for (size_t i = 0; i <= path.size(); ++i) {
    if (i == path.size() || path[i] == '/' || path[i] == '\\') {
      if (comp == "..") throw std::runtime_error(err("Config path must not contain path traversal (..): " + path));
      comp.clear();
    } else comp.push_back(path[i]);
  }
}

// ------------------------------------------------------------------------------------- setters
void SetSearchNumber(SearchConfig& s, std::string_view name, double v) {
  auto I = [&] { return SafeDoubleToInt(v, name); };
  if (name == "min_length") s.min_length = I();
  else if (name == "max_length") s.max_length = I();
  else if (name == "batch_size") s.batch_size = I();
  else if (name == "num_beams") s.num_beams = I();
  else if (name == "num_return_sequences") s.num_return_sequences = I();
  else if (name == "top_k") s.top_k = I();
  else if (name == "top_p") s.top_p = float(v);
  else if (name == "temperature") s.temperature = float(v);
  else if (name == "repetition_penalty") s.repetition_penalty = float(v);
  else if (name == "length_penalty") s.length_penalty = float(v);
  else if (name == "no_repeat_ngram_size") s.no_repeat_ngram_size = I();
  else if (name == "diversity_penalty") s.diversity_penalty = float(v);
  else if (name == "random_seed") s.random_seed = I();
  else if (name == "blank_penalty") s.blank_penalty = float(v);
  else if (name == "chunk_size") {
    if (v > 0) s.chunk_size = size_t(v); else s.chunk_size.reset();
  } else if (name == "do_sample" || name == "past_present_share_buffer" || name == "early_stopping") {
    throw std::runtime_error("search option '" + std::string(name) + "' expects a bool");
  } else {
    throw std::runtime_error("Unknown search option: \"" + std::string(name) + "\"");
  }
}

void SetSearchBool(SearchConfig& s, std::string_view name, bool v) {
  if (name == "do_sample") s.do_sample = v;
  else if (name == "past_present_share_buffer") s.past_present_share_buffer = v;
  else if (name == "early_stopping") s.early_stopping = v;
  else throw std::runtime_error("Unknown boolean search option: \"" + std::string(name) + "\"");
}

void SetSpeculativeNumber(SpeculativeConfig& s, std::string_view name, double v) {
  constexpr int kMinK = 1, kMaxK = 16;
  int k = SafeDoubleToInt(v, name);
  if (name == "max_draft_tokens") {
    if (k < kMinK || k > kMaxK)
      throw std::runtime_error("speculative.max_draft_tokens must be between 1 and 16. Got: " + std::to_string(k) + ".");
    s.max_draft_tokens = k;
  } else if (name == "ngram_size") {
    if (k != 0 && (k < 2 || k > kMaxK))
      throw std::runtime_error("speculative.ngram_size must be 0 or between 2 and 16. Got: " + std::to_string(k) + ".");
    s.ngram_size = k;
  } else if (name == "min_adaptive_k") {
    if (k < 0 || k > kMaxK)
      throw std::runtime_error("speculative.min_adaptive_k must be 0 or between 1 and 16. Got: " + std::to_string(k) + ".");
    s.min_adaptive_k = k;
  } else {
    throw std::runtime_error("Unknown speculative option: \"" + std::string(name) + "\"");
  }
}

void SetSpeculativeBool(SpeculativeConfig& s, std::string_view name, bool v) {
  if (name == "ngram_chained_lookup") s.ngram_chained_lookup = v;
  else if (name == "cooldown") s.cooldown = v;
  else throw std::runtime_error("Unknown boolean speculative option: \"" + std::string(name) + "\"");
}

// ------------------------------------------------------------------------------------- Config
Config::Config(const std::string& dir, std::string_view overlay) : config_path(dir) {
  std::string file = dir + "/genai_config.json";
  std::ifstream f(file, std::ios::binary);
  if (!f) throw std::runtime_error("Error opening " + file);
  std::stringstream ss;
  ss << f.rdbuf();
  try {
    tree = json::Parse(ss.str());
    if (!overlay.empty()) Merge(tree, json::Parse(overlay));
  } catch (const json::ParseError& e) {
    throw std::runtime_error("Error encountered while parsing '" + file + "': " + e.what());
  }
  Finish();
}

Config Config::FromJson(std::string_view text, std::string_view overlay) {
  Config c;
  c.tree = json::Parse(text);
  if (!overlay.empty()) Merge(c.tree, json::Parse(overlay));
  c.Finish();
  return c;
}

void Config::Overlay(std::string_view text) {
  json::Value next = DeepCopy(tree);
  Merge(next, json::Parse(text));
  Validate(next, Root(), "");
  json::Value saved = tree;
  tree = next;
  try {
    Finish();
  } catch (...) {
    tree = saved;
    Finish();
    throw;
  }
}

std::string Config::ToJson(int indent) const { return json::Dump(tree, indent); }

void Config::Finish() {
  if (!tree.is_object()) throw std::runtime_error("genai_config: document root must be an object");
  Validate(tree, Root(), "");
  Project();
}

void Config::Project() {
  model = ModelConfig{};
  search = SearchConfig{};
  speculative = SpeculativeConfig{};
  engine = EngineConfig{};
  if (auto* m = tree.find("model")) {
    model.type = GetStr(*m, "type");
    model.tokenizer_dir = GetStr(*m, "tokenizer_dir");
    model.pad_token_id = GetInt(*m, "pad_token_id", 0);
    model.bos_token_id = GetInt(*m, "bos_token_id", 0);
    model.vocab_size = GetInt(*m, "vocab_size", 0);
    model.context_length = GetInt(*m, "context_length", 0);
    if (auto* e = m->find("eos_token_id")) {
      if (e->is_number()) model.eos_token_id.push_back(SafeDoubleToInt(e->num, "eos_token_id"));
      else for (auto& x : *e->arr) model.eos_token_id.push_back(SafeDoubleToInt(x.num, "eos_token_id"));
    }
    if (auto* d = m->find("decoder")) model.decoder = ProjectDecoder(*d);
    if (auto* d = m->find("draft")) model.draft = ProjectDecoder(*d);
    for (const char* sub : {"encoder", "embedding", "vision", "speech", "joiner", "vad", "decoder", "draft", "mtp"})
      if (auto* s = m->find(sub)) {
        ValidateConfigPath(GetStr(*s, "filename"), std::string("model.") + sub + ".filename");
        ValidateConfigPath(GetStr(*s, "config_filename"), std::string("model.") + sub + ".config_filename");
        ValidateConfigPath(GetStr(*s, "adapter_filename"), std::string("model.") + sub + ".adapter_filename");
      }
    ValidateConfigPath(model.tokenizer_dir, "model.tokenizer_dir");
  }
  if (auto* s = tree.find("search")) {
    for (auto& kv : *s->obj) {
      if (kv.second.is_bool()) SetSearchBool(search, kv.first, kv.second.b);
      else SetSearchNumber(search, kv.first, kv.second.num);
    }
  }
  if (auto* s = tree.find("speculative")) {
    for (auto& kv : *s->obj) {
      if (kv.second.is_bool()) SetSpeculativeBool(speculative, kv.first, kv.second.b);
      else SetSpeculativeNumber(speculative, kv.first, kv.second.num);
    }
  }
  if (auto* e = tree.find("engine")) {
    // The later of the two sections in document order wins (they are mutually exclusive).
    for (auto& kv : *e->obj) {
      if (kv.first == "dynamic_batching") {
        engine.static_batching.reset();
        DynamicBatching d;
        auto positive = [&](const char* k, size_t dflt) -> size_t {
          auto* p = kv.second.find(k);
          if (!p) return dflt;
          int v = SafeDoubleToInt(p->num, k);
          if (v <= 0) throw std::out_of_range(std::string(k) + " must be > 0");
          return size_t(v);
        };
        d.block_size = positive("block_size", d.block_size);
        if (kv.second.find("num_blocks")) d.num_blocks = positive("num_blocks", 0);
        d.max_batch_size = positive("max_batch_size", d.max_batch_size);
        d.max_scheduled_tokens = positive("max_scheduled_tokens", d.max_scheduled_tokens);
        if (auto* g = kv.second.find("gpu_utilization_factor")) {
          if (!std::isfinite(g->num) || g->num <= 0 || g->num > 1)
            throw std::out_of_range("gpu_utilization_factor must be > 0 and <= 1");
          d.gpu_utilization_factor = float(g->num);
        }
        engine.dynamic_batching = d;
      } else if (kv.first == "static_batching") {
        engine.dynamic_batching.reset();
        StaticBatching sb;
        if (auto* p = kv.second.find("max_batch_size")) sb.max_batch_size = size_t(p->num);
        engine.static_batching = sb;
      }
    }
  }
  if (model.context_length == 0) throw std::runtime_error("model context_length is 0 or was not set. It must be greater than 0");
  if (search.max_length == 0) search.max_length = model.context_length;
  if (model.eos_token_id.empty()) model.eos_token_id.push_back(model.pad_token_id);
}

// ----------------------------------------------------------------------------- provider edits
namespace {
json::Value& EnsureObject(json::Value& parent, const char* key) {
  if (auto* p = parent.find(key)) return *p;
  return parent.set(key, json::Value::MakeObject());
}
json::Value& DecoderProviderArray(json::Value& tree) {
  auto& so = EnsureObject(EnsureObject(EnsureObject(tree, "model"), "decoder"), "session_options");
  if (auto* p = so.find("provider_options")) return *p;
  return so.set("provider_options", json::Value::MakeArray());
}
}  // namespace

void Config::ClearProviders() {
  DecoderProviderArray(tree).arr->clear();
  Project();
}

void Config::AppendProvider(std::string_view name) {
  std::string n = NormalizeProviderName(name);
  auto& arr = DecoderProviderArray(tree);
  for (auto& e : *arr.arr)
    for (auto& prov : *e.obj)
      if (NormalizeProviderName(prov.first) == n) return;
  json::Value entry = json::Value::MakeObject();
  entry.set(n, json::Value::MakeObject());
  arr.arr->push_back(entry);
  Project();
}

void Config::SetProviderOption(std::string_view provider, std::string_view key, std::string_view value) {
  std::string n = NormalizeProviderName(provider);
  AppendProvider(n);
  auto& arr = DecoderProviderArray(tree);
  for (auto& e : *arr.arr)
    for (auto& prov : *e.obj)
      if (NormalizeProviderName(prov.first) == n) prov.second.set(key, json::Value::MakeString(std::string(value)));
  Project();
}

}  // namespace ogb
