#include "tracing.h"

#include <cstdlib>
#include <stdexcept>
#include <thread>

namespace ogb {

Tracer& Tracer::Get() {
  static Tracer t;
  return t;
}

int64_t Tracer::NowUs() {
  return std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

void Tracer::Enable(const std::string& path) {
  std::lock_guard<std::mutex> lk(mu_);
  if (file_) return;
  std::string p = path;
  if (p.empty()) {
    const char* env = std::getenv("ORTGENAI_TRACE_FILE_PATH");
    p = env && *env ? env : "ortgenai_trace.log";
  }
  file_ = std::fopen(p.c_str(), "w");
  if (!file_) throw std::runtime_error("cannot open trace file " + p);
  std::fputs("[\n", file_);
  first_ = true;
}

void Tracer::Disable() {
  std::lock_guard<std::mutex> lk(mu_);
  if (!file_) return;
  std::fputs("\n]\n", file_);
  std::fclose(file_);
  file_ = nullptr;
}

void Tracer::Complete(const char* category, const std::string& name, int64_t begin_us, int64_t dur_us) {
  std::lock_guard<std::mutex> lk(mu_);
  if (!file_) return;
  std::string safe;
  for (char c : name) safe.push_back(c == '"' || c == '\\' ? '_' : c);
  auto tid = std::hash<std::thread::id>()(std::this_thread::get_id()) % 100000;
  std::fprintf(file_, "%s{\"name\":\"%s\",\"cat\":\"%s\",\"ph\":\"X\",\"ts\":%lld,\"dur\":%lld,\"pid\":1,\"tid\":%llu}",
               first_ ? "" : ",\n", safe.c_str(), category, (long long)begin_us, (long long)dur_us, (unsigned long long)tid);
  first_ = false;
}

Log& Log::Get() {
  static Log l;
  return l;
}

Log::Log() {
  for (const char* n : {"enabled", "ansi_tags", "warning", "generate_next_token", "append_next_tokens", "hit_eos",
                        "hit_max_length", "model_input_values", "model_output_shapes", "model_output_values",
                        "model_logits", "ort_lib", "value_stats"})
    flags_[n] = false;
  flags_["ansi_tags"] = true;
  flags_["warning"] = true;
}

void Log::SetBool(const std::string& name, bool v) {
  std::lock_guard<std::mutex> lk(mu_);
  auto it = flags_.find(name);
  if (it == flags_.end()) throw std::runtime_error("Unknown log option: " + name);
  it->second = v;
}

void Log::SetString(const std::string& name, const std::string& v) {
  std::lock_guard<std::mutex> lk(mu_);
  if (name != "filename") throw std::runtime_error("Unknown log option: " + name);
  if (file_) { std::fclose(file_); file_ = nullptr; }
  if (!v.empty()) {
    file_ = std::fopen(v.c_str(), "w");
    if (!file_) throw std::runtime_error("cannot open log file " + v);
  }
}

bool Log::Flag(const std::string& name) const {
  std::lock_guard<std::mutex> lk(mu_);
  auto it = flags_.find(name);
  return it != flags_.end() && it->second;
}

void Log::SetCallback(std::function<void(const std::string&)> cb) {
  std::lock_guard<std::mutex> lk(mu_);
  cb_ = std::move(cb);
}

void Log::Write(const std::string& label, const std::string& text) {
  std::function<void(const std::string&)> cb;
  std::string line;
  {
    std::lock_guard<std::mutex> lk(mu_);
    if (!flags_["enabled"]) return;
    if (label == "warning" && !flags_["warning"]) return;
    line = flags_["ansi_tags"] && !cb_ && !file_ ? "\x1b[33m" + label + "\x1b[0m " + text : "  " + label + "  " + text;
    cb = cb_;
    if (!cb) {
      std::FILE* out = file_ ? file_ : stderr;
      std::fprintf(out, "%s\n", line.c_str());
      std::fflush(out);
      return;
    }
  }
  cb(line);
}

}  // namespace ogb
