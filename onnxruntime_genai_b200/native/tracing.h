// Chrome trace-event sink and log-flag table.
//
// Tracing: scopes write "X" (complete) events to a JSON array file that chrome://tracing and
// Perfetto load; the file path comes from ORTGENAI_TRACE_FILE_PATH (default ortgenai_trace.log),
// the same contract as the reference (src/tracing.h, src/tracing.cpp).  The reference compiles
// tracing in only with ENABLE_TRACING; here it is always compiled and switched on at run time.
//
// Logging: a table of named boolean flags plus a sink (stderr or a callback), mirroring
// src/logging.h:33-50.
#pragma once
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <functional>
#include <map>
#include <mutex>
#include <string>

namespace ogb {

class Tracer {
 public:
  static Tracer& Get();
  void Enable(const std::string& path);  // empty path -> env var / default name
  void Disable();                        // closes the JSON array
  bool Enabled() const { return file_ != nullptr; }
  void Complete(const char* category, const std::string& name, int64_t begin_us, int64_t dur_us);
  static int64_t NowUs();

 private:
  std::mutex mu_;
  std::FILE* file_{nullptr};
  bool first_{true};
};

struct TraceScope {
  TraceScope(const char* category, std::string name)
      : cat_(category), name_(std::move(name)), t0_(Tracer::Get().Enabled() ? Tracer::NowUs() : -1) {}
  ~TraceScope() {
    if (t0_ >= 0) Tracer::Get().Complete(cat_, name_, t0_, Tracer::NowUs() - t0_);
  }
  const char* cat_;
  std::string name_;
  int64_t t0_;
};

class Log {
 public:
  static Log& Get();
  // Known flags: enabled, ansi_tags, warning, generate_next_token, append_next_tokens, hit_eos,
  // hit_max_length, model_input_values, model_output_shapes, model_output_values, model_logits,
  // ort_lib, value_stats.  Unknown names throw.
  void SetBool(const std::string& name, bool v);
  void SetString(const std::string& name, const std::string& v);  // "filename"
  bool Flag(const std::string& name) const;
  void SetCallback(std::function<void(const std::string&)> cb);
  void Write(const std::string& label, const std::string& text);

 private:
  Log();
  mutable std::mutex mu_;
  std::map<std::string, bool> flags_;
  std::function<void(const std::string&)> cb_;
  std::FILE* file_{nullptr};
};

}  // namespace ogb
