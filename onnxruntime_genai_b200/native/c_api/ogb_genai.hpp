// C++ convenience layer over the C API: move-only owners that destroy their handle, and errors as exceptions.
//
// Role of the reference's src/ort_genai.h (zero-cost C++ wrappers over the C API); the shape is different: the owners live in
// namespace ogb and hold the C handle (`get()` hands it to any C function that has no wrapper here), instead of giving the
// opaque C structs C++ member functions.
//
//   ogb::Model model(dir);
//   ogb::Tokenizer tok(model);
//   ogb::GeneratorParams params(model);
//   params.SetSearchOption("max_length", 64);
//   ogb::Generator gen(model, params);
//   gen.AppendTokens(tok.Encode("Hello"));
//   while (!gen.IsDone()) gen.GenerateNextToken();
//   std::string text = tok.Decode(gen.GetSequence(0));
#pragma once

#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "ogb_genai_c.h"

namespace ogb {

inline void Check(OgaResult* r) {
  if (!r) return;
  std::string m = OgaResultGetError(r);
  OgaDestroyResult(r);
  throw std::runtime_error(m);
}

template <class T, void (*Destroy)(T*)>
class Owner {
 public:
  Owner() = default;
  explicit Owner(T* p) : p_(p) {}
  Owner(Owner&& o) noexcept : p_(std::exchange(o.p_, nullptr)) {}
  Owner& operator=(Owner&& o) noexcept {
    if (this != &o) {
      reset();
      p_ = std::exchange(o.p_, nullptr);
    }
    return *this;
  }
  Owner(const Owner&) = delete;
  Owner& operator=(const Owner&) = delete;
  ~Owner() { reset(); }
  void reset() {
    if (p_) Destroy(p_);
    p_ = nullptr;
  }
  T* get() const { return p_; }
  explicit operator bool() const { return p_ != nullptr; }

 protected:
  T* p_ = nullptr;
};

inline std::string TakeString(const char* s) {
  std::string out = s ? s : "";
  OgaDestroyString(s);
  return out;
}

class Config : public Owner<OgaConfig, OgaDestroyConfig> {
 public:
  explicit Config(const std::string& path) { Check(OgaCreateConfig(path.c_str(), &p_)); }
  void ClearProviders() { Check(OgaConfigClearProviders(p_)); }
  void AppendProvider(const std::string& p) { Check(OgaConfigAppendProvider(p_, p.c_str())); }
  void SetProviderOption(const std::string& p, const std::string& k, const std::string& v) { Check(OgaConfigSetProviderOption(p_, p.c_str(), k.c_str(), v.c_str())); }
  void Overlay(const std::string& json) { Check(OgaConfigOverlay(p_, json.c_str())); }
};

class Model : public Owner<OgaModel, OgaDestroyModel> {
 public:
  explicit Model(const std::string& path) { Check(OgaCreateModel(path.c_str(), &p_)); }
  explicit Model(const Config& c) { Check(OgaCreateModelFromConfig(c.get(), &p_)); }
  std::string Type() const {
    const char* s;
    Check(OgaModelGetType(p_, &s));
    return TakeString(s);
  }
  std::string DeviceType() const {
    const char* s;
    Check(OgaModelGetDeviceType(p_, &s));
    return TakeString(s);
  }
};

class Sequences : public Owner<OgaSequences, OgaDestroySequences> {
 public:
  Sequences() { Check(OgaCreateSequences(&p_)); }
  explicit Sequences(const std::vector<int32_t>& tokens) : Sequences() { Append(tokens); }
  void Append(const std::vector<int32_t>& tokens) { Check(OgaAppendTokenSequence(tokens.data(), tokens.size(), p_)); }
  size_t Count() const { return OgaSequencesCount(p_); }
  std::vector<int32_t> Get(size_t i) const {
    const int32_t* d = OgaSequencesGetSequenceData(p_, i);
    return std::vector<int32_t>(d, d + OgaSequencesGetSequenceCount(p_, i));
  }
};

class TokenizerStream : public Owner<OgaTokenizerStream, OgaDestroyTokenizerStream> {
 public:
  using Owner::Owner;
  std::string Decode(int32_t token) {
    const char* s;
    Check(OgaTokenizerStreamDecode(p_, token, &s));
    return s;  // owned by the stream until its next call
  }
};

class Tokenizer : public Owner<OgaTokenizer, OgaDestroyTokenizer> {
 public:
  explicit Tokenizer(const Model& m) { Check(OgaCreateTokenizer(m.get(), &p_)); }
  std::vector<int32_t> Encode(const std::string& text) const {
    Sequences s;
    Check(OgaTokenizerEncode(p_, text.c_str(), s.get()));
    return s.Get(0);
  }
  std::string Decode(const std::vector<int32_t>& tokens) const {
    const char* s;
    Check(OgaTokenizerDecode(p_, tokens.data(), tokens.size(), &s));
    return TakeString(s);
  }
  std::string ApplyChatTemplate(const std::string& messages, const std::string& template_str = "", const std::string& tools = "",
                                bool add_generation_prompt = true) const {
    const char* s;
    Check(OgaTokenizerApplyChatTemplate(p_, template_str.c_str(), messages.c_str(), tools.c_str(), add_generation_prompt, &s));
    return TakeString(s);
  }
  TokenizerStream CreateStream() const {
    OgaTokenizerStream* s;
    Check(OgaCreateTokenizerStream(p_, &s));
    return TokenizerStream(s);
  }
  int32_t BosTokenId() const {
    int32_t id;
    Check(OgaTokenizerGetBosTokenId(p_, &id));
    return id;
  }
  std::vector<int32_t> EosTokenIds() const {
    const int32_t* ids;
    size_t n;
    Check(OgaTokenizerGetEosTokenIds(p_, &ids, &n));
    return std::vector<int32_t>(ids, ids + n);
  }
};

class GeneratorParams : public Owner<OgaGeneratorParams, OgaDestroyGeneratorParams> {
 public:
  explicit GeneratorParams(const Model& m) { Check(OgaCreateGeneratorParams(m.get(), &p_)); }
  void SetSearchOption(const std::string& name, double v) { Check(OgaGeneratorParamsSetSearchNumber(p_, name.c_str(), v)); }
  void SetSearchOptionBool(const std::string& name, bool v) { Check(OgaGeneratorParamsSetSearchBool(p_, name.c_str(), v)); }
  double GetSearchNumber(const std::string& name) const {
    double v;
    Check(OgaGeneratorParamsGetSearchNumber(p_, name.c_str(), &v));
    return v;
  }
  void SetSpeculativeOption(const std::string& name, double v) { Check(OgaGeneratorParamsSetSpeculativeNumber(p_, name.c_str(), v)); }
  void SetGuidance(const std::string& type, const std::string& data, bool enable_ff_tokens = false) {
    Check(OgaGeneratorParamsSetGuidance(p_, type.c_str(), data.c_str(), enable_ff_tokens));
  }
};

class Tensor : public Owner<OgaTensor, OgaDestroyTensor> {
 public:
  using Owner::Owner;
  // `data` stays owned by the caller and must outlive the tensor.
  Tensor(void* data, const std::vector<int64_t>& shape, OgaElementType type) { Check(OgaCreateTensorFromBuffer(data, shape.data(), shape.size(), type, &p_)); }
  OgaElementType Type() const {
    OgaElementType t;
    Check(OgaTensorGetType(p_, &t));
    return t;
  }
  std::vector<int64_t> Shape() const {
    size_t rank;
    Check(OgaTensorGetShapeRank(p_, &rank));
    std::vector<int64_t> s(rank);
    Check(OgaTensorGetShape(p_, s.data(), rank));
    return s;
  }
  void* Data() const {
    void* d;
    Check(OgaTensorGetData(p_, &d));
    return d;
  }
};

class Adapters : public Owner<OgaAdapters, OgaDestroyAdapters> {
 public:
  explicit Adapters(const Model& m) { Check(OgaCreateAdapters(m.get(), &p_)); }
  void Load(const std::string& path, const std::string& name) { Check(OgaLoadAdapter(p_, path.c_str(), name.c_str())); }
  void Unload(const std::string& name) { Check(OgaUnloadAdapter(p_, name.c_str())); }
};

class Generator : public Owner<OgaGenerator, OgaDestroyGenerator> {
 public:
  Generator(const Model& m, const GeneratorParams& p) { Check(OgaCreateGenerator(m.get(), p.get(), &p_)); }
  void AppendTokens(const std::vector<int32_t>& t) { Check(OgaGenerator_AppendTokens(p_, t.data(), t.size())); }
  void AppendTokenSequences(const Sequences& s) { Check(OgaGenerator_AppendTokenSequences(p_, s.get())); }
  bool IsDone() const { return OgaGenerator_IsDone(p_); }
  void GenerateNextToken() { Check(OgaGenerator_GenerateNextToken(p_)); }
  std::vector<int32_t> GetNextTokens() const {
    const int32_t* t;
    size_t n;
    Check(OgaGenerator_GetNextTokens(p_, &t, &n));
    return std::vector<int32_t>(t, t + n);
  }
  std::vector<int32_t> GetSequence(size_t i) const {
    size_t n = OgaGenerator_GetSequenceCount(p_, i);
    const int32_t* d = OgaGenerator_GetSequenceData(p_, i);
    return std::vector<int32_t>(d, d + n);
  }
  size_t TokenCount() const { return OgaGenerator_TokenCount(p_); }
  void RewindTo(size_t length) { Check(OgaGenerator_RewindTo(p_, length)); }
  Tensor GetLogits() {
    OgaTensor* t;
    Check(OgaGenerator_GetLogits(p_, &t));
    return Tensor(t);
  }
  void SetLogits(const Tensor& t) { Check(OgaGenerator_SetLogits(p_, t.get())); }
  Tensor GetOutput(const std::string& name) const {
    OgaTensor* t;
    Check(OgaGenerator_GetOutput(p_, name.c_str(), &t));
    return Tensor(t);
  }
  void SetActiveAdapter(Adapters& a, const std::string& name) { Check(OgaSetActiveAdapter(p_, a.get(), name.c_str())); }
  void SetRuntimeOption(const std::string& k, const std::string& v) { Check(OgaGenerator_SetRuntimeOption(p_, k.c_str(), v.c_str())); }
};

class Request : public Owner<OgaRequest, OgaDestroyRequest> {
 public:
  using Owner::Owner;
  explicit Request(GeneratorParams& p) { Check(OgaCreateRequest(p.get(), &p_)); }
  void AddTokens(const std::vector<int32_t>& t) { Check(OgaRequestAddTokens(p_, Sequences(t).get())); }
  void Continue(const std::vector<int32_t>& t) { Check(OgaRequestContinue(p_, Sequences(t).get())); }
  void Continue(const std::vector<int32_t>& t, size_t max_length) { Check(OgaRequestContinueWithMaxLength(p_, Sequences(t).get(), max_length)); }
  void SetActiveAdapter(OgaAdapters* adapters, const char* name) { Check(OgaRequestSetActiveAdapter(p_, adapters, name)); }
  void SetOpaqueData(void* d) { Check(OgaRequestSetOpaqueData(p_, d)); }
  void* GetOpaqueData() const {
    void* d;
    Check(OgaRequestGetOpaqueData(p_, &d));
    return d;
  }
  bool HasUnseenTokens() const {
    bool b;
    Check(OgaRequestHasUnseenTokens(p_, &b));
    return b;
  }
  int32_t GetUnseenToken() {
    int32_t t;
    Check(OgaRequestGetUnseenToken(p_, &t));
    return t;
  }
  bool IsTurnComplete() const {
    bool b;
    Check(OgaRequestIsTurnComplete(p_, &b));
    return b;
  }
};

class Engine : public Owner<OgaEngine, OgaDestroyEngine> {
 public:
  explicit Engine(Model& m) { Check(OgaCreateEngine(m.get(), &p_)); }
  void Add(Request& r) { Check(OgaEngineAddRequest(p_, r.get())); }
  void Remove(Request& r) { Check(OgaEngineRemoveRequest(p_, r.get())); }
  bool HasPendingRequests() {
    bool b;
    Check(OgaEngineHasPendingRequests(p_, &b));
    return b;
  }
  // A handle on a request that has tokens to read (empty when none is ready); destroying it does not remove the request.
  Request Step() {
    OgaRequest* r = nullptr;
    Check(OgaEngineStep(p_, &r));
    return Request(r);
  }
};

// Calls OgaShutdown when it goes out of scope: declare one first in main() so that it runs after every owner is gone.
struct ShutdownGuard {
  ~ShutdownGuard() { OgaShutdown(); }
};

}  // namespace ogb
