// C API of onnxruntime_genai_b200 (see ogb_genai_c.h): opaque handles over the Python-level runtime objects.
//
// Behavioural model: the reference's C API (src/ort_genai_c.cpp:60-1250): every entry point catches all errors and
// returns them as an OgaResult; handles are counted per type and OgaShutdown prints the ones that were never destroyed
// (src/generators.cpp:83-199 LeakChecked / Shutdown).  The objects behind the handles are the package's Python classes; the
// interpreter is started here when the host program has none (its prefix is taken from the python executable named by
// OGB_PYTHON, else the first `python3` on PATH, so a virtual environment's packages are found), and joined through the GIL
// when the library is loaded into a Python process.
#include "ogb_genai_c.h"

#include <dlfcn.h>
#include <pybind11/embed.h>
#include <pybind11/numpy.h>
#include <pybind11/stl.h>
#include <unistd.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

namespace py = pybind11;

// ------------------------------------------------------------------------------------------------ handle bookkeeping
namespace {

std::mutex g_count_mu;
std::map<std::string, long>& Counts() {
  static auto* m = new std::map<std::string, long>();  // never destroyed: handles may be released during process exit
  return *m;
}
void Count(const char* kind, long d) {
  std::lock_guard<std::mutex> lk(g_count_mu);
  Counts()[kind] += d;
}

struct Handle {
  const char* kind;
  explicit Handle(const char* k) : kind(k) { Count(k, +1); }
  virtual ~Handle() { Count(kind, -1); }
  Handle(const Handle&) = delete;
  Handle& operator=(const Handle&) = delete;
};

}  // namespace

struct OgaResult { std::string msg; };
#define OGB_HANDLE(Name)                      \
  struct Name : Handle {                      \
    Name() : Handle(#Name) {}                 \
    py::object obj;
#define OGB_END };

OGB_HANDLE(OgaConfig) OGB_END
OGB_HANDLE(OgaModel) OGB_END
OGB_HANDLE(OgaGeneratorParams) OGB_END
OGB_HANDLE(OgaGenerator)
  std::vector<int32_t> next;
  std::map<size_t, std::vector<int32_t>> seqs;
OGB_END
OGB_HANDLE(OgaMtpGenerator)
  std::vector<int32_t> seq;
OGB_END
OGB_HANDLE(OgaSpeculativeStats) OGB_END
OGB_HANDLE(OgaTokenizer)
  std::vector<int32_t> eos;
OGB_END
OGB_HANDLE(OgaTokenizerStream)
  std::string last;
OGB_END
OGB_HANDLE(OgaTensor)  // obj: a numpy array (C-contiguous); bf16 data is held as uint16 with the tag below
  OgaElementType type = OgaElementType_undefined;
OGB_END
OGB_HANDLE(OgaNamedTensors) OGB_END  // obj: the package's NamedTensors (a dict name -> array)
OGB_HANDLE(OgaImages) OGB_END
OGB_HANDLE(OgaAudios) OGB_END
OGB_HANDLE(OgaMultiModalProcessor) OGB_END
OGB_HANDLE(OgaStreamingProcessor)
  std::string option;   // the string the last GetOption returned
OGB_END
OGB_HANDLE(OgaAdapters) OGB_END
OGB_HANDLE(OgaEngine) OGB_END
OGB_HANDLE(OgaRequest) OGB_END

struct OgaSequences : Handle {
  OgaSequences() : Handle("OgaSequences") {}
  std::vector<std::vector<int32_t>> rows;
};
struct OgaStringArray : Handle {
  OgaStringArray() : Handle("OgaStringArray") {}
  std::vector<std::string> strs;
};

// ------------------------------------------------------------------------------------------------ interpreter
namespace {

std::mutex g_init_mu;
bool g_ready = false;
bool g_owns_interpreter = false;
PyObject* g_og = nullptr;  // the package module (strong reference, dropped by OgaShutdown)
void (*g_log_cb)(const char*, size_t) = nullptr;

std::string FindPython() {
  if (const char* e = getenv("OGB_PYTHON")) return e;
  const char* path = getenv("PATH");
  std::string p = path ? path : "";
  size_t b = 0;
  while (b <= p.size()) {
    size_t e = p.find(':', b);
    if (e == std::string::npos) e = p.size();
    std::string cand = p.substr(b, e - b) + "/python3";
    if (access(cand.c_str(), X_OK) == 0) return cand;
    b = e + 1;
  }
  return "python3";
}

// Directory that holds the package: this library lives in <root>/onnxruntime_genai_b200/native/c_api/.
std::string PackageParent() {
  Dl_info info;
  if (!dladdr(reinterpret_cast<void*>(&FindPython), &info) || !info.dli_fname) return "";
  std::string s = info.dli_fname;
  for (int i = 0; i < 4; ++i) {
    size_t k = s.rfind('/');
    if (k == std::string::npos) return "";
    s.resize(k);
  }
  return s;
}

struct Gil {
  PyGILState_STATE st;
  Gil() : st(PyGILState_Ensure()) {}
  ~Gil() { PyGILState_Release(st); }
};

void EnsurePython() {
  std::lock_guard<std::mutex> lk(g_init_mu);
  if (g_ready) return;
  if (!Py_IsInitialized()) {
    PyConfig config;
    PyConfig_InitPythonConfig(&config);
    std::string exe = FindPython();
    PyStatus st = PyConfig_SetBytesString(&config, &config.program_name, exe.c_str());
    if (!PyStatus_Exception(st)) st = Py_InitializeFromConfig(&config);
    PyConfig_Clear(&config);
    if (PyStatus_Exception(st)) throw std::runtime_error(std::string("cannot start the Python interpreter: ") + (st.err_msg ? st.err_msg : "?"));
    g_owns_interpreter = true;
    PyEval_SaveThread();  // every entry point takes the GIL itself
  }
  Gil g;
  std::string root = PackageParent();
  if (!root.empty()) {
    py::list path = py::module_::import("sys").attr("path");
    bool have = false;
    for (auto h : path)
      if (py::isinstance<py::str>(h) && h.cast<std::string>() == root) have = true;
    if (!have) path.insert(0, root);
  }
  py::object og = py::module_::import("onnxruntime_genai_b200");
  g_og = og.release().ptr();
  g_ready = true;
}

py::object Og() {
  return py::reinterpret_borrow<py::object>(g_og);
}
py::module_ Np() { return py::module_::import("numpy"); }

char* DupString(const std::string& s) {
  char* p = static_cast<char*>(malloc(s.size() + 1));
  memcpy(p, s.c_str(), s.size() + 1);
  return p;
}

// Runs `fn` with the interpreter up and the GIL held; any failure becomes an OgaResult.
template <class F>
OgaResult* Guard(F&& fn) {
  try {
    EnsurePython();
    Gil g;
    try {
      fn();
    } catch (py::error_already_set& e) {
      std::string m;
      try {
        m = py::str(e.value()).cast<std::string>();  // the exception's message, without the traceback
      } catch (...) {
        m = e.what();
      }
      return new OgaResult{m};
    }
    return nullptr;
  } catch (const std::exception& e) {
    return new OgaResult{e.what()};
  } catch (...) {
    return new OgaResult{"unknown error"};
  }
}

// For the few calls of the C API that return a value instead of an OgaResult.
template <class T, class F>
T Value(T fallback, F&& fn) {
  T out = fallback;
  OgaResult* r = Guard([&] { out = fn(); });
  if (r) {
    fprintf(stderr, "onnxruntime_genai_b200: %s\n", r->msg.c_str());
    delete r;
  }
  return out;
}

template <class H>
void Destroy(H* h) {
  if (!h) return;
  if (!Py_IsInitialized()) {  // no interpreter (never started, or the host program finalised its own): only the C++ part can go
    h->obj.release();
    delete h;
    return;
  }
  Gil g;
  delete h;
}

struct DType { OgaElementType t; const char* np; size_t size; };
const DType kTypes[] = {
    {OgaElementType_float32, "float32", 4}, {OgaElementType_uint8, "uint8", 1},   {OgaElementType_int8, "int8", 1},
    {OgaElementType_uint16, "uint16", 2},   {OgaElementType_int16, "int16", 2},   {OgaElementType_int32, "int32", 4},
    {OgaElementType_int64, "int64", 8},     {OgaElementType_bool, "bool", 1},     {OgaElementType_float16, "float16", 2},
    {OgaElementType_float64, "float64", 8}, {OgaElementType_uint32, "uint32", 4}, {OgaElementType_uint64, "uint64", 8},
    {OgaElementType_bfloat16, "uint16", 2},
};
const DType& TypeOf(OgaElementType t) {
  for (auto& d : kTypes)
    if (d.t == t) return d;
  throw std::runtime_error("unsupported tensor element type");
}
OgaElementType TypeFromNumpy(const py::array& a) {
  std::string n = py::str(a.dtype().attr("name")).cast<std::string>();
  for (auto& d : kTypes)
    if (n == d.np) return d.t;
  throw std::runtime_error("unsupported array dtype: " + n);
}

// A numpy array (C order) from whatever the Python API handed back: ndarray, torch tensor, the package's Tensor.
py::array ToArray(py::handle v) {
  py::object o = py::reinterpret_borrow<py::object>(v);
  if (py::hasattr(o, "as_numpy")) o = o.attr("as_numpy")();
  else if (py::hasattr(o, "detach")) o = o.attr("detach")().attr("cpu")().attr("numpy")();
  return Np().attr("ascontiguousarray")(o).cast<py::array>();
}
OgaTensor* WrapArray(py::handle v) {
  auto t = std::make_unique<OgaTensor>();
  py::array a = ToArray(v);
  t->type = TypeFromNumpy(a);
  t->obj = a;
  return t.release();
}
py::array TokensArray(const int32_t* p, size_t n) {
  py::array_t<int32_t> a(static_cast<py::ssize_t>(n));
  if (n) memcpy(a.mutable_data(), p, n * sizeof(int32_t));
  return std::move(a);
}
void CopyTokens(py::handle v, std::vector<int32_t>& out) {
  py::array_t<int32_t, py::array::c_style | py::array::forcecast> a = Np().attr("asarray")(v, "int32").attr("reshape")(-1);
  out.assign(a.data(), a.data() + a.size());
}
py::dict OneKw(const char* name, py::object v) {
  py::dict d;
  d[name] = v;
  return d;
}
py::object NumberArg(double v) {  // whole numbers travel as ints (max_length, top_k ...), the rest as floats
  if (v == static_cast<double>(static_cast<long long>(v))) return py::int_(static_cast<long long>(v));
  return py::float_(v);
}

}  // namespace

extern "C" {

// ------------------------------------------------------------------------------------------------ lifetime / errors / logging
size_t OgaLiveHandleCount(void) {
  std::lock_guard<std::mutex> lk(g_count_mu);
  long n = 0;
  for (auto& kv : Counts()) n += kv.second;
  return static_cast<size_t>(n > 0 ? n : 0);
}

void OgaShutdown(void) {
  {
    std::lock_guard<std::mutex> lk(g_count_mu);
    bool any = false;
    for (auto& kv : Counts())
      if (kv.second > 0) {
        if (!any) fprintf(stderr, "OGA Error: Shutdown must be called after all other objects are destroyed. Still alive:\n");
        any = true;
        fprintf(stderr, "  %s: %ld\n", kv.first.c_str(), kv.second);
      }
  }
  std::lock_guard<std::mutex> lk(g_init_mu);
  if (!g_ready || !Py_IsInitialized()) return;
  {
    Gil g;
    try {
      py::object og = Og();
      if (g_log_cb) og.attr("set_log_callback")(py::none());
      g_log_cb = nullptr;
      py::module_::import("gc").attr("collect")();
      py::object torch = py::module_::import("sys").attr("modules").attr("get")("torch");
      if (!torch.is_none() && torch.attr("cuda").attr("is_available")().cast<bool>()) {
        torch.attr("cuda").attr("synchronize")();
        torch.attr("cuda").attr("empty_cache")();
      }
    } catch (py::error_already_set& e) {
      fprintf(stderr, "onnxruntime_genai_b200: shutdown: %s\n", e.what());
    }
    Py_CLEAR(g_og);
  }
  // The hosted interpreter stays up: extension modules such as torch cannot be initialised twice in one process.  With the
  // package reference dropped and the caches released, the next API call re-imports and works as after a fresh start.
  g_ready = false;
}

const char* OgaResultGetError(const OgaResult* r) { return r ? r->msg.c_str() : ""; }
void OgaDestroyResult(OgaResult* r) { delete r; }
void OgaDestroyString(const char* s) { free(const_cast<char*>(s)); }

OgaResult* OgaSetLogBool(const char* name, bool value) {
  return Guard([&] { Og().attr("set_log_options")(**OneKw(name, py::bool_(value))); });
}
OgaResult* OgaSetLogString(const char* name, const char* value) {
  return Guard([&] { Og().attr("set_log_options")(**OneKw(name, py::str(value ? value : ""))); });
}
OgaResult* OgaSetLogCallback(void (*callback)(const char*, size_t)) {
  return Guard([&] {
    g_log_cb = callback;
    if (!callback) {
      Og().attr("set_log_callback")(py::none());
      return;
    }
    Og().attr("set_log_callback")(py::cpp_function([](const std::string& s) {
      if (g_log_cb) g_log_cb(s.c_str(), s.size());
    }));
  });
}
void OgaSetTelemetryEnabled(bool) {}  // this runtime collects no telemetry
OgaResult* OgaSetCurrentGpuDeviceId(int id) {
  return Guard([&] { Og().attr("set_current_gpu_device_id")(id); });
}
OgaResult* OgaGetCurrentGpuDeviceId(int* id) {
  return Guard([&] { *id = Og().attr("get_current_gpu_device_id")().cast<int>(); });
}

// ------------------------------------------------------------------------------------------------ sequences / strings
OgaResult* OgaCreateSequences(OgaSequences** out) {
  *out = new OgaSequences();
  return nullptr;
}
void OgaDestroySequences(OgaSequences* s) { delete s; }
size_t OgaSequencesCount(const OgaSequences* s) { return s->rows.size(); }
OgaResult* OgaAppendTokenSequence(const int32_t* p, size_t n, OgaSequences* s) {
  s->rows.emplace_back(p, p + n);
  return nullptr;
}
OgaResult* OgaAppendTokenToSequence(int32_t token, OgaSequences* s, size_t index) {
  if (index > s->rows.size()) return new OgaResult{"sequence index out of bounds"};
  if (index == s->rows.size()) s->rows.emplace_back();
  s->rows[index].push_back(token);
  return nullptr;
}
size_t OgaSequencesGetSequenceCount(const OgaSequences* s, size_t i) { return i < s->rows.size() ? s->rows[i].size() : 0; }
const int32_t* OgaSequencesGetSequenceData(const OgaSequences* s, size_t i) { return i < s->rows.size() ? s->rows[i].data() : nullptr; }

OgaResult* OgaCreateStringArray(OgaStringArray** out) {
  *out = new OgaStringArray();
  return nullptr;
}
OgaResult* OgaCreateStringArrayFromStrings(const char* const* strs, size_t count, OgaStringArray** out) {
  auto a = new OgaStringArray();
  for (size_t i = 0; i < count; ++i) a->strs.emplace_back(strs[i]);
  *out = a;
  return nullptr;
}
void OgaDestroyStringArray(OgaStringArray* a) { delete a; }
OgaResult* OgaStringArrayAddString(OgaStringArray* a, const char* s) {
  a->strs.emplace_back(s);
  return nullptr;
}
OgaResult* OgaStringArrayGetCount(const OgaStringArray* a, size_t* out) {
  *out = a->strs.size();
  return nullptr;
}
OgaResult* OgaStringArrayGetString(const OgaStringArray* a, size_t i, const char** out) {
  if (i >= a->strs.size()) return new OgaResult{"string index out of bounds"};
  *out = a->strs[i].c_str();
  return nullptr;
}

// ------------------------------------------------------------------------------------------------ tensors
OgaResult* OgaCreateTensorFromBuffer(void* data, const int64_t* dims, size_t rank, OgaElementType type, OgaTensor** out) {
  return Guard([&] {
    const DType& d = TypeOf(type);
    std::vector<py::ssize_t> shape(dims, dims + rank);
    auto t = std::make_unique<OgaTensor>();
    t->type = type;
    if (data) {
      // the caller's memory, not copied: it must outlive the tensor (same rule as the reference)
      t->obj = py::array(py::dtype(d.np), shape, data, py::capsule(data, [](void*) {}));
    } else {
      t->obj = Np().attr("zeros")(shape, d.np);
    }
    *out = t.release();
  });
}
void OgaDestroyTensor(OgaTensor* t) { Destroy(t); }
OgaResult* OgaTensorGetType(OgaTensor* t, OgaElementType* out) {
  *out = t->type;
  return nullptr;
}
OgaResult* OgaTensorGetShapeRank(OgaTensor* t, size_t* out) {
  return Guard([&] { *out = static_cast<size_t>(t->obj.cast<py::array>().ndim()); });
}
OgaResult* OgaTensorGetShape(OgaTensor* t, int64_t* dims, size_t rank) {
  return Guard([&] {
    py::array a = t->obj.cast<py::array>();
    if (rank != static_cast<size_t>(a.ndim())) throw std::runtime_error("shape_dims_count doesn't match result of OgaTensorGetShapeRank");
    for (size_t i = 0; i < rank; ++i) dims[i] = a.shape(i);
  });
}
OgaResult* OgaTensorGetData(OgaTensor* t, void** out) {
  return Guard([&] { *out = t->obj.cast<py::array>().mutable_data(); });
}

OgaResult* OgaCreateNamedTensors(OgaNamedTensors** out) {
  return Guard([&] {
    auto n = std::make_unique<OgaNamedTensors>();
    n->obj = Og().attr("NamedTensors")();
    *out = n.release();
  });
}
void OgaDestroyNamedTensors(OgaNamedTensors* n) { Destroy(n); }
OgaResult* OgaNamedTensorsGet(OgaNamedTensors* n, const char* name, OgaTensor** out) {
  return Guard([&] {
    py::dict d = n->obj;
    if (!d.contains(name)) throw std::runtime_error(std::string("no tensor named ") + name);
    *out = WrapArray(d[name]);
  });
}
OgaResult* OgaNamedTensorsSet(OgaNamedTensors* n, const char* name, OgaTensor* t) {
  return Guard([&] { n->obj[py::str(name)] = t->obj; });
}
OgaResult* OgaNamedTensorsDelete(OgaNamedTensors* n, const char* name) {
  return Guard([&] { n->obj.attr("pop")(name, py::none()); });
}
OgaResult* OgaNamedTensorsCount(const OgaNamedTensors* n, size_t* out) {
  return Guard([&] { *out = py::len(n->obj); });
}
OgaResult* OgaNamedTensorsGetNames(const OgaNamedTensors* n, OgaStringArray** out) {
  return Guard([&] {
    auto a = std::make_unique<OgaStringArray>();
    for (auto k : py::dict(n->obj)) a->strs.push_back(py::str(k.first).cast<std::string>());
    *out = a.release();
  });
}

// ------------------------------------------------------------------------------------------------ config / model
OgaResult* OgaCreateConfig(const char* path, OgaConfig** out) {
  return Guard([&] {
    auto c = std::make_unique<OgaConfig>();
    c->obj = Og().attr("Config")(path);
    *out = c.release();
  });
}
OgaResult* OgaCreateConfigFromPackageEp(const char* path, const char* ep, OgaConfig** out) {
  return Guard([&] {
    auto c = std::make_unique<OgaConfig>();
    c->obj = Og().attr("Config")(path, "", ep ? py::object(py::str(ep)) : py::object(py::none()));
    *out = c.release();
  });
}
void OgaDestroyConfig(OgaConfig* c) { Destroy(c); }
OgaResult* OgaConfigClearProviders(OgaConfig* c) {
  return Guard([&] { c->obj.attr("clear_providers")(); });
}
OgaResult* OgaConfigAppendProvider(OgaConfig* c, const char* p) {
  return Guard([&] { c->obj.attr("append_provider")(p); });
}
OgaResult* OgaConfigSetProviderOption(OgaConfig* c, const char* p, const char* k, const char* v) {
  return Guard([&] { c->obj.attr("set_provider_option")(p, k, v); });
}
OgaResult* OgaConfigAddModelData(OgaConfig* c, const char* name, const void* data, size_t len) {
  return Guard([&] { c->obj.attr("add_model_data")(name, py::bytes(static_cast<const char*>(data), len)); });
}
OgaResult* OgaConfigRemoveModelData(OgaConfig* c, const char* name) {
  return Guard([&] { c->obj.attr("remove_model_data")(name); });
}
OgaResult* OgaConfigOverlay(OgaConfig* c, const char* json) {
  return Guard([&] { c->obj.attr("overlay")(json); });
}
OgaResult* OgaCreateModel(const char* path, OgaModel** out) {
  return Guard([&] {
    auto m = std::make_unique<OgaModel>();
    m->obj = Og().attr("Model")(path);
    *out = m.release();
  });
}
OgaResult* OgaCreateModelFromConfig(const OgaConfig* c, OgaModel** out) {
  return Guard([&] {
    auto m = std::make_unique<OgaModel>();
    m->obj = Og().attr("Model")(c->obj);
    *out = m.release();
  });
}
void OgaDestroyModel(OgaModel* m) { Destroy(m); }
OgaResult* OgaModelGetType(const OgaModel* m, const char** out) {
  return Guard([&] { *out = DupString(py::str(m->obj.attr("type")).cast<std::string>()); });
}
OgaResult* OgaModelGetDeviceType(const OgaModel* m, const char** out) {
  return Guard([&] { *out = DupString(py::str(m->obj.attr("device_type")).cast<std::string>()); });
}

// ------------------------------------------------------------------------------------------------ generator params
OgaResult* OgaCreateGeneratorParams(const OgaModel* m, OgaGeneratorParams** out) {
  return Guard([&] {
    auto p = std::make_unique<OgaGeneratorParams>();
    p->obj = Og().attr("GeneratorParams")(m->obj);
    *out = p.release();
  });
}
void OgaDestroyGeneratorParams(OgaGeneratorParams* p) { Destroy(p); }
OgaResult* OgaGeneratorParamsSetSearchNumber(OgaGeneratorParams* p, const char* name, double v) {
  return Guard([&] { p->obj.attr("set_search_options")(**OneKw(name, NumberArg(v))); });
}
OgaResult* OgaGeneratorParamsSetSearchBool(OgaGeneratorParams* p, const char* name, bool v) {
  return Guard([&] { p->obj.attr("set_search_options")(**OneKw(name, py::bool_(v))); });
}
static py::object Option(const py::object& params, const char* getter, const char* name) {
  py::dict d = params.attr(getter)();
  if (!d.contains(name)) throw std::runtime_error(std::string("Unknown option: ") + name);
  return d[name];
}
OgaResult* OgaGeneratorParamsGetSearchNumber(const OgaGeneratorParams* p, const char* name, double* v) {
  return Guard([&] { *v = Option(p->obj, "get_search_options", name).cast<double>(); });
}
OgaResult* OgaGeneratorParamsGetSearchBool(const OgaGeneratorParams* p, const char* name, bool* v) {
  return Guard([&] { *v = py::bool_(Option(p->obj, "get_search_options", name)); });
}
OgaResult* OgaGeneratorParamsSetSpeculativeNumber(OgaGeneratorParams* p, const char* name, double v) {
  return Guard([&] { p->obj.attr("set_speculative_options")(**OneKw(name, NumberArg(v))); });
}
OgaResult* OgaGeneratorParamsGetSpeculativeNumber(const OgaGeneratorParams* p, const char* name, double* v) {
  return Guard([&] { *v = Option(p->obj, "get_speculative_options", name).cast<double>(); });
}
OgaResult* OgaGeneratorParamsSetSpeculativeBool(OgaGeneratorParams* p, const char* name, bool v) {
  return Guard([&] { p->obj.attr("set_speculative_options")(**OneKw(name, py::bool_(v))); });
}
OgaResult* OgaGeneratorParamsGetSpeculativeBool(const OgaGeneratorParams* p, const char* name, bool* v) {
  return Guard([&] { *v = py::bool_(Option(p->obj, "get_speculative_options", name)); });
}
OgaResult* OgaGeneratorParamsSetGuidance(OgaGeneratorParams* p, const char* type, const char* data, bool ff) {
  return Guard([&] { p->obj.attr("set_guidance")(type, data, ff); });
}

// ------------------------------------------------------------------------------------------------ generator
OgaResult* OgaCreateGenerator(const OgaModel* m, const OgaGeneratorParams* p, OgaGenerator** out) {
  return Guard([&] {
    auto g = std::make_unique<OgaGenerator>();
    g->obj = Og().attr("Generator")(m->obj, p->obj);
    *out = g.release();
  });
}
void OgaDestroyGenerator(OgaGenerator* g) { Destroy(g); }
bool OgaGenerator_IsDone(OgaGenerator* g) {
  return Value<bool>(true, [&] { return g->obj.attr("is_done")().cast<bool>(); });
}
bool OgaGenerator_IsSessionTerminated(const OgaGenerator* g) {
  return Value<bool>(false, [&] { return py::bool_(py::getattr(g->obj, "_terminated", py::bool_(false))).cast<bool>(); });
}
OgaResult* OgaGenerator_SetModelInput(OgaGenerator* g, const char* name, OgaTensor* t) {
  return Guard([&] { g->obj.attr("set_model_input")(name, t->obj); });
}
OgaResult* OgaGenerator_SetInputs(OgaGenerator* g, const OgaNamedTensors* n) {
  return Guard([&] { g->obj.attr("set_inputs")(n->obj); });
}
OgaResult* OgaGenerator_AppendTokenSequences(OgaGenerator* g, const OgaSequences* s) {
  return Guard([&] {
    if (s->rows.empty()) throw std::runtime_error("input sequences are empty");
    py::list rows;
    for (auto& r : s->rows) rows.append(TokensArray(r.data(), r.size()));
    g->obj.attr("append_tokens")(s->rows.size() == 1 ? py::object(rows[0]) : py::object(rows));
  });
}
OgaResult* OgaGenerator_AppendTokens(OgaGenerator* g, const int32_t* ids, size_t n) {
  return Guard([&] { g->obj.attr("append_tokens")(TokensArray(ids, n)); });
}
size_t OgaGenerator_TokenCount(const OgaGenerator* g) {
  return Value<size_t>(0, [&] { return g->obj.attr("token_count")().cast<size_t>(); });
}
OgaResult* OgaGenerator_GenerateNextToken(OgaGenerator* g) {
  return Guard([&] { g->obj.attr("generate_next_token")(); });
}
OgaResult* OgaGenerator_GetNextTokens(const OgaGenerator* g, const int32_t** out, size_t* count) {
  return Guard([&] {
    auto* gg = const_cast<OgaGenerator*>(g);
    CopyTokens(g->obj.attr("get_next_tokens")(), gg->next);
    *out = gg->next.data();
    *count = gg->next.size();
  });
}
OgaResult* OgaGenerator_SetRuntimeOption(OgaGenerator* g, const char* k, const char* v) {
  return Guard([&] { g->obj.attr("set_runtime_option")(k, v); });
}
OgaResult* OgaGenerator_RewindTo(OgaGenerator* g, size_t len) {
  return Guard([&] { g->obj.attr("rewind_to")(len); });
}
OgaResult* OgaGenerator_SnapshotState(OgaGenerator* g) {
  return Guard([&] { g->obj.attr("snapshot_state")(); });
}
OgaResult* OgaGenerator_SetHiddenStates(OgaGenerator* g, OgaTensor* t) {
  return Guard([&] { g->obj.attr("set_hidden_states")(t->obj); });
}
OgaResult* OgaGenerator_GetInput(const OgaGenerator* g, const char* name, OgaTensor** out) {
  return Guard([&] { *out = WrapArray(g->obj.attr("get_input")(name)); });
}
OgaResult* OgaGenerator_GetOutput(const OgaGenerator* g, const char* name, OgaTensor** out) {
  return Guard([&] { *out = WrapArray(g->obj.attr("get_output")(name)); });
}
OgaResult* OgaGenerator_GetLogits(OgaGenerator* g, OgaTensor** out) {
  return Guard([&] { *out = WrapArray(g->obj.attr("get_logits")()); });
}
OgaResult* OgaGenerator_SetLogits(OgaGenerator* g, OgaTensor* t) {
  return Guard([&] { g->obj.attr("set_logits")(t->obj); });
}
static const std::vector<int32_t>& Sequence(const OgaGenerator* g, size_t i) {
  auto* gg = const_cast<OgaGenerator*>(g);
  CopyTokens(g->obj.attr("get_sequence")(i), gg->seqs[i]);
  return gg->seqs[i];
}
size_t OgaGenerator_GetSequenceCount(const OgaGenerator* g, size_t i) {
  return Value<size_t>(0, [&] { return Sequence(g, i).size(); });
}
const int32_t* OgaGenerator_GetSequenceData(const OgaGenerator* g, size_t i) {
  return Value<const int32_t*>(nullptr, [&] { return Sequence(g, i).data(); });
}
OgaResult* OgaGenerator_GetSpeculativeStats(const OgaGenerator* g, OgaSpeculativeStats** out) {
  return Guard([&] {
    auto s = std::make_unique<OgaSpeculativeStats>();
    s->obj = g->obj.attr("get_speculative_stats")();
    *out = s.release();
  });
}
void OgaDestroySpeculativeStats(OgaSpeculativeStats* s) { Destroy(s); }
static py::object Stat(const OgaSpeculativeStats* s, const char* name) {
  py::dict d = s->obj;
  if (!d.contains(name)) throw std::runtime_error(std::string("unknown speculative statistic: ") + name);
  return d[name];
}
OgaResult* OgaSpeculativeStatsGetCount(const OgaSpeculativeStats* s, const char* name, size_t* out) {
  return Guard([&] { *out = Stat(s, name).cast<size_t>(); });
}
OgaResult* OgaSpeculativeStatsGetNumber(const OgaSpeculativeStats* s, const char* name, double* out) {
  return Guard([&] { *out = Stat(s, name).cast<double>(); });
}
OgaResult* OgaSpeculativeStatsGetBool(const OgaSpeculativeStats* s, const char* name, bool* out) {
  return Guard([&] { *out = py::bool_(Stat(s, name)); });
}

// ------------------------------------------------------------------------------------------------ MTP generator
OgaResult* OgaCreateMtpGeneratorFromHeadDir(const OgaModel* m, const char* head_dir, const OgaGeneratorParams* p, OgaMtpGenerator** out) {
  return Guard([&] {
    auto g = std::make_unique<OgaMtpGenerator>();
    g->obj = Og().attr("MtpGenerator")(m->obj, head_dir, p->obj);
    *out = g.release();
  });
}
OgaResult* OgaMtpGenerator_AppendTokens(OgaMtpGenerator* g, const int32_t* ids, size_t n) {
  return Guard([&] { g->obj.attr("append_tokens")(TokensArray(ids, n)); });
}
OgaResult* OgaMtpGenerator_GenerateNextToken(OgaMtpGenerator* g) {
  return Guard([&] { g->obj.attr("generate_next_token")(); });
}
bool OgaMtpGenerator_IsDone(const OgaMtpGenerator* g) {
  return Value<bool>(true, [&] { return g->obj.attr("is_done")().cast<bool>(); });
}
static const std::vector<int32_t>& MtpSequence(const OgaMtpGenerator* g) {
  auto* gg = const_cast<OgaMtpGenerator*>(g);
  CopyTokens(g->obj.attr("get_sequence")(0), gg->seq);
  return gg->seq;
}
size_t OgaMtpGenerator_GetSequenceCount(const OgaMtpGenerator* g) {
  return Value<size_t>(0, [&] { return MtpSequence(g).size(); });
}
const int32_t* OgaMtpGenerator_GetSequenceData(const OgaMtpGenerator* g) {
  return Value<const int32_t*>(nullptr, [&] { return MtpSequence(g).data(); });
}
OgaResult* OgaMtpGenerator_GetSpeculativeStats(const OgaMtpGenerator* g, OgaSpeculativeStats** out) {
  return Guard([&] {
    auto s = std::make_unique<OgaSpeculativeStats>();
    s->obj = g->obj.attr("get_speculative_stats")();
    *out = s.release();
  });
}
void OgaDestroyMtpGenerator(OgaMtpGenerator* g) { Destroy(g); }

// ------------------------------------------------------------------------------------------------ tokenizer
OgaResult* OgaCreateTokenizer(const OgaModel* m, OgaTokenizer** out) {
  return Guard([&] {
    auto t = std::make_unique<OgaTokenizer>();
    t->obj = Og().attr("Tokenizer")(m->obj);
    *out = t.release();
  });
}
void OgaDestroyTokenizer(OgaTokenizer* t) { Destroy(t); }
OgaResult* OgaUpdateTokenizerOptions(OgaTokenizer* t, const char* const* keys, const char* const* values, size_t n) {
  return Guard([&] {
    py::dict kw;
    for (size_t i = 0; i < n; ++i) kw[py::str(keys[i])] = py::str(values[i]);
    t->obj.attr("update_options")(**kw);
  });
}
OgaResult* OgaTokenizerGetBosTokenId(const OgaTokenizer* t, int32_t* id) {
  return Guard([&] { *id = t->obj.attr("bos_token_id").cast<int32_t>(); });
}
OgaResult* OgaTokenizerGetEosTokenIds(const OgaTokenizer* t, const int32_t** ids, size_t* count) {
  return Guard([&] {
    auto* tt = const_cast<OgaTokenizer*>(t);
    CopyTokens(t->obj.attr("eos_token_ids"), tt->eos);
    *ids = tt->eos.data();
    *count = tt->eos.size();
  });
}
OgaResult* OgaTokenizerGetPadTokenId(const OgaTokenizer* t, int32_t* id) {
  return Guard([&] { *id = t->obj.attr("pad_token_id").cast<int32_t>(); });
}
OgaResult* OgaTokenizerEncode(const OgaTokenizer* t, const char* str, OgaSequences* s) {
  return Guard([&] {
    std::vector<int32_t> ids;
    CopyTokens(t->obj.attr("encode")(str), ids);
    s->rows.push_back(std::move(ids));
  });
}
OgaResult* OgaTokenizerEncodeBatch(const OgaTokenizer* t, const char** strings, size_t count, OgaTensor** out) {
  return Guard([&] {
    py::list l;
    for (size_t i = 0; i < count; ++i) l.append(py::str(strings[i]));
    *out = WrapArray(Np().attr("asarray")(t->obj.attr("encode_batch")(l), "int64"));
  });
}
OgaResult* OgaTokenizerDecodeBatch(const OgaTokenizer* t, const OgaTensor* tensor, OgaStringArray** out) {
  return Guard([&] {
    auto a = std::make_unique<OgaStringArray>();
    for (auto s : t->obj.attr("decode_batch")(tensor->obj)) a->strs.push_back(py::str(s).cast<std::string>());
    *out = a.release();
  });
}
OgaResult* OgaTokenizerToTokenId(const OgaTokenizer* t, const char* str, int32_t* id) {
  return Guard([&] { *id = t->obj.attr("to_token_id")(str).cast<int32_t>(); });
}
OgaResult* OgaTokenizerDecode(const OgaTokenizer* t, const int32_t* tokens, size_t n, const char** out) {
  return Guard([&] { *out = DupString(t->obj.attr("decode")(TokensArray(tokens, n)).cast<std::string>()); });
}
OgaResult* OgaTokenizerApplyChatTemplate(const OgaTokenizer* t, const char* template_str, const char* messages, const char* tools, bool add_generation_prompt,
                                         const char** out) {
  return Guard([&] {
    py::dict kw;
    if (template_str && *template_str) kw["template_str"] = py::str(template_str);
    if (tools && *tools) kw["tools"] = py::str(tools);
    kw["add_generation_prompt"] = py::bool_(add_generation_prompt);
    *out = DupString(t->obj.attr("apply_chat_template")(messages, **kw).cast<std::string>());
  });
}
OgaResult* OgaCreateTokenizerStream(const OgaTokenizer* t, OgaTokenizerStream** out) {
  return Guard([&] {
    auto s = std::make_unique<OgaTokenizerStream>();
    s->obj = t->obj.attr("create_stream")();
    *out = s.release();
  });
}
OgaResult* OgaCreateTokenizerStreamFromProcessor(const OgaMultiModalProcessor* p, OgaTokenizerStream** out) {
  return Guard([&] {
    auto s = std::make_unique<OgaTokenizerStream>();
    s->obj = p->obj.attr("create_stream")();
    *out = s.release();
  });
}
void OgaDestroyTokenizerStream(OgaTokenizerStream* s) { Destroy(s); }
OgaResult* OgaTokenizerStreamDecode(OgaTokenizerStream* s, int32_t token, const char** out) {
  return Guard([&] {
    s->last = s->obj.attr("decode")(token).cast<std::string>();  // valid until the next call on this stream
    *out = s->last.c_str();
  });
}

// ------------------------------------------------------------------------------------------------ images / audio / processor
static py::tuple Strings(const OgaStringArray* a) {
  py::tuple t(a->strs.size());
  for (size_t i = 0; i < a->strs.size(); ++i) t[i] = py::str(a->strs[i]);
  return t;
}
OgaResult* OgaLoadImage(const char* path, OgaImages** out) {
  return Guard([&] {
    auto i = std::make_unique<OgaImages>();
    i->obj = Og().attr("Images").attr("open")(path);
    *out = i.release();
  });
}
OgaResult* OgaLoadImages(const OgaStringArray* paths, OgaImages** out) {
  return Guard([&] {
    auto i = std::make_unique<OgaImages>();
    i->obj = Og().attr("Images").attr("open")(*Strings(paths));
    *out = i.release();
  });
}
OgaResult* OgaLoadImagesFromBuffers(const void** data, const size_t* sizes, size_t count, OgaImages** out) {
  return Guard([&] {
    py::tuple blobs(count);
    for (size_t k = 0; k < count; ++k) blobs[k] = py::bytes(static_cast<const char*>(data[k]), sizes[k]);
    auto i = std::make_unique<OgaImages>();
    i->obj = Og().attr("Images").attr("open_bytes")(*blobs);
    *out = i.release();
  });
}
void OgaDestroyImages(OgaImages* i) { Destroy(i); }
OgaResult* OgaLoadAudio(const char* path, OgaAudios** out) {
  return Guard([&] {
    auto a = std::make_unique<OgaAudios>();
    a->obj = Og().attr("Audios").attr("open")(path);
    *out = a.release();
  });
}
OgaResult* OgaLoadAudios(const OgaStringArray* paths, OgaAudios** out) {
  return Guard([&] {
    auto a = std::make_unique<OgaAudios>();
    a->obj = Og().attr("Audios").attr("open")(*Strings(paths));
    *out = a.release();
  });
}
void OgaDestroyAudios(OgaAudios* a) { Destroy(a); }
OgaResult* OgaCreateMultiModalProcessor(const OgaModel* m, OgaMultiModalProcessor** out) {
  return Guard([&] {
    auto p = std::make_unique<OgaMultiModalProcessor>();
    p->obj = m->obj.attr("create_multimodal_processor")();
    *out = p.release();
  });
}
void OgaDestroyMultiModalProcessor(OgaMultiModalProcessor* p) { Destroy(p); }

// ---- streaming audio front end
OgaResult* OgaCreateStreamingProcessor(OgaModel* m, OgaStreamingProcessor** out) {
  return Guard([&] {
    auto p = std::make_unique<OgaStreamingProcessor>();
    p->obj = m->obj.attr("create_streaming_processor")();
    *out = p.release();
  });
}
void OgaDestroyStreamingProcessor(OgaStreamingProcessor* p) { Destroy(p); }
static void FramesToNamedTensors(const py::object& frames, OgaNamedTensors** out) {
  *out = nullptr;
  if (frames.is_none()) return;
  auto n = std::make_unique<OgaNamedTensors>();
  n->obj = Og().attr("streaming").attr("frames_as_inputs")(frames);
  *out = n.release();
}
OgaResult* OgaStreamingProcessorProcess(OgaStreamingProcessor* p, const float* audio, size_t num_samples, OgaNamedTensors** out) {
  return Guard([&] {
    py::array_t<float> samples(static_cast<py::ssize_t>(num_samples));
    if (num_samples) std::memcpy(samples.mutable_data(), audio, num_samples * sizeof(float));
    FramesToNamedTensors(p->obj.attr("process")(samples), out);
  });
}
OgaResult* OgaStreamingProcessorFlush(OgaStreamingProcessor* p, OgaNamedTensors** out) {
  return Guard([&] { FramesToNamedTensors(p->obj.attr("flush")(), out); });
}
OgaResult* OgaStreamingProcessorSetOption(OgaStreamingProcessor* p, const char* key, const char* value) {
  return Guard([&] { p->obj.attr("set_option")(key, value); });
}
OgaResult* OgaStreamingProcessorGetOption(const OgaStreamingProcessor* p, const char* key, const char** value) {
  return Guard([&] {
    auto* self = const_cast<OgaStreamingProcessor*>(p);
    self->option = p->obj.attr("get_option")(key).cast<std::string>();
    *value = self->option.c_str();
  });
}
static OgaResult* Process(const OgaMultiModalProcessor* p, const char* prompt, const OgaImages* images, const OgaAudios* audios, OgaNamedTensors** out) {
  return Guard([&] {
    py::dict kw;
    if (images) kw["images"] = images->obj;
    if (audios) kw["audios"] = audios->obj;
    auto n = std::make_unique<OgaNamedTensors>();
    n->obj = p->obj(prompt ? py::object(py::str(prompt)) : py::object(py::none()), **kw);
    *out = n.release();
  });
}
OgaResult* OgaProcessorProcessImages(const OgaMultiModalProcessor* p, const char* prompt, const OgaImages* images, OgaNamedTensors** out) {
  return Process(p, prompt, images, nullptr, out);
}
OgaResult* OgaProcessorProcessAudios(const OgaMultiModalProcessor* p, const char* prompt, const OgaAudios* audios, OgaNamedTensors** out) {
  return Process(p, prompt, nullptr, audios, out);
}
OgaResult* OgaProcessorProcessImagesAndAudios(const OgaMultiModalProcessor* p, const char* prompt, const OgaImages* images, const OgaAudios* audios,
                                              OgaNamedTensors** out) {
  return Process(p, prompt, images, audios, out);
}
OgaResult* OgaProcessorDecode(const OgaMultiModalProcessor* p, const int32_t* tokens, size_t n, const char** out) {
  return Guard([&] { *out = DupString(p->obj.attr("decode")(TokensArray(tokens, n)).cast<std::string>()); });
}

// ------------------------------------------------------------------------------------------------ adapters
OgaResult* OgaCreateAdapters(const OgaModel* m, OgaAdapters** out) {
  return Guard([&] {
    auto a = std::make_unique<OgaAdapters>();
    a->obj = Og().attr("Adapters")(m->obj);
    *out = a.release();
  });
}
void OgaDestroyAdapters(OgaAdapters* a) { Destroy(a); }
OgaResult* OgaLoadAdapter(OgaAdapters* a, const char* path, const char* name) {
  return Guard([&] { a->obj.attr("load")(path, name); });
}
OgaResult* OgaUnloadAdapter(OgaAdapters* a, const char* name) {
  return Guard([&] { a->obj.attr("unload")(name); });
}
OgaResult* OgaSetActiveAdapter(OgaGenerator* g, OgaAdapters* a, const char* name) {
  return Guard([&] { g->obj.attr("set_active_adapter")(a->obj, name); });
}

// ------------------------------------------------------------------------------------------------ engine
OgaResult* OgaCreateEngine(OgaModel* m, OgaEngine** out) {
  return Guard([&] {
    auto e = std::make_unique<OgaEngine>();
    e->obj = Og().attr("Engine")(m->obj);
    *out = e.release();
  });
}
void OgaDestroyEngine(OgaEngine* e) { Destroy(e); }
OgaResult* OgaEngineStep(OgaEngine* e, OgaRequest** request) {
  *request = nullptr;
  return Guard([&] {
    py::object r = e->obj.attr("step")();
    if (r.is_none()) return;
    auto h = std::make_unique<OgaRequest>();  // one more external handle on the same request
    h->obj = r;
    *request = h.release();
  });
}
OgaResult* OgaEngineHasPendingRequests(OgaEngine* e, bool* out) {
  return Guard([&] { *out = e->obj.attr("has_pending_requests")().cast<bool>(); });
}
OgaResult* OgaEngineAddRequest(OgaEngine* e, OgaRequest* r) {
  return Guard([&] { e->obj.attr("add_request")(r->obj); });
}
OgaResult* OgaEngineRemoveRequest(OgaEngine* e, OgaRequest* r) {
  return Guard([&] { e->obj.attr("remove_request")(r->obj); });
}
OgaResult* OgaCreateRequest(OgaGeneratorParams* p, OgaRequest** out) {
  return Guard([&] {
    auto r = std::make_unique<OgaRequest>();
    r->obj = Og().attr("Request")(p->obj);
    *out = r.release();
  });
}
void OgaDestroyRequest(OgaRequest* r) { Destroy(r); }
static py::object OneSequence(const OgaSequences* s) {
  if (s->rows.size() != 1) throw std::runtime_error("a request takes exactly one token sequence");
  return TokensArray(s->rows[0].data(), s->rows[0].size());
}
OgaResult* OgaRequestAddTokens(OgaRequest* r, const OgaSequences* s) {
  return Guard([&] { r->obj.attr("add_tokens")(OneSequence(s)); });
}
OgaResult* OgaRequestContinue(OgaRequest* r, const OgaSequences* s) {
  return Guard([&] { r->obj.attr("continue_with")(OneSequence(s)); });
}
OgaResult* OgaRequestContinueWithMaxLength(OgaRequest* r, const OgaSequences* s, size_t max_length) {
  return Guard([&] { r->obj.attr("continue_with")(OneSequence(s), max_length); });
}
OgaResult* OgaRequestSetOpaqueData(OgaRequest* r, void* data) {
  return Guard([&] { r->obj.attr("set_opaque_data")(py::int_(reinterpret_cast<uintptr_t>(data))); });
}
OgaResult* OgaRequestGetOpaqueData(OgaRequest* r, void** data) {
  return Guard([&] {
    py::object v = r->obj.attr("get_opaque_data")();
    *data = v.is_none() ? nullptr : reinterpret_cast<void*>(v.cast<uintptr_t>());
  });
}
OgaResult* OgaRequestHasUnseenTokens(const OgaRequest* r, bool* out) {
  return Guard([&] { *out = r->obj.attr("has_unseen_tokens")().cast<bool>(); });
}
OgaResult* OgaRequestGetUnseenToken(OgaRequest* r, int32_t* out) {
  return Guard([&] { *out = r->obj.attr("get_unseen_token")().cast<int32_t>(); });
}
OgaResult* OgaRequestSetActiveAdapter(OgaRequest* r, OgaAdapters* a, const char* name) {
  return Guard([&] { r->obj.attr("set_active_adapter")(a->obj, name ? py::object(py::str(name)) : py::object(py::none())); });
}
OgaResult* OgaRequestIsTurnComplete(const OgaRequest* r, bool* out) {
  return Guard([&] { *out = r->obj.attr("is_turn_complete")().cast<bool>(); });
}

}  // extern "C"
