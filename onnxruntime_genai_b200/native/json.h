// Small JSON document model + recursive-descent parser and serializer.
//
// The runtime's configuration file (genai_config.json) and overlays are read with this parser and
// then validated key-by-key against a schema table (config.cpp).  The reference reads the same
// files with a hand-written SAX parser (reference: src/json.h, src/json.cpp); a DOM plus schema
// table is used here instead because overlays, provider options and Python-side inspection all
// want the same tree.
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <string_view>
#include <utility>
#include <variant>
#include <vector>

namespace ogb::json {

struct Value;
using Array = std::vector<Value>;
// Object keeps insertion order (config round trips keep the author's ordering).
using Member = std::pair<std::string, Value>;
using Object = std::vector<Member>;

struct Value {
  enum class Kind { Null, Bool, Number, String, Array, Object };
  Kind kind{Kind::Null};
  bool b{};
  double num{};
  std::string str;
  std::shared_ptr<Array> arr;
  std::shared_ptr<Object> obj;

  Value() = default;
  static Value MakeBool(bool v) { Value x; x.kind = Kind::Bool; x.b = v; return x; }
  static Value MakeNumber(double v) { Value x; x.kind = Kind::Number; x.num = v; return x; }
  static Value MakeString(std::string v) { Value x; x.kind = Kind::String; x.str = std::move(v); return x; }
  static Value MakeArray() { Value x; x.kind = Kind::Array; x.arr = std::make_shared<Array>(); return x; }
  static Value MakeObject() { Value x; x.kind = Kind::Object; x.obj = std::make_shared<Object>(); return x; }

  bool is_null() const { return kind == Kind::Null; }
  bool is_bool() const { return kind == Kind::Bool; }
  bool is_number() const { return kind == Kind::Number; }
  bool is_string() const { return kind == Kind::String; }
  bool is_array() const { return kind == Kind::Array; }
  bool is_object() const { return kind == Kind::Object; }

  const Value* find(std::string_view key) const;
  Value* find(std::string_view key);
  Value& set(std::string_view key, Value v);  // insert or replace
  const char* kind_name() const;
};

struct ParseError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

// Parses a complete JSON document; throws ParseError with line/column on malformed input.
Value Parse(std::string_view text);
std::string Dump(const Value& v, int indent = -1);

}  // namespace ogb::json
