#include "json.h"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <sstream>

namespace ogb::json {

const Value* Value::find(std::string_view key) const {
  if (!is_object()) return nullptr;
  for (auto& m : *obj)
    if (m.first == key) return &m.second;
  return nullptr;
}
Value* Value::find(std::string_view key) {
  if (!is_object()) return nullptr;
  for (auto& m : *obj)
    if (m.first == key) return &m.second;
  return nullptr;
}
Value& Value::set(std::string_view key, Value v) {
  if (!is_object()) throw std::runtime_error("json: set() on a non-object");
  if (auto* p = find(key)) {
    *p = std::move(v);
    return *p;
  }
  obj->emplace_back(std::string(key), std::move(v));
  return obj->back().second;
}
const char* Value::kind_name() const {
  switch (kind) {
    case Kind::Null: return "null";
    case Kind::Bool: return "bool";
    case Kind::Number: return "number";
    case Kind::String: return "string";
    case Kind::Array: return "array";
    case Kind::Object: return "object";
  }
  return "?";
}

namespace {
struct Parser {
  std::string_view s;
  size_t i{0};

  [[noreturn]] void Fail(const std::string& what) const {
    size_t line = 1, col = 1;
    for (size_t k = 0; k < i && k < s.size(); ++k) {
      if (s[k] == '\n') { ++line; col = 1; } else ++col;
    }
    std::ostringstream o;
    o << "JSON parse error at line " << line << " column " << col << ": " << what;
    throw ParseError(o.str());
  }
  void Ws() {
    while (i < s.size()) {
      char c = s[i];
      if (c == ' ' || c == '\t' || c == '\n' || c == '\r') ++i;
      else if (c == '/' && i + 1 < s.size() && s[i + 1] == '/') {  // tolerate // comments
        while (i < s.size() && s[i] != '\n') ++i;
      } else break;
    }
  }
  bool Eat(char c) {
    Ws();
    if (i < s.size() && s[i] == c) { ++i; return true; }
    return false;
  }
  void Expect(char c) {
    if (!Eat(c)) Fail(std::string("expected '") + c + "'");
  }
  static void AppendUtf8(std::string& out, uint32_t cp) {
    if (cp < 0x80) out.push_back(char(cp));
    else if (cp < 0x800) { out.push_back(char(0xC0 | (cp >> 6))); out.push_back(char(0x80 | (cp & 0x3F))); }
    else if (cp < 0x10000) {
      out.push_back(char(0xE0 | (cp >> 12))); out.push_back(char(0x80 | ((cp >> 6) & 0x3F))); out.push_back(char(0x80 | (cp & 0x3F)));
    } else {
      out.push_back(char(0xF0 | (cp >> 18))); out.push_back(char(0x80 | ((cp >> 12) & 0x3F)));
      out.push_back(char(0x80 | ((cp >> 6) & 0x3F))); out.push_back(char(0x80 | (cp & 0x3F)));
    }
  }
  uint32_t Hex4() {
    if (i + 4 > s.size()) Fail("truncated \\u escape");
    uint32_t v = 0;
    for (int k = 0; k < 4; ++k) {
      char c = s[i++];
      v <<= 4;
      if (c >= '0' && c <= '9') v |= c - '0';
      else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
      else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
      else Fail("bad hex digit in \\u escape");
    }
    return v;
  }
  std::string String() {
    Ws();
    if (i >= s.size() || s[i] != '"') Fail("expected string");
    ++i;
    std::string out;
    while (true) {
      if (i >= s.size()) Fail("unterminated string");
      char c = s[i++];
      if (c == '"') break;
      if (c == '\\') {
        if (i >= s.size()) Fail("unterminated escape");
        char e = s[i++];
        switch (e) {
          case '"': out.push_back('"'); break;
          case '\\': out.push_back('\\'); break;
          case '/': out.push_back('/'); break;
          case 'b': out.push_back('\b'); break;
          case 'f': out.push_back('\f'); break;
          case 'n': out.push_back('\n'); break;
          case 'r': out.push_back('\r'); break;
          case 't': out.push_back('\t'); break;
          case 'u': {
            uint32_t cp = Hex4();
            if (cp >= 0xD800 && cp <= 0xDBFF && i + 1 < s.size() && s[i] == '\\' && s[i + 1] == 'u') {
              i += 2;
              uint32_t lo = Hex4();
              cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
            }
            AppendUtf8(out, cp);
            break;
          }
          default: Fail("unknown escape");
        }
      } else {
        out.push_back(c);
      }
    }
    return out;
  }
  Value Any(int depth) {
    if (depth > 256) Fail("nesting too deep");
    Ws();
    if (i >= s.size()) Fail("unexpected end of input");
    char c = s[i];
    if (c == '{') {
      ++i;
      Value v = Value::MakeObject();
      if (Eat('}')) return v;
      while (true) {
        std::string k = String();
        Expect(':');
        Value child = Any(depth + 1);
        if (v.find(k)) Fail("duplicate key \"" + k + "\"");
        v.obj->emplace_back(std::move(k), std::move(child));
        if (Eat(',')) continue;
        Expect('}');
        return v;
      }
    }
    if (c == '[') {
      ++i;
      Value v = Value::MakeArray();
      if (Eat(']')) return v;
      while (true) {
        v.arr->push_back(Any(depth + 1));
        if (Eat(',')) continue;
        Expect(']');
        return v;
      }
    }
    if (c == '"') return Value::MakeString(String());
    if (s.compare(i, 4, "true") == 0) { i += 4; return Value::MakeBool(true); }
    if (s.compare(i, 5, "false") == 0) { i += 5; return Value::MakeBool(false); }
    if (s.compare(i, 4, "null") == 0) { i += 4; return Value(); }
    // number
    size_t start = i;
    if (i < s.size() && (s[i] == '-' || s[i] == '+')) ++i;
    bool digits = false;
    while (i < s.size() && ((s[i] >= '0' && s[i] <= '9') || s[i] == '.' || s[i] == 'e' || s[i] == 'E' || s[i] == '-' || s[i] == '+')) {
      if (s[i] >= '0' && s[i] <= '9') digits = true;
      ++i;
    }
    if (!digits) { i = start; Fail("unexpected character"); }
    std::string tmp(s.substr(start, i - start));
    char* endp = nullptr;
    double d = std::strtod(tmp.c_str(), &endp);
    if (endp == tmp.c_str() || *endp != 0) { i = start; Fail("malformed number"); }
    return Value::MakeNumber(d);
  }
};

void DumpString(std::string& out, const std::string& s) {
  out.push_back('"');
  for (unsigned char c : s) {
    switch (c) {
      case '"': out += "\\\""; break;
      case '\\': out += "\\\\"; break;
      case '\n': out += "\\n"; break;
      case '\r': out += "\\r"; break;
      case '\t': out += "\\t"; break;
      default:
        if (c < 0x20) {
          char buf[8];
          std::snprintf(buf, sizeof buf, "\\u%04x", c);
          out += buf;
        } else out.push_back(char(c));
    }
  }
  out.push_back('"');
}

void DumpRec(std::string& out, const Value& v, int indent, int level) {
  auto nl = [&](int lv) {
    if (indent < 0) return;
    out.push_back('\n');
    out.append(size_t(indent * lv), ' ');
  };
  switch (v.kind) {
    case Value::Kind::Null: out += "null"; break;
    case Value::Kind::Bool: out += v.b ? "true" : "false"; break;
    case Value::Kind::Number: {
      double d = v.num;
      if (std::isfinite(d) && d == std::floor(d) && std::fabs(d) < 9.0e15) {
        out += std::to_string((long long)d);
      } else {
        char buf[40];
        std::snprintf(buf, sizeof buf, "%.9g", d);
        out += buf;
      }
      break;
    }
    case Value::Kind::String: DumpString(out, v.str); break;
    case Value::Kind::Array: {
      out.push_back('[');
      bool first = true;
      for (auto& e : *v.arr) {
        if (!first) out.push_back(',');
        first = false;
        nl(level + 1);
        DumpRec(out, e, indent, level + 1);
      }
      if (!v.arr->empty()) nl(level);
      out.push_back(']');
      break;
    }
    case Value::Kind::Object: {
      out.push_back('{');
      bool first = true;
      for (auto& m : *v.obj) {
        if (!first) out.push_back(',');
        first = false;
        nl(level + 1);
        DumpString(out, m.first);
        out += indent < 0 ? ":" : ": ";
        DumpRec(out, m.second, indent, level + 1);
      }
      if (!v.obj->empty()) nl(level);
      out.push_back('}');
      break;
    }
  }
}
}  // namespace

Value Parse(std::string_view text) {
  Parser p{text};
  Value v = p.Any(0);
  p.Ws();
  if (p.i != text.size()) p.Fail("trailing characters after document");
  return v;
}

std::string Dump(const Value& v, int indent) {
  std::string out;
  DumpRec(out, v, indent, 0);
  return out;
}

}  // namespace ogb::json
