// Minimal JSON document model, parser and writer for the control plane (config files, specs and
// control messages). Objects keep insertion order so that serialised specs are stable.
// Numbers remember whether they were written as integers, so u64 seeds survive a round trip.
#pragma once
#include <cerrno>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace ono {

struct JsonError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

class Json {
 public:
  enum Type { Null, Bool, Int, Float, String, Array, Object };
  using Member = std::pair<std::string, Json>;

  Json() : type_(Null) {}
  Json(std::nullptr_t) : type_(Null) {}
  Json(bool b) : type_(Bool), b_(b) {}
  Json(int v) : type_(Int), i_(v) {}
  Json(long v) : type_(Int), i_(v) {}
  Json(long long v) : type_(Int), i_(v) {}
  Json(unsigned v) : type_(Int), i_(v) {}
  Json(unsigned long v) : type_(Int), i_((long long)v), u_(v), big_(v > 0x7fffffffffffffffULL) {}
  Json(unsigned long long v) : type_(Int), i_((long long)v), u_(v), big_(v > 0x7fffffffffffffffULL) {}
  Json(double v) : type_(Float), d_(v) {}
  Json(float v) : type_(Float), d_(v) {}
  Json(const char* s) : type_(String), s_(s) {}
  Json(std::string s) : type_(String), s_(std::move(s)) {}

  static Json array() { Json j; j.type_ = Array; return j; }
  static Json object() { Json j; j.type_ = Object; return j; }
  // {"key": value} : the serde encoding of a struct enum variant.
  static Json tagged(const std::string& key, Json value) {
    Json j = object();
    j.set(key, std::move(value));
    return j;
  }

  Type type() const { return type_; }
  bool is_null() const { return type_ == Null; }
  bool is_bool() const { return type_ == Bool; }
  bool is_number() const { return type_ == Int || type_ == Float; }
  bool is_int() const { return type_ == Int; }
  bool is_string() const { return type_ == String; }
  bool is_array() const { return type_ == Array; }
  bool is_object() const { return type_ == Object; }

  bool as_bool() const { need(Bool, "bool"); return b_; }
  double as_double() const {
    if (type_ == Int) return big_ ? (double)u_ : (double)i_;
    need(Float, "number");
    return d_;
  }
  long long as_int() const {
    if (type_ == Float && std::floor(d_) == d_ && std::fabs(d_) < 9e15) return (long long)d_;
    need(Int, "integer");
    if (big_) throw JsonError("integer out of i64 range");
    return i_;
  }
  unsigned long long as_u64() const {
    if (type_ == Float && d_ >= 0 && std::floor(d_) == d_ && d_ < 1.8e19) return (unsigned long long)d_;
    need(Int, "unsigned integer");
    if (!big_ && i_ < 0) throw JsonError("expected a non-negative integer");
    return big_ ? u_ : (unsigned long long)i_;
  }
  const std::string& as_string() const { need(String, "string"); return s_; }

  // arrays
  const std::vector<Json>& items() const { need(Array, "array"); return arr_; }
  std::vector<Json>& items() { need(Array, "array"); return arr_; }
  void push(Json v) { need(Array, "array"); arr_.push_back(std::move(v)); }
  size_t size() const { return type_ == Array ? arr_.size() : type_ == Object ? obj_.size() : 0; }
  const Json& operator[](size_t i) const { need(Array, "array"); return arr_.at(i); }

  // objects
  const std::vector<Member>& members() const { need(Object, "object"); return obj_; }
  void set(const std::string& k, Json v) {
    need(Object, "object");
    for (auto& m : obj_)
      if (m.first == k) { m.second = std::move(v); return; }
    obj_.emplace_back(k, std::move(v));
  }
  const Json* find(const std::string& k) const {
    if (type_ != Object) return nullptr;
    for (auto& m : obj_)
      if (m.first == k) return &m.second;
    return nullptr;
  }
  bool has(const std::string& k) const { return find(k) != nullptr; }
  const Json& at(const std::string& k) const {
    const Json* p = find(k);
    if (!p) throw JsonError("missing field `" + k + "`");
    return *p;
  }

  std::string dump() const { std::string out; write(out); return out; }
  static Json parse(const std::string& text) {
    Parser p{text.data(), text.data() + text.size()};
    p.ws();
    Json v = p.value();
    p.ws();
    if (p.cur != p.end) throw JsonError("trailing characters after JSON document");
    return v;
  }

 private:
  Type type_;
  bool b_ = false;
  long long i_ = 0;
  unsigned long long u_ = 0;
  bool big_ = false;
  double d_ = 0.0;
  std::string s_;
  std::vector<Json> arr_;
  std::vector<Member> obj_;

  void need(Type t, const char* what) const {
    if (type_ != t) throw JsonError(std::string("expected ") + what);
  }

  static void write_string(const std::string& s, std::string& out) {
    out.push_back('"');
    for (unsigned char c : s) {
      switch (c) {
        case '"': out += "\\\""; break;
        case '\\': out += "\\\\"; break;
        case '\n': out += "\\n"; break;
        case '\r': out += "\\r"; break;
        case '\t': out += "\\t"; break;
        default:
          if (c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); out += b; }
          else out.push_back((char)c);
      }
    }
    out.push_back('"');
  }

  void write(std::string& out) const {
    switch (type_) {
      case Null: out += "null"; break;
      case Bool: out += b_ ? "true" : "false"; break;
      case Int: out += big_ ? std::to_string(u_) : std::to_string(i_); break;
      case Float: {
        if (!std::isfinite(d_)) { out += "null"; break; }  // serde_json writes non-finite floats as null
        char b[40];
        snprintf(b, sizeof b, "%.17g", d_);
        std::string s(b);
        if (s.find_first_of(".eE") == std::string::npos) s += ".0";
        out += s;
        break;
      }
      case String: write_string(s_, out); break;
      case Array:
        out.push_back('[');
        for (size_t i = 0; i < arr_.size(); ++i) { if (i) out.push_back(','); arr_[i].write(out); }
        out.push_back(']');
        break;
      case Object:
        out.push_back('{');
        for (size_t i = 0; i < obj_.size(); ++i) {
          if (i) out.push_back(',');
          write_string(obj_[i].first, out);
          out.push_back(':');
          obj_[i].second.write(out);
        }
        out.push_back('}');
        break;
    }
  }

  struct Parser {
    const char* cur;
    const char* end;
    void ws() { while (cur != end && (*cur == ' ' || *cur == '\n' || *cur == '\t' || *cur == '\r')) ++cur; }
    [[noreturn]] void fail(const char* m) { throw JsonError(std::string("JSON parse error: ") + m); }
    bool eat(const char* lit) {
      size_t n = strlen_(lit);
      if ((size_t)(end - cur) >= n && std::char_traits<char>::compare(cur, lit, n) == 0) { cur += n; return true; }
      return false;
    }
    static size_t strlen_(const char* s) { size_t n = 0; while (s[n]) ++n; return n; }
    Json value() {
      if (cur == end) fail("unexpected end");
      switch (*cur) {
        case '{': return object();
        case '[': return array();
        case '"': return Json(string());
        case 't': if (eat("true")) return Json(true); fail("bad literal");
        case 'f': if (eat("false")) return Json(false); fail("bad literal");
        case 'n': if (eat("null")) return Json(); fail("bad literal");
        default: return number();
      }
    }
    Json number() {
      const char* s = cur;
      bool is_float = false;
      if (cur != end && (*cur == '-' || *cur == '+')) ++cur;
      while (cur != end && ((*cur >= '0' && *cur <= '9') || *cur == '.' || *cur == 'e' || *cur == 'E' || *cur == '-' || *cur == '+')) {
        if (*cur == '.' || *cur == 'e' || *cur == 'E') is_float = true;
        ++cur;
      }
      if (s == cur) fail("unexpected character");
      std::string tok(s, cur);
      if (!is_float) {
        errno = 0;
        if (tok[0] == '-') {
          long long v = strtoll(tok.c_str(), nullptr, 10);
          if (errno == 0) return Json(v);
        } else {
          unsigned long long v = strtoull(tok.c_str(), nullptr, 10);
          if (errno == 0) return Json(v);
        }
      }
      return Json(strtod(tok.c_str(), nullptr));
    }
    std::string string() {
      ++cur;  // opening quote
      std::string out;
      while (true) {
        if (cur == end) fail("unterminated string");
        char c = *cur++;
        if (c == '"') break;
        if (c != '\\') { out.push_back(c); continue; }
        if (cur == end) fail("bad escape");
        char e = *cur++;
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
            if (end - cur < 4) fail("bad \\u escape");
            unsigned cp = (unsigned)strtoul(std::string(cur, cur + 4).c_str(), nullptr, 16);
            cur += 4;
            if (cp < 0x80) out.push_back((char)cp);
            else if (cp < 0x800) { out.push_back((char)(0xC0 | (cp >> 6))); out.push_back((char)(0x80 | (cp & 0x3F))); }
            else { out.push_back((char)(0xE0 | (cp >> 12))); out.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out.push_back((char)(0x80 | (cp & 0x3F))); }
            break;
          }
          default: fail("bad escape");
        }
      }
      return out;
    }
    Json array() {
      ++cur;
      Json a = Json::array();
      ws();
      if (cur != end && *cur == ']') { ++cur; return a; }
      while (true) {
        ws();
        a.push(value());
        ws();
        if (cur == end) fail("unterminated array");
        if (*cur == ',') { ++cur; continue; }
        if (*cur == ']') { ++cur; break; }
        fail("expected , or ]");
      }
      return a;
    }
    Json object() {
      ++cur;
      Json o = Json::object();
      ws();
      if (cur != end && *cur == '}') { ++cur; return o; }
      while (true) {
        ws();
        if (cur == end || *cur != '"') fail("expected object key");
        std::string k = string();
        ws();
        if (cur == end || *cur != ':') fail("expected :");
        ++cur;
        ws();
        o.set(k, value());
        ws();
        if (cur == end) fail("unterminated object");
        if (*cur == ',') { ++cur; continue; }
        if (*cur == '}') { ++cur; break; }
        fail("expected , or }");
      }
      return o;
    }
  };
};

}  // namespace ono
