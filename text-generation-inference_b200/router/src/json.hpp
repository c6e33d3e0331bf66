// Small JSON value type with a strict parser and a serializer (UTF-8, \uXXXX escapes, surrogate
// pairs).  Objects keep insertion order so responses are stable.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace json {

class Value {
 public:
  enum Type { Null, Bool, Number, String, Array, Object };
  Value() : type_(Null) {}
  Value(std::nullptr_t) : type_(Null) {}
  Value(bool b) : type_(Bool), b_(b) {}
  Value(int v) : type_(Number), n_(v), is_int_(true) {}
  Value(unsigned v) : type_(Number), n_(v), is_int_(true) {}
  Value(long v) : type_(Number), n_(static_cast<double>(v)), is_int_(true), i_(v) {}
  Value(long long v) : type_(Number), n_(static_cast<double>(v)), is_int_(true), i_(v) {}
  Value(unsigned long v) : type_(Number), n_(static_cast<double>(v)), is_int_(true), u_(v), is_u_(true) {}
  Value(unsigned long long v) : type_(Number), n_(static_cast<double>(v)), is_int_(true), u_(v), is_u_(true) {}
  Value(double v) : type_(Number), n_(v) {}
  Value(float v) : type_(Number), n_(v) {}
  Value(const char* s) : type_(String), s_(s) {}
  Value(std::string s) : type_(String), s_(std::move(s)) {}
  static Value array() { Value v; v.type_ = Array; return v; }
  static Value object() { Value v; v.type_ = Object; return v; }

  Type type() const { return type_; }
  bool is_null() const { return type_ == Null; }
  bool is_bool() const { return type_ == Bool; }
  bool is_number() const { return type_ == Number; }
  bool is_string() const { return type_ == String; }
  bool is_array() const { return type_ == Array; }
  bool is_object() const { return type_ == Object; }
  bool as_bool() const { return b_; }
  double as_double() const { return n_; }
  long long as_int() const { return is_u_ ? static_cast<long long>(u_) : (i_ != 0 ? i_ : static_cast<long long>(n_)); }
  unsigned long long as_u64() const { return is_u_ ? u_ : static_cast<unsigned long long>(as_int()); }
  bool is_integer() const { return type_ == Number && (is_int_ || std::floor(n_) == n_); }
  const std::string& as_string() const { return s_; }
  const std::vector<Value>& items() const { return a_; }
  std::vector<Value>& items() { return a_; }
  const std::vector<std::pair<std::string, Value>>& members() const { return o_; }

  void push(Value v) { a_.push_back(std::move(v)); }
  Value& set(const std::string& k, Value v) {
    for (auto& kv : o_)
      if (kv.first == k) { kv.second = std::move(v); return kv.second; }
    o_.emplace_back(k, std::move(v));
    return o_.back().second;
  }
  const Value* find(const std::string& k) const {
    if (type_ != Object) return nullptr;
    for (auto& kv : o_)
      if (kv.first == k) return &kv.second;
    return nullptr;
  }
  bool has(const std::string& k) const { const Value* v = find(k); return v && !v->is_null(); }
  const Value& operator[](const std::string& k) const {
    static const Value null_v;
    const Value* v = find(k);
    return v ? *v : null_v;
  }

  std::string dump() const { std::string out; write(out); return out; }
  void write(std::string& out) const;
  static Value parse(const std::string& text);

 private:
  Type type_;
  bool b_ = false;
  double n_ = 0;
  bool is_int_ = false;
  long long i_ = 0;
  unsigned long long u_ = 0;
  bool is_u_ = false;
  std::string s_;
  std::vector<Value> a_;
  std::vector<std::pair<std::string, Value>> o_;
};

inline void escape_to(const std::string& s, std::string& out) {
  out.push_back('"');
  for (unsigned char c : s) {
    switch (c) {
      case '"': out += "\\\""; break;
      case '\\': out += "\\\\"; break;
      case '\n': out += "\\n"; break;
      case '\r': out += "\\r"; break;
      case '\t': out += "\\t"; break;
      case '\b': out += "\\b"; break;
      case '\f': out += "\\f"; break;
      default:
        if (c < 0x20) {
          char buf[8];
          snprintf(buf, sizeof buf, "\\u%04x", c);
          out += buf;
        } else {
          out.push_back(static_cast<char>(c));
        }
    }
  }
  out.push_back('"');
}

inline void Value::write(std::string& out) const {
  switch (type_) {
    case Null: out += "null"; break;
    case Bool: out += b_ ? "true" : "false"; break;
    case Number: {
      char buf[40];
      if (is_u_) snprintf(buf, sizeof buf, "%llu", u_);
      else if (is_int_) snprintf(buf, sizeof buf, "%lld", i_ != 0 ? i_ : static_cast<long long>(n_));
      else if (std::isnan(n_) || std::isinf(n_)) snprintf(buf, sizeof buf, "null");
      else snprintf(buf, sizeof buf, "%.9g", n_);
      out += buf;
      break;
    }
    case String: escape_to(s_, out); break;
    case Array:
      out.push_back('[');
      for (size_t i = 0; i < a_.size(); ++i) {
        if (i) out.push_back(',');
        a_[i].write(out);
      }
      out.push_back(']');
      break;
    case Object:
      out.push_back('{');
      for (size_t i = 0; i < o_.size(); ++i) {
        if (i) out.push_back(',');
        escape_to(o_[i].first, out);
        out.push_back(':');
        o_[i].second.write(out);
      }
      out.push_back('}');
      break;
  }
}

namespace detail {
struct Parser {
  const std::string& t;
  size_t p = 0;
  int depth = 0;
  explicit Parser(const std::string& s) : t(s) {}
  [[noreturn]] void fail(const char* m) { throw std::runtime_error(std::string("json: ") + m + " at offset " + std::to_string(p)); }
  void ws() { while (p < t.size() && (t[p] == ' ' || t[p] == '\n' || t[p] == '\r' || t[p] == '\t')) ++p; }
  static void utf8(uint32_t cp, std::string& o) {
    if (cp < 0x80) o.push_back(static_cast<char>(cp));
    else if (cp < 0x800) { o.push_back(static_cast<char>(0xC0 | (cp >> 6))); o.push_back(static_cast<char>(0x80 | (cp & 0x3F))); }
    else if (cp < 0x10000) { o.push_back(static_cast<char>(0xE0 | (cp >> 12))); o.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F))); o.push_back(static_cast<char>(0x80 | (cp & 0x3F))); }
    else { o.push_back(static_cast<char>(0xF0 | (cp >> 18))); o.push_back(static_cast<char>(0x80 | ((cp >> 12) & 0x3F))); o.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F))); o.push_back(static_cast<char>(0x80 | (cp & 0x3F))); }
  }
  uint32_t hex4() {
    if (p + 4 > t.size()) fail("truncated \\u escape");
    uint32_t v = 0;
    for (int i = 0; i < 4; ++i) {
      char c = t[p++];
      v <<= 4;
      if (c >= '0' && c <= '9') v |= c - '0';
      else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
      else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
      else fail("bad \\u escape");
    }
    return v;
  }
  std::string str() {
    std::string o;
    ++p;
    while (true) {
      if (p >= t.size()) fail("unterminated string");
      char c = t[p++];
      if (c == '"') return o;
      if (c == '\\') {
        if (p >= t.size()) fail("bad escape");
        char e = t[p++];
        switch (e) {
          case '"': o.push_back('"'); break;
          case '\\': o.push_back('\\'); break;
          case '/': o.push_back('/'); break;
          case 'b': o.push_back('\b'); break;
          case 'f': o.push_back('\f'); break;
          case 'n': o.push_back('\n'); break;
          case 'r': o.push_back('\r'); break;
          case 't': o.push_back('\t'); break;
          case 'u': {
            uint32_t cp = hex4();
            if (cp >= 0xD800 && cp <= 0xDBFF && p + 1 < t.size() && t[p] == '\\' && t[p + 1] == 'u') {
              p += 2;
              uint32_t lo = hex4();
              if (lo >= 0xDC00 && lo <= 0xDFFF) cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
            }
            utf8(cp, o);
            break;
          }
          default: fail("bad escape");
        }
      } else {
        o.push_back(c);
      }
    }
  }
  Value value() {
    if (++depth > 256) fail("nesting too deep");
    ws();
    if (p >= t.size()) fail("unexpected end");
    Value out;
    char c = t[p];
    if (c == '{') {
      out = Value::object();
      ++p;
      ws();
      if (p < t.size() && t[p] == '}') { ++p; --depth; return out; }
      while (true) {
        ws();
        if (p >= t.size() || t[p] != '"') fail("expected object key");
        std::string k = str();
        ws();
        if (p >= t.size() || t[p] != ':') fail("expected ':'");
        ++p;
        out.set(k, value());
        ws();
        if (p < t.size() && t[p] == ',') { ++p; continue; }
        if (p < t.size() && t[p] == '}') { ++p; break; }
        fail("expected ',' or '}'");
      }
    } else if (c == '[') {
      out = Value::array();
      ++p;
      ws();
      if (p < t.size() && t[p] == ']') { ++p; --depth; return out; }
      while (true) {
        out.push(value());
        ws();
        if (p < t.size() && t[p] == ',') { ++p; continue; }
        if (p < t.size() && t[p] == ']') { ++p; break; }
        fail("expected ',' or ']'");
      }
    } else if (c == '"') {
      out = Value(str());
    } else if (t.compare(p, 4, "true") == 0) { p += 4; out = Value(true); }
    else if (t.compare(p, 5, "false") == 0) { p += 5; out = Value(false); }
    else if (t.compare(p, 4, "null") == 0) { p += 4; out = Value(); }
    else {
      size_t s = p;
      bool is_float = false;
      if (t[p] == '-') ++p;
      while (p < t.size() && ((t[p] >= '0' && t[p] <= '9') || t[p] == '.' || t[p] == 'e' || t[p] == 'E' || t[p] == '+' || t[p] == '-')) {
        if (t[p] == '.' || t[p] == 'e' || t[p] == 'E') is_float = true;
        ++p;
      }
      if (s == p) fail("unexpected character");
      std::string num = t.substr(s, p - s);
      if (is_float) out = Value(strtod(num.c_str(), nullptr));
      else if (num[0] == '-') out = Value(static_cast<long long>(strtoll(num.c_str(), nullptr, 10)));
      else out = Value(static_cast<unsigned long long>(strtoull(num.c_str(), nullptr, 10)));
    }
    --depth;
    return out;
  }
};
}  // namespace detail

inline Value Value::parse(const std::string& text) {
  detail::Parser ps(text);
  Value v = ps.value();
  ps.ws();
  if (ps.p != text.size()) ps.fail("trailing characters");
  return v;
}

}  // namespace json
