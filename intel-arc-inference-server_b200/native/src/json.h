// A small JSON value with ordered objects: parse, dump, lookup.
//
// Objects keep their keys in insertion order: a chat completion's tool-call arguments are echoed
// back by clients and re-rendered into the next prompt, and the session's cached prefix stays a
// prefix only if the key order survives the round trip (the reference uses nlohmann's
// ordered_json for the same reason, src/server/toolcall.h:20-26).
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

namespace b2host {

class Json {
 public:
  enum Type { Null, Bool, Int, Float, String, Array, Object };
  using Member = std::pair<std::string, Json>;

  Json() = default;
  Json(std::nullptr_t) {}
  Json(bool b) : t_(Bool), b_(b) {}
  Json(int v) : t_(Int), i_(v) {}
  Json(int64_t v) : t_(Int), i_(v) {}
  Json(uint32_t v) : t_(Int), i_(v) {}
  Json(uint64_t v) : t_(Int), i_((int64_t)v) {}
  Json(double v) : t_(Float), d_(v) {}
  Json(const char* s) : t_(String), s_(s) {}
  Json(std::string s) : t_(String), s_(std::move(s)) {}
  static Json array() { Json j; j.t_ = Array; return j; }
  static Json object() { Json j; j.t_ = Object; return j; }

  Type type() const { return t_; }
  bool is_null() const { return t_ == Null; }
  bool is_bool() const { return t_ == Bool; }
  bool is_number() const { return t_ == Int || t_ == Float; }
  bool is_int() const { return t_ == Int; }
  bool is_string() const { return t_ == String; }
  bool is_array() const { return t_ == Array; }
  bool is_object() const { return t_ == Object; }

  bool as_bool() const { return t_ == Bool ? b_ : (t_ == Int ? i_ != 0 : false); }
  int64_t as_int() const { return t_ == Int ? i_ : (t_ == Float ? (int64_t)d_ : 0); }
  double as_double() const { return t_ == Float ? d_ : (t_ == Int ? (double)i_ : 0.0); }
  const std::string& as_string() const { return s_; }
  const std::vector<Json>& items() const { return a_; }
  std::vector<Json>& items() { return a_; }
  const std::vector<Member>& members() const { return o_; }
  size_t size() const { return t_ == Array ? a_.size() : (t_ == Object ? o_.size() : 0); }

  void push_back(Json v) {
    if (t_ == Null) t_ = Array;
    a_.push_back(std::move(v));
  }
  const Json* find(const std::string& k) const {
    if (t_ != Object) return nullptr;
    for (const auto& m : o_)
      if (m.first == k) return &m.second;
    return nullptr;
  }
  bool contains(const std::string& k) const { return find(k) != nullptr; }
  const Json& at(const std::string& k) const {
    const Json* p = find(k);
    if (!p) throw std::out_of_range("missing key: " + k);
    return *p;
  }
  Json& operator[](const std::string& k) {
    if (t_ == Null) t_ = Object;
    for (auto& m : o_)
      if (m.first == k) return m.second;
    o_.emplace_back(k, Json());
    return o_.back().second;
  }
  const Json& operator[](size_t i) const { return a_.at(i); }

  // ---------------------------------------------------------------- dump
  std::string dump() const {
    std::string out;
    write(out);
    return out;
  }
  static void escape(const std::string& s, std::string& out) {
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
            out.push_back((char)c);
          }
      }
    }
    out.push_back('"');
  }
  void write(std::string& out) const {
    switch (t_) {
      case Null: out += "null"; break;
      case Bool: out += b_ ? "true" : "false"; break;
      case Int: out += std::to_string(i_); break;
      case Float: {
        if (!std::isfinite(d_)) { out += "null"; break; }
        char buf[40];
        snprintf(buf, sizeof buf, "%.17g", d_);
        // shortest representation that round-trips
        for (int prec = 1; prec < 17; ++prec) {
          char b2[40];
          snprintf(b2, sizeof b2, "%.*g", prec, d_);
          if (strtod(b2, nullptr) == d_) { snprintf(buf, sizeof buf, "%s", b2); break; }
        }
        out += buf;
        if (std::string(buf).find_first_of(".eE") == std::string::npos) out += ".0";  // stays a float on re-parse
        break;
      }
      case String: escape(s_, out); break;
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
          escape(o_[i].first, out);
          out.push_back(':');
          o_[i].second.write(out);
        }
        out.push_back('}');
        break;
    }
  }

  // ---------------------------------------------------------------- parse
  static Json parse(const std::string& text) {
    size_t pos = 0;
    Json v = parse_value(text, pos, 0);
    skip_ws(text, pos);
    if (pos != text.size()) throw std::invalid_argument("JSON: trailing characters at offset " + std::to_string(pos));
    return v;
  }
  static bool try_parse(const std::string& text, Json& out) {
    try {
      out = parse(text);
      return true;
    } catch (const std::exception&) {
      return false;
    }
  }

 private:
  static void skip_ws(const std::string& s, size_t& p) {
    while (p < s.size() && (s[p] == ' ' || s[p] == '\n' || s[p] == '\r' || s[p] == '\t')) ++p;
  }
  [[noreturn]] static void fail(const char* what, size_t p) {
    throw std::invalid_argument(std::string("JSON: ") + what + " at offset " + std::to_string(p));
  }
  static void put_utf8(uint32_t cp, std::string& out) {
    if (cp < 0x80) out.push_back((char)cp);
    else if (cp < 0x800) { out.push_back((char)(0xC0 | (cp >> 6))); out.push_back((char)(0x80 | (cp & 0x3F))); }
    else if (cp < 0x10000) {
      out.push_back((char)(0xE0 | (cp >> 12))); out.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
      out.push_back((char)(0x80 | (cp & 0x3F)));
    } else {
      out.push_back((char)(0xF0 | (cp >> 18))); out.push_back((char)(0x80 | ((cp >> 12) & 0x3F)));
      out.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out.push_back((char)(0x80 | (cp & 0x3F)));
    }
  }
  static uint32_t hex4(const std::string& s, size_t& p) {
    if (p + 4 > s.size()) fail("short \\u escape", p);
    uint32_t v = 0;
    for (int i = 0; i < 4; ++i) {
      const char c = s[p++];
      v <<= 4;
      if (c >= '0' && c <= '9') v |= c - '0';
      else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
      else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
      else fail("bad \\u escape", p);
    }
    return v;
  }
  static std::string parse_string(const std::string& s, size_t& p) {
    std::string out;
    ++p;  // opening quote
    for (;;) {
      if (p >= s.size()) fail("unterminated string", p);
      const unsigned char c = s[p++];
      if (c == '"') return out;
      if (c < 0x20) fail("raw control character in string", p - 1);
      if (c != '\\') { out.push_back((char)c); continue; }
      if (p >= s.size()) fail("unterminated escape", p);
      const char e = s[p++];
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
          uint32_t cp = hex4(s, p);
          if (cp >= 0xD800 && cp < 0xDC00 && p + 1 < s.size() && s[p] == '\\' && s[p + 1] == 'u') {
            p += 2;
            const uint32_t lo = hex4(s, p);
            cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
          }
          put_utf8(cp, out);
          break;
        }
        default: fail("bad escape", p - 1);
      }
    }
  }
  static Json parse_value(const std::string& s, size_t& p, int depth) {
    if (depth > 200) fail("nesting too deep", p);
    skip_ws(s, p);
    if (p >= s.size()) fail("unexpected end", p);
    const char c = s[p];
    if (c == '{') {
      Json o = object();
      ++p;
      skip_ws(s, p);
      if (p < s.size() && s[p] == '}') { ++p; return o; }
      for (;;) {
        skip_ws(s, p);
        if (p >= s.size() || s[p] != '"') fail("expected a key", p);
        std::string k = parse_string(s, p);
        skip_ws(s, p);
        if (p >= s.size() || s[p] != ':') fail("expected ':'", p);
        ++p;
        Json v = parse_value(s, p, depth + 1);
        o[k] = std::move(v);
        skip_ws(s, p);
        if (p < s.size() && s[p] == ',') { ++p; continue; }
        if (p < s.size() && s[p] == '}') { ++p; return o; }
        fail("expected ',' or '}'", p);
      }
    }
    if (c == '[') {
      Json a = array();
      ++p;
      skip_ws(s, p);
      if (p < s.size() && s[p] == ']') { ++p; return a; }
      for (;;) {
        a.a_.push_back(parse_value(s, p, depth + 1));
        skip_ws(s, p);
        if (p < s.size() && s[p] == ',') { ++p; continue; }
        if (p < s.size() && s[p] == ']') { ++p; return a; }
        fail("expected ',' or ']'", p);
      }
    }
    if (c == '"') return Json(parse_string(s, p));
    if (s.compare(p, 4, "true") == 0) { p += 4; return Json(true); }
    if (s.compare(p, 5, "false") == 0) { p += 5; return Json(false); }
    if (s.compare(p, 4, "null") == 0) { p += 4; return Json(); }
    // number
    const size_t b = p;
    if (p < s.size() && (s[p] == '-' || s[p] == '+')) ++p;
    bool is_float = false, digits = false;
    while (p < s.size()) {
      const char d = s[p];
      if (d >= '0' && d <= '9') { digits = true; ++p; }
      else if (d == '.' || d == 'e' || d == 'E' || d == '-' || d == '+') { is_float = true; ++p; }
      else break;
    }
    if (!digits) fail("unexpected character", b);
    const std::string num = s.substr(b, p - b);
    if (!is_float) {
      errno = 0;
      const long long v = strtoll(num.c_str(), nullptr, 10);
      if (errno == 0) return Json((int64_t)v);
    }
    return Json(strtod(num.c_str(), nullptr));
  }

  Type t_ = Null;
  bool b_ = false;
  int64_t i_ = 0;
  double d_ = 0;
  std::string s_;
  std::vector<Json> a_;
  std::vector<Member> o_;
};

}  // namespace b2host
