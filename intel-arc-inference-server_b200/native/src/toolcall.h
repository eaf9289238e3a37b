// Incremental parser of generated chat text: reasoning, content and tool calls.
//
// Two call syntaxes, as in the reference (src/server/toolcall.h:17-118, toolcall_kolibri.h):
//   Qwen XML   <tool_call>\n<function=NAME>\n<parameter=KEY>\nVALUE\n</parameter>\n...</function>\n</tool_call>
//   hermes     <tool_call>\n{"name": NAME, "arguments": {...}}\n</tool_call>
// With thinking on the prompt ends in "<think>\n", so the output up to "</think>" is reasoning.
// The stream property holds: the concatenated deltas of any split of a text equal the deltas of
// the whole text; only a suffix that may still become a tag is held back.  A call still open when
// generation ends is dropped (never executed with half its parameters) unless its </function> had
// closed.  Parameter values are converted by the tool's JSON schema: a parameter the schema types
// as a string stays a string, anything else is parsed as JSON when it parses.
#pragma once
#include <cstdint>
#include <cstdio>
#include <random>
#include <string>
#include <vector>

#include "json.h"

namespace b2host {

struct ToolCall {
  std::string id;
  std::string name;
  Json arguments = Json::object();
};

struct Delta {
  enum Kind { Reasoning = 0, Content = 1, Call = 2 };
  int kind = Content;
  std::string text;
  ToolCall call;
  uint32_t index = 0;
};

// longest suffix of s that is a proper prefix of tag
inline size_t tag_prefix_suffix(const std::string& s, const std::string& tag) {
  const size_t maxn = std::min(s.size(), tag.size() - 1);
  for (size_t n = maxn; n > 0; --n)
    if (s.compare(s.size() - n, n, tag, 0, n) == 0) return n;
  return 0;
}

inline std::string make_call_id(uint64_t seed, uint32_t index) {
  uint64_t x = seed + 0x9E3779B97F4A7C15ull * (index + 1);
  char buf[40];
  std::string out = "call_";
  for (int i = 0; i < 2; ++i) {
    x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull; x ^= x >> 27; x *= 0x94D049BB133111EBull; x ^= x >> 31;
    snprintf(buf, sizeof buf, "%012llx", (unsigned long long)(x & 0xFFFFFFFFFFFFull));
    out += buf;
  }
  return out;  // "call_" + 24 hex chars
}
inline uint64_t new_call_seed() {
  std::random_device rd;
  return (uint64_t(rd()) << 32) ^ rd();
}

// 1: the schema types `key` of `function` as a string (or string | null); 0: another type; -1: unknown
inline int schema_string_type(const std::string& function, const std::string& key, const Json& tools) {
  if (!tools.is_array()) return -1;
  for (const Json& t : tools.items()) {
    const Json* fn = t.find("function");
    if (!fn) fn = &t;
    const Json* name = fn->find("name");
    if (!name || !name->is_string() || name->as_string() != function) continue;
    const Json* params = fn->find("parameters");
    if (!params) return -1;
    const Json* props = params->find("properties");
    if (!props) return -1;
    const Json* p = props->find(key);
    if (!p) return -1;
    const Json* ty = p->find("type");
    if (!ty) return -1;
    if (ty->is_string()) return ty->as_string() == "string" ? 1 : 0;
    if (ty->is_array()) {
      bool has_string = false, other = false;
      for (const Json& e : ty->items()) {
        if (!e.is_string()) continue;
        if (e.as_string() == "string") has_string = true;
        else if (e.as_string() != "null") other = true;
      }
      return has_string && !other ? 1 : 0;
    }
    return -1;
  }
  return -1;
}

inline Json convert_value(const std::string& value, const std::string& function, const std::string& key,
                          const Json& tools) {
  const int st = schema_string_type(function, key, tools);
  if (st == 1) return Json(value);
  Json parsed;
  if (Json::try_parse(value, parsed)) {
    if (st == -1 && parsed.is_string()) return Json(value);  // untyped: keep the text as written
    return parsed;
  }
  return Json(value);
}

// Escape raw control bytes inside JSON string literals (models write multi-line string arguments
// with raw newlines).  False when nothing was escaped or the text ends inside a literal.
inline bool escape_raw_controls(const std::string& text, std::string& out) {
  out.clear();
  bool in_str = false, changed = false;
  for (size_t i = 0; i < text.size(); ++i) {
    const unsigned char c = text[i];
    if (!in_str) {
      out.push_back((char)c);
      if (c == '"') in_str = true;
      continue;
    }
    if (c == '\\') {
      out.push_back((char)c);
      if (i + 1 < text.size()) out.push_back(text[++i]);
      continue;
    }
    if (c == '"') {
      in_str = false;
      out.push_back('"');
      continue;
    }
    if (c < 0x20) {
      changed = true;
      switch (c) {
        case '\n': out += "\\n"; break;
        case '\r': out += "\\r"; break;
        case '\t': out += "\\t"; break;
        case '\b': out += "\\b"; break;
        case '\f': out += "\\f"; break;
        default: {
          char buf[8];
          snprintf(buf, sizeof buf, "\\u%04x", c);
          out += buf;
        }
      }
      continue;
    }
    out.push_back((char)c);
  }
  return changed && !in_str;
}

inline std::string trim(const std::string& s) {
  size_t a = 0, b = s.size();
  while (a < b && (s[a] == ' ' || s[a] == '\n' || s[a] == '\r' || s[a] == '\t')) ++a;
  while (b > a && (s[b - 1] == ' ' || s[b - 1] == '\n' || s[b - 1] == '\r' || s[b - 1] == '\t')) --b;
  return s.substr(a, b - a);
}

// hermes call body: {"name": <string>, "arguments": <object | string holding an object | null | absent>}
inline bool parse_json_call(const std::string& body, const Json& tools, ToolCall& call) {
  Json j;
  const std::string t = trim(body);
  if (!Json::try_parse(t, j)) {
    std::string fixed;
    if (!escape_raw_controls(t, fixed) || !Json::try_parse(fixed, j)) return false;
  }
  if (!j.is_object()) return false;
  const Json* name = j.find("name");
  if (!name || !name->is_string() || name->as_string().empty() ||
      name->as_string().find_first_of(" \n\t\r") != std::string::npos)
    return false;
  Json args = Json::object();
  if (const Json* a = j.find("arguments")) {
    if (a->is_object()) args = *a;
    else if (a->is_string()) {
      Json inner;
      std::string fixed;
      if (Json::try_parse(a->as_string(), inner) && inner.is_object()) args = inner;
      else if (escape_raw_controls(a->as_string(), fixed) && Json::try_parse(fixed, inner) && inner.is_object()) args = inner;
      else return false;
    } else if (!a->is_null()) return false;
  }
  call.name = name->as_string();
  call.arguments = Json::object();
  for (const auto& m : args.members()) {
    if (!m.second.is_string() && schema_string_type(call.name, m.first, tools) == 1)
      call.arguments[m.first] = Json(m.second.dump());  // typed as a string, written as another value
    else
      call.arguments[m.first] = m.second;
  }
  return true;
}

// Qwen XML call body (between <tool_call> and </tool_call>); `closed` reports whether </function> was seen
inline bool parse_xml_call(const std::string& body, const Json& tools, ToolCall& call, bool* closed) {
  const size_t f = body.find("<function=");
  if (f == std::string::npos) return false;
  const size_t fe = body.find('>', f);
  if (fe == std::string::npos) return false;
  call.name = trim(body.substr(f + 10, fe - f - 10));
  if (call.name.empty()) return false;
  call.arguments = Json::object();
  size_t pos = fe + 1;
  const size_t fclose = body.find("</function>", pos);
  if (closed) *closed = fclose != std::string::npos;
  const size_t end = fclose == std::string::npos ? body.size() : fclose;
  for (;;) {
    const size_t p = body.find("<parameter=", pos);
    if (p == std::string::npos || p >= end) break;
    const size_t pe = body.find('>', p);
    if (pe == std::string::npos || pe >= end) break;
    const std::string key = trim(body.substr(p + 11, pe - p - 11));
    const size_t pc = body.find("</parameter>", pe + 1);
    if (pc == std::string::npos || pc > end) break;  // a parameter that never closed is not part of the call
    std::string val = body.substr(pe + 1, pc - pe - 1);
    if (!val.empty() && val.front() == '\n') val.erase(0, 1);
    if (!val.empty() && val.back() == '\n') val.pop_back();
    call.arguments[key] = convert_value(val, call.name, key, tools);
    pos = pc + 12;
  }
  return true;
}

class OutputStream {
 public:
  enum Format { QwenXml = 0, Hermes = 1 };
  OutputStream(bool thinking, Json tools, int format = QwenXml, uint64_t seed = 0)
      : state_(thinking ? St::Reasoning : St::Body), tools_(std::move(tools)), format_(format),
        seed_(seed ? seed : new_call_seed()) {}
  void set_drop_cut_calls(bool on) { drop_cut_ = on; }

  std::vector<Delta> push(const std::string& piece) {
    buf_ += piece;
    std::vector<Delta> out;
    run(out, false);
    return out;
  }
  std::vector<Delta> finish() {
    std::vector<Delta> out;
    run(out, true);
    return out;
  }

 private:
  enum class St { Reasoning, Body, Call };
  static constexpr const char* kThinkEnd = "</think>";
  static constexpr const char* kCallOpen = "<tool_call>";
  static constexpr const char* kCallClose = "</tool_call>";

  void emit_text(std::vector<Delta>& out, int kind, const std::string& text) {
    if (text.empty()) return;
    if (!out.empty() && out.back().kind == kind) out.back().text += text;
    else {
      Delta d;
      d.kind = kind;
      d.text = text;
      out.push_back(std::move(d));
    }
  }
  // text of a reasoning / content segment: leading whitespace of the segment is dropped, trailing
  // whitespace is held until more text shows it is interior
  void segment_text(std::vector<Delta>& out, int kind, std::string text) {
    if (!seg_started_) {
      size_t a = 0;
      while (a < text.size() && (text[a] == ' ' || text[a] == '\n' || text[a] == '\r' || text[a] == '\t')) ++a;
      text.erase(0, a);
      if (text.empty()) return;
      seg_started_ = true;
    }
    text = held_ws_ + text;
    held_ws_.clear();
    size_t b = text.size();
    while (b > 0 && (text[b - 1] == ' ' || text[b - 1] == '\n' || text[b - 1] == '\r' || text[b - 1] == '\t')) --b;
    held_ws_ = text.substr(b);
    text.erase(b);
    emit_text(out, kind, text);
  }
  void end_segment() {
    held_ws_.clear();
    seg_started_ = false;
  }
  void run(std::vector<Delta>& out, bool final) {
    for (;;) {
      if (state_ == St::Reasoning) {
        const size_t e = buf_.find(kThinkEnd);
        if (e != std::string::npos) {
          segment_text(out, Delta::Reasoning, buf_.substr(0, e));
          end_segment();
          buf_.erase(0, e + 8);
          state_ = St::Body;
          continue;
        }
        const size_t hold = final ? 0 : tag_prefix_suffix(buf_, kThinkEnd);
        segment_text(out, Delta::Reasoning, buf_.substr(0, buf_.size() - hold));
        buf_.erase(0, buf_.size() - hold);
        return;
      }
      if (state_ == St::Body) {
        const size_t o = tools_.is_null() ? std::string::npos : buf_.find(kCallOpen);
        if (o != std::string::npos) {
          segment_text(out, Delta::Content, buf_.substr(0, o));
          end_segment();
          buf_.erase(0, o + 11);
          state_ = St::Call;
          continue;
        }
        const size_t hold = (final || tools_.is_null()) ? 0 : tag_prefix_suffix(buf_, kCallOpen);
        segment_text(out, Delta::Content, buf_.substr(0, buf_.size() - hold));
        buf_.erase(0, buf_.size() - hold);
        return;
      }
      // inside a call
      const size_t c = buf_.find(kCallClose);
      if (c == std::string::npos && !final) return;
      const std::string body = c == std::string::npos ? buf_ : buf_.substr(0, c);
      ToolCall call;
      bool ok, closed = true;
      if (format_ == Hermes) ok = parse_json_call(body, tools_, call);
      else ok = parse_xml_call(body, tools_, call, &closed);
      const bool cut = c == std::string::npos;
      if (ok && (!cut || (format_ == QwenXml && (closed || !drop_cut_)))) {
        Delta d;
        d.kind = Delta::Call;
        call.id = make_call_id(seed_, calls_);
        d.call = std::move(call);
        d.index = calls_++;
        out.push_back(std::move(d));
      } else if (!ok && !cut) {
        // not a call after all: keep the text as content, tags included
        emit_text(out, Delta::Content, std::string(kCallOpen) + body + kCallClose);
      }
      if (cut) {
        buf_.clear();
        return;
      }
      buf_.erase(0, c + 12);
      state_ = St::Body;
    }
  }

  St state_;
  Json tools_;
  int format_;
  uint64_t seed_;
  std::string buf_, held_ws_;
  bool seg_started_ = false, drop_cut_ = true;
  uint32_t calls_ = 0;
};

struct ParsedOutput {
  std::string reasoning, content;
  std::vector<ToolCall> tool_calls;
};
inline ParsedOutput parse_output(const std::string& text, bool thinking, const Json& tools, int format = 0) {
  OutputStream s(thinking, tools, format, 1);
  ParsedOutput po;
  auto fold = [&](std::vector<Delta> ds) {
    for (auto& d : ds) {
      if (d.kind == Delta::Reasoning) po.reasoning += d.text;
      else if (d.kind == Delta::Content) po.content += d.text;
      else po.tool_calls.push_back(d.call);
    }
  };
  fold(s.push(text));
  fold(s.finish());
  return po;
}

}  // namespace b2host
