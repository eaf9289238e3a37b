// Byte-level BPE tokenizer (the Hugging Face "tokenizer.json" of GPT-2 / Qwen style models),
// detokenizer and hold-and-flush streamer.
//
// The reference links the Rust `tokenizers` crate behind a C ABI (src/tokenizer/rs/src/lib.rs:1-60,
// b70_tok.h:14-41) and streams text with a detokeniser that never emits half a UTF-8 character
// (src/tokenizer/streamer.h:13-27).  Here the same pipeline is native C++: added (special) tokens
// are split off first, the rest is cut by a hand-written scanner that implements the Qwen / GPT-4
// style pre-tokenisation pattern
//   (?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,D}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+
// bytes are mapped to the printable alphabet of GPT-2, and merges are applied by rank.
// Truncation and padding do not exist here (the reference disables them too).
#pragma once
#include <algorithm>
#include <cstdint>
#include <fstream>
#include <map>
#include <sstream>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "json.h"
#include "unicode_tables.h"

namespace b2host {

namespace uni {
inline bool in_ranges(const uint32_t (*r)[2], int n, uint32_t cp) {
  int lo = 0, hi = n - 1;
  while (lo <= hi) {
    const int mid = (lo + hi) / 2;
    if (cp < r[mid][0]) hi = mid - 1;
    else if (cp > r[mid][1]) lo = mid + 1;
    else return true;
  }
  return false;
}
inline bool is_letter(uint32_t cp) { return in_ranges(kLetter, kLetter_n, cp); }
inline bool is_number(uint32_t cp) { return in_ranges(kNumber, kNumber_n, cp); }
inline bool is_space(uint32_t cp) {  // \s of the regex engines the pattern was written for (Unicode White_Space)
  return (cp >= 9 && cp <= 13) || cp == 0x20 || cp == 0x85 || cp == 0xA0 || cp == 0x1680 ||
         (cp >= 0x2000 && cp <= 0x200A) || cp == 0x2028 || cp == 0x2029 || cp == 0x202F || cp == 0x205F || cp == 0x3000;
}
inline void append_utf8(uint32_t cp, std::string& out) {
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
// decode UTF-8 leniently: an invalid byte becomes U+FFFD and is consumed alone
inline void decode_utf8(const std::string& s, std::vector<uint32_t>& cps, std::vector<uint32_t>& offs) {
  size_t i = 0;
  while (i < s.size()) {
    const unsigned char c = s[i];
    uint32_t cp = 0xFFFD;
    int len = 1;
    if (c < 0x80) cp = c;
    else if ((c & 0xE0) == 0xC0 && i + 1 < s.size()) { cp = ((c & 0x1F) << 6) | (s[i + 1] & 0x3F); len = 2; }
    else if ((c & 0xF0) == 0xE0 && i + 2 < s.size()) {
      cp = ((c & 0x0F) << 12) | ((s[i + 1] & 0x3F) << 6) | (s[i + 2] & 0x3F); len = 3;
    } else if ((c & 0xF8) == 0xF0 && i + 3 < s.size()) {
      cp = ((c & 0x07) << 18) | ((s[i + 1] & 0x3F) << 12) | ((s[i + 2] & 0x3F) << 6) | (s[i + 3] & 0x3F); len = 4;
    }
    cps.push_back(cp);
    offs.push_back((uint32_t)i);
    i += len;
  }
  offs.push_back((uint32_t)s.size());
}
}  // namespace uni

class Tokenizer {
 public:
  Tokenizer() { build_byte_maps(); }

  static Tokenizer from_file(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("cannot open " + path);
    std::stringstream ss;
    ss << f.rdbuf();
    return from_json(ss.str());
  }
  static Tokenizer from_json(const std::string& text) {
    Tokenizer t;
    const Json j = Json::parse(text);
    const Json& model = j.at("model");
    for (const auto& m : model.at("vocab").members()) t.add_vocab(m.first, (uint32_t)m.second.as_int());
    uint32_t rank = 0;
    for (const Json& mg : model.at("merges").items()) {
      std::string a, b;
      if (mg.is_string()) {
        const std::string& s = mg.as_string();
        const size_t sp = s.find(' ');
        a = s.substr(0, sp);
        b = s.substr(sp + 1);
      } else {
        a = mg[0].as_string();
        b = mg[1].as_string();
      }
      t.merges_[a + " " + b] = rank++;
    }
    if (const Json* added = j.find("added_tokens"))
      for (const Json& a : added->items()) {
        const std::string& content = a.at("content").as_string();
        const uint32_t id = (uint32_t)a.at("id").as_int();
        const Json* sp = a.find("special");
        t.add_special(content, id, sp && sp->as_bool());
      }
    // digit run length of the pattern: \p{N} (Qwen) or \p{N}{1,3} (Llama-3 / GPT-4)
    const std::string dump = j.contains("pre_tokenizer") ? j.at("pre_tokenizer").dump() : "";
    t.digits_max_ = dump.find("{1,3}") != std::string::npos ? 3 : 1;
    return t;
  }

  void add_vocab(const std::string& tok, uint32_t id) {
    vocab_[tok] = id;
    if (id >= id_to_tok_.size()) id_to_tok_.resize(id + 1);
    id_to_tok_[id] = tok;
  }
  void add_special(const std::string& content, uint32_t id, bool special) {
    added_[content] = id;
    if (id >= id_to_tok_.size()) id_to_tok_.resize(id + 1);
    id_to_tok_[id] = content;
    if (id >= is_added_.size()) is_added_.resize(id + 1, 0);
    is_added_[id] = special ? 2 : 1;
    added_sorted_.clear();
  }
  size_t vocab_size() const { return id_to_tok_.size(); }
  int token_to_id(const std::string& tok) const {
    auto a = added_.find(tok);
    if (a != added_.end()) return (int)a->second;
    auto v = vocab_.find(tok);
    return v == vocab_.end() ? -1 : (int)v->second;
  }

  // ---------------------------------------------------------------- encode
  std::vector<uint32_t> encode(const std::string& text) const {
    std::vector<uint32_t> out;
    if (added_sorted_.empty() && !added_.empty()) {
      for (const auto& a : added_) added_sorted_.push_back(a.first);
      std::sort(added_sorted_.begin(), added_sorted_.end(),
                [](const std::string& x, const std::string& y) { return x.size() > y.size(); });
    }
    size_t pos = 0, seg = 0;
    while (pos < text.size()) {
      bool hit = false;
      if (!added_sorted_.empty()) {
        for (const std::string& a : added_sorted_) {
          if (text.compare(pos, a.size(), a) == 0) {
            if (pos > seg) encode_plain(text.substr(seg, pos - seg), out);
            out.push_back(added_.at(a));
            pos += a.size();
            seg = pos;
            hit = true;
            break;
          }
        }
      }
      if (!hit) ++pos;
    }
    if (seg < text.size()) encode_plain(text.substr(seg), out);
    return out;
  }

  // ---------------------------------------------------------------- decode
  // raw bytes of one token (added tokens are their literal text)
  std::string token_bytes(uint32_t id) const {
    if (id >= id_to_tok_.size()) return std::string();
    const std::string& tok = id_to_tok_[id];
    if (id < is_added_.size() && is_added_[id]) return tok;
    std::string out;
    std::vector<uint32_t> cps, offs;
    uni::decode_utf8(tok, cps, offs);
    for (uint32_t cp : cps) {
      auto it = cp_to_byte_.find(cp);
      if (it != cp_to_byte_.end()) out.push_back((char)it->second);
      else uni::append_utf8(cp, out);
    }
    return out;
  }
  bool is_special(uint32_t id) const { return id < is_added_.size() && is_added_[id] == 2; }
  std::string decode(const std::vector<uint32_t>& ids, bool skip_special = false) const {
    std::string out;
    for (uint32_t id : ids) {
      if (skip_special && is_special(id)) continue;
      out += token_bytes(id);
    }
    return out;
  }

  // pieces of the pre-tokenisation pattern (exposed for tests)
  std::vector<std::string> pre_tokenize(const std::string& text) const {
    std::vector<uint32_t> cps, offs;
    uni::decode_utf8(text, cps, offs);
    std::vector<std::string> out;
    size_t i = 0;
    const size_t n = cps.size();
    auto L = [&](size_t k) { return k < n && uni::is_letter(cps[k]); };
    auto N = [&](size_t k) { return k < n && uni::is_number(cps[k]); };
    auto S = [&](size_t k) { return k < n && uni::is_space(cps[k]); };
    auto NL = [&](size_t k) { return k < n && (cps[k] == '\r' || cps[k] == '\n'); };
    auto lower = [&](size_t k) -> uint32_t { return (cps[k] >= 'A' && cps[k] <= 'Z') ? cps[k] + 32 : cps[k]; };
    while (i < n) {
      size_t end = i;
      // 1. contractions
      if (cps[i] == '\'' && i + 1 < n) {
        const uint32_t c1 = lower(i + 1);
        if (c1 == 's' || c1 == 't' || c1 == 'm' || c1 == 'd') end = i + 2;
        else if (i + 2 < n) {
          const uint32_t c2 = lower(i + 2);
          if ((c1 == 'r' && c2 == 'e') || (c1 == 'v' && c2 == 'e') || (c1 == 'l' && c2 == 'l')) end = i + 3;
        }
      }
      // 2. [^\r\n\p{L}\p{N}]?\p{L}+
      if (end == i) {
        size_t k = i;
        if (!NL(k) && !L(k) && !N(k) && L(k + 1)) ++k;
        if (L(k)) {
          while (L(k)) ++k;
          end = k;
        }
      }
      // 3. \p{N}{1,D}
      if (end == i && N(i)) {
        size_t k = i;
        while (k < i + (size_t)digits_max_ && N(k)) ++k;
        end = k;
      }
      // 4.  ?[^\s\p{L}\p{N}]+[\r\n]*
      if (end == i) {
        size_t k = i;
        if (cps[k] == ' ' && k + 1 < n && !S(k + 1) && !L(k + 1) && !N(k + 1)) ++k;
        if (k < n && !S(k) && !L(k) && !N(k)) {
          while (k < n && !S(k) && !L(k) && !N(k)) ++k;
          while (NL(k)) ++k;
          end = k;
        }
      }
      if (end == i && S(i)) {
        size_t k = i;
        while (S(k)) ++k;  // the whole whitespace run [i, k)
        // 5. \s*[\r\n]+ : up to and including the last newline of the run
        size_t last_nl = n;
        for (size_t q = i; q < k; ++q)
          if (NL(q)) last_nl = q;
        if (last_nl != n) end = last_nl + 1;
        // 6. \s+(?!\S): all but the last character when something follows the run
        else if (k == n) end = k;
        else if (k - i >= 2) end = k - 1;
        // 7. \s+
        else end = k;
      }
      if (end == i) end = i + 1;  // cannot happen; never loop forever
      out.push_back(text.substr(offs[i], offs[end] - offs[i]));
      i = end;
    }
    return out;
  }

 private:
  void build_byte_maps() {
    // GPT-2's bytes_to_unicode: printable bytes map to themselves, the rest to 256, 257, ...
    int n = 0;
    for (int b = 0; b < 256; ++b) {
      const bool keep = (b >= '!' && b <= '~') || (b >= 0xA1 && b <= 0xAC) || (b >= 0xAE && b <= 0xFF);
      const uint32_t cp = keep ? (uint32_t)b : 256u + n++;
      std::string s;
      uni::append_utf8(cp, s);
      byte_to_str_[b] = s;
      cp_to_byte_[cp] = (uint8_t)b;
    }
  }
  void encode_plain(const std::string& text, std::vector<uint32_t>& out) const {
    for (const std::string& piece : pre_tokenize(text)) {
      auto c = cache_.find(piece);
      if (c != cache_.end()) {
        out.insert(out.end(), c->second.begin(), c->second.end());
        continue;
      }
      std::vector<std::string> sym;
      for (unsigned char b : piece) sym.push_back(byte_to_str_[b]);
      bpe(sym);
      std::vector<uint32_t> ids;
      for (const std::string& s : sym) {
        auto v = vocab_.find(s);
        if (v != vocab_.end()) ids.push_back(v->second);
        else {  // unknown symbol: fall back to its bytes' tokens where they exist
          std::vector<uint32_t> cps, offs;
          uni::decode_utf8(s, cps, offs);
          for (uint32_t cp : cps) {
            std::string one;
            uni::append_utf8(cp, one);
            auto v1 = vocab_.find(one);
            if (v1 != vocab_.end()) ids.push_back(v1->second);
          }
        }
      }
      if (cache_.size() < 200000) cache_[piece] = ids;
      out.insert(out.end(), ids.begin(), ids.end());
    }
  }
  void bpe(std::vector<std::string>& sym) const {
    while (sym.size() > 1) {
      uint32_t best = 0xFFFFFFFFu;
      size_t at = 0;
      for (size_t i = 0; i + 1 < sym.size(); ++i) {
        auto it = merges_.find(sym[i] + " " + sym[i + 1]);
        if (it != merges_.end() && it->second < best) {
          best = it->second;
          at = i;
        }
      }
      if (best == 0xFFFFFFFFu) return;
      // merge every occurrence of that pair, left to right
      const std::string a = sym[at], b = sym[at + 1];
      std::vector<std::string> next;
      for (size_t i = 0; i < sym.size(); ++i) {
        if (i + 1 < sym.size() && sym[i] == a && sym[i + 1] == b) {
          next.push_back(a + b);
          ++i;
        } else {
          next.push_back(sym[i]);
        }
      }
      sym.swap(next);
    }
  }

  std::unordered_map<std::string, uint32_t> vocab_, merges_;
  std::map<std::string, uint32_t> added_;
  mutable std::vector<std::string> added_sorted_;
  std::vector<std::string> id_to_tok_;
  std::vector<uint8_t> is_added_;
  std::string byte_to_str_[256];
  std::unordered_map<uint32_t, uint8_t> cp_to_byte_;
  mutable std::unordered_map<std::string, std::vector<uint32_t>> cache_;
  int digits_max_ = 1;
};

// Incremental detokeniser: bytes of an unfinished UTF-8 character are held until the character is
// complete, so a streamed delta never carries U+FFFD for a character split across tokens.
class Streamer {
 public:
  explicit Streamer(const Tokenizer* tok, bool skip_special = true) : tok_(tok), skip_special_(skip_special) {}
  std::string push(uint32_t id) {
    if (skip_special_ && tok_->is_special(id)) return std::string();
    held_ += tok_->token_bytes(id);
    // longest prefix that ends on a character boundary
    size_t cut = held_.size();
    size_t back = 0;
    while (back < 4 && back < held_.size()) {
      const unsigned char c = held_[held_.size() - 1 - back];
      if ((c & 0xC0) == 0x80) { ++back; continue; }  // continuation byte
      int need = 1;
      if ((c & 0xE0) == 0xC0) need = 2;
      else if ((c & 0xF0) == 0xE0) need = 3;
      else if ((c & 0xF8) == 0xF0) need = 4;
      if ((size_t)need > back + 1) cut = held_.size() - 1 - back;  // the last character is incomplete
      break;
    }
    std::string out = held_.substr(0, cut);
    held_.erase(0, cut);
    return out;
  }
  std::string finish() {
    std::string out;
    out.swap(held_);
    return out;
  }

 private:
  const Tokenizer* tok_;
  bool skip_special_;
  std::string held_;
};

}  // namespace b2host
