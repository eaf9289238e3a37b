// Copy proposer ("prompt lookup"): drafts taken from an earlier place where the text already read like it does now.
//
// Behaviour (what the reference's matcher promises, src/server/prompt_lookup.h:1-125): over the sequence seen so
// far, an earlier position e matches with length m(e) = number of trailing symbols that e and the current end have
// in common (capped at `max_match`); the proposer picks the e with the largest m(e), the most recent one among
// equals, if m(e) >= min_n, and copies what followed e -- continuing into its own output when the copy runs into
// the present (the overlapping copy of LZ77).  A separator never equals anything, so no match or copy crosses it.
//
// How it is built here.  Symbols are 64-bit: a token id keeps its value, a separator is 2^32 + serial, so no range of
// ids has to be reserved.  Two indexes over "the n symbols that end at position i" give candidates:
//   * pairs (n = 2): an open-addressing table keyed by the EXACT pair; every position with m(e) >= 2 is on the chain
//     of the current pair;
//   * octets (n = 8): the same, keyed by a 64-bit mix of eight symbols; every position with m(e) >= 8 is on the
//     chain of the current octet (entries are confirmed by comparison, the key being a hash).
// Chains run from the most recent position backwards through one link word per position and index.  A query walks
// the octet chain first: if any position matches 8 or more symbols, the longest match is on that chain; otherwise
// the pair chain decides.  Walks are bounded by a candidate cap and a step cap (the result then says `truncated`).
// Appending is O(1) amortised (tables double at half load), removing the tail is O(1) per symbol because the
// newest position is always the head of its chains.
#pragma once
#include <cstdint>
#include <stdexcept>
#include <vector>

namespace b2host {

class PromptLookup {
 public:
  static constexpr uint32_t kNone = 0xFFFFFFFFu;
  static constexpr uint32_t kIdLimit = 0x80000000u;   // token ids are non-negative 32-bit integers
  static constexpr uint32_t kSeparatorId = 0xFFFFFFFFu;   // what ids() shows at a separator

  struct Match {
    uint32_t end = kNone;     // matched earlier position (the copy starts after it)
    uint32_t length = 0;      // symbols in common (the best seen, even when below min_n)
    uint32_t steps = 0;       // chain entries visited
    bool truncated = false;   // a cap ended the walk: a longer or more recent match may exist
  };

  explicit PromptLookup(uint32_t max_match = 64, uint32_t max_candidates = 64, uint32_t max_steps = 1024)
      : longest_(max_match), cand_cap_(max_candidates), step_cap_(max_steps) {
    if (max_match < 2 || max_match > 64) throw std::invalid_argument("max_match must be in [2, 64]");
    clear();
  }

  void clear() {
    sym_.clear();
    shown_.clear();
    link2_.clear();
    link8_.clear();
    pairs_.reset(8);
    octets_.reset(8);
    separators_ = 0;
  }

  size_t size() const { return sym_.size(); }
  const std::vector<uint32_t>& ids() const { return shown_; }

  void append(uint32_t id) {
    if (id >= kIdLimit) throw std::invalid_argument("token id out of range (ids are below 2^31)");
    push(uint64_t(id), id);
  }
  void append_many(const std::vector<uint32_t>& v) {
    for (uint32_t id : v) append(id);
  }
  void boundary() { push((uint64_t(1) << 32) + separators_++, kSeparatorId); }

  // keep the first n symbols
  void truncate(size_t n) {
    while (sym_.size() > n) {
      const uint32_t i = uint32_t(sym_.size() - 1);
      if (i >= 1) pairs_.unlink(pair_key(i), i, link2_[i]);
      if (i >= 7) octets_.unlink(octet_key(i), i, link8_[i]);
      sym_.pop_back();
      shown_.pop_back();
      link2_.pop_back();
      link8_.pop_back();
    }
  }

  // `source_before`: only positions e with e + 1 < source_before may be proposed from (kNone: any)
  Match match(uint32_t min_n, uint32_t source_before = kNone) const {
    if (min_n < 2 || min_n > longest_) throw std::invalid_argument("min_n out of range");
    Match r;
    const uint32_t n = uint32_t(sym_.size());
    if (n < 2) return r;
    const uint32_t cur = n - 1;
    bool found = false;
    if (n >= 8 && longest_ >= 8) {
      walk(octets_.find(octet_key(cur)), link8_, 8, cur, min_n, source_before, r, found);
      if (found) return r;
      if (r.truncated && min_n >= 8) return r;
    }
    if (min_n < 8 || longest_ < 8) {
      // no position shares 8 symbols (or the index is not in use): every match of 2..7 is on the pair chain
      walk(pairs_.find(pair_key(cur)), link2_, 2, cur, min_n, source_before, r, found);
    }
    if (!found) r.end = kNone;
    return r;
  }

  std::vector<uint32_t> propose(uint32_t max_k, uint32_t min_n, Match* info = nullptr,
                                uint32_t source_before = kNone) const {
    std::vector<uint32_t> out;
    const Match m = match(min_n, source_before);
    if (info) *info = m;
    if (m.end == kNone) return out;
    const uint32_t n = uint32_t(sym_.size());
    for (uint32_t i = 0; i < max_k; ++i) {
      const uint32_t src = m.end + 1 + i;
      if (src < n) {
        if (sym_[src] >> 32) break;   // a separator ends the copy
        out.push_back(uint32_t(sym_[src]));
      } else {
        out.push_back(out[src - n]);  // the copy has caught up with its own output
      }
    }
    return out;
  }

 private:
  // Open addressing, linear probing: key -> most recent position.  A slot whose chain became empty keeps its key
  // (head = kNone) so that probe sequences stay intact; growth drops such slots.
  struct Table {
    std::vector<uint64_t> key;
    std::vector<uint32_t> head;
    std::vector<uint8_t> used;
    uint32_t bits = 0, filled = 0;
    void reset(uint32_t b) {
      bits = b;
      filled = 0;
      key.assign(size_t(1) << b, 0);
      head.assign(size_t(1) << b, kNone);
      used.assign(size_t(1) << b, 0);
    }
    static uint64_t mix(uint64_t x) {   // the finaliser of splitmix64
      x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull;
      x ^= x >> 27; x *= 0x94D049BB133111EBull;
      return x ^ (x >> 31);
    }
    size_t slot(uint64_t k) const {
      const size_t mask = (size_t(1) << bits) - 1;
      size_t s = size_t(mix(k)) & mask;
      while (used[s] && key[s] != k) s = (s + 1) & mask;
      return s;
    }
    uint32_t find(uint64_t k) const {
      const size_t s = slot(k);
      return used[s] ? head[s] : kNone;
    }
    // position i becomes the head of k's chain; returns the previous head
    uint32_t link(uint64_t k, uint32_t i) {
      const size_t s = slot(k);
      uint32_t before = kNone;
      if (used[s]) before = head[s];
      else {
        used[s] = 1;
        key[s] = k;
        ++filled;
      }
      head[s] = i;
      return before;
    }
    void unlink(uint64_t k, uint32_t i, uint32_t before) {
      const size_t s = slot(k);
      if (used[s] && head[s] == i) head[s] = before;
    }
  };

  uint64_t pair_key(uint32_t i) const {
    // exact for token pairs (two 32-bit ids); a pair with a separator is folded so that it cannot equal a token pair
    const uint64_t a = sym_[i - 1], b = sym_[i];
    if ((a | b) >> 32) return Table::mix(a * 0x9FB21C651E98DF25ull + b) | (uint64_t(1) << 63);
    return ((a << 32) | b) & ~(uint64_t(1) << 63);
  }
  uint64_t octet_key(uint32_t i) const {
    uint64_t h = 0x2545F4914F6CDD1Dull;
    for (uint32_t d = 0; d < 8; ++d) h = Table::mix(h ^ sym_[i - d]);
    return h;
  }
  uint32_t common(uint32_t e, uint32_t cur) const {   // trailing symbols e and cur share, up to longest_
    uint32_t m = 0;
    while (m < longest_ && m <= e && sym_[e - m] == sym_[cur - m]) ++m;
    return m;
  }
  void walk(uint32_t e, const std::vector<uint32_t>& links, uint32_t floor, uint32_t cur, uint32_t min_n,
            uint32_t source_before, Match& r, bool& found) const {
    uint32_t cands = 0, steps = 0;
    for (; e != kNone; e = links[e]) {
      if (e == cur) continue;
      if (source_before != kNone && e + 1 >= source_before) continue;   // too recent for the caller: free of charge
      ++steps;
      ++r.steps;
      const uint32_t m = common(e, cur);
      if (m >= floor) {   // a real member of the chain (hashed keys can collide)
        if (m >= min_n && (!found || m > r.length)) {   // most recent first: only a longer match replaces
          r.end = e;
          r.length = m;
          found = true;
          if (m >= longest_) return;
        } else if (!found && m > r.length) {
          r.length = m;
        }
        if (++cands >= cand_cap_) {
          r.truncated = true;
          return;
        }
      }
      if (steps >= step_cap_) {
        r.truncated = true;
        return;
      }
    }
  }
  void push(uint64_t s, uint32_t shown) {
    sym_.push_back(s);
    shown_.push_back(shown);
    link2_.push_back(kNone);
    link8_.push_back(kNone);
    const uint32_t i = uint32_t(sym_.size() - 1);
    if (2 * size_t(pairs_.filled + 1) > (size_t(1) << pairs_.bits) || 2 * size_t(octets_.filled + 1) > (size_t(1) << octets_.bits)) {
      regrow();
      return;   // regrow indexed position i too
    }
    if (i >= 1) link2_[i] = pairs_.link(pair_key(i), i);
    if (i >= 7) link8_[i] = octets_.link(octet_key(i), i);
  }
  void regrow() {
    pairs_.reset(pairs_.bits + 1);
    octets_.reset(octets_.bits + 1);
    for (uint32_t i = 0; i < sym_.size(); ++i) {
      link2_[i] = i >= 1 ? pairs_.link(pair_key(i), i) : kNone;
      link8_[i] = i >= 7 ? octets_.link(octet_key(i), i) : kNone;
    }
  }

  uint32_t longest_, cand_cap_, step_cap_;
  std::vector<uint64_t> sym_;
  std::vector<uint32_t> shown_;
  std::vector<uint32_t> link2_, link8_;
  Table pairs_, octets_;
  uint64_t separators_ = 0;
};

// When a block drafter and the copy proposer are both present, this decides which of them drafts the next step.
// Behaviour asked for (the reference's lookup-in-DFlash rule, src/server/lookup_in_dflash.h:58-100): the copy
// proposer takes over once the context repeats an earlier stretch of at least eight tokens, keeps the turn while
// at least three still match, asks for a 16-row verify first and doubles it (32, then 64) every time a whole copy was
// accepted; any rejection brings the width back to 16, and a copy of which nothing was accepted hands the turn back.
class LookupPolicy {
 public:
  bool active() const { return copying_; }
  uint32_t width() const { return rows_; }
  // longest match of the current context -> rows of the copy step to run now (0: let the learned drafter draft)
  uint32_t decide(uint32_t match_len) {
    const uint32_t needed = copying_ ? 3u : 8u;
    if (match_len >= needed) {
      if (!copying_) rows_ = 16;
      copying_ = true;
    } else {
      copying_ = false;
      rows_ = 16;
    }
    return copying_ ? rows_ : 0;
  }
  void observe(uint32_t proposed, uint32_t accepted) {
    if (!copying_) return;
    if (proposed > 0 && accepted >= proposed) {
      rows_ = rows_ >= 64 ? 64 : rows_ * 2;
      return;
    }
    rows_ = 16;
    if (accepted == 0) copying_ = false;
  }

 private:
  bool copying_ = false;
  uint32_t rows_ = 16;
};

}  // namespace b2host
