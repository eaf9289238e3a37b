// Prompt-lookup proposer: drafts copied from an earlier occurrence of the current context.
//
// Semantics follow the reference's matcher (src/server/prompt_lookup.h:1-125): for the indexed
// sequence s[0..t), an earlier end position e < t-1 matches with length m(e) = the longest
// common suffix of s[0..e] and s[0..t-1], capped at max_match; the proposal takes the e with the
// largest m(e), the most recent among equals, only when m(e) >= min_n, and copies s[e+1], ...
// forward, continuing from its own drafts when the copy reaches the end (an overlapping LZ77
// copy).  A boundary() id is unique, so neither a match nor a continuation crosses it.
//
// Implementation: one polynomial prefix hash over the ids (so the hash of any window is two
// multiplications) and, per key length in {2,4,8,16,32,64}, an open hash table "window hash ->
// most recent end" with a per-position back link to the previous end in the same bucket.
// append is O(1) amortised (tables double at 50 % load); match walks the chain of the longest
// key length that has a verified candidate.
#pragma once
#include <cstdint>
#include <stdexcept>
#include <vector>

namespace b2host {

class PromptLookup {
 public:
  static constexpr uint32_t kNone = 0xFFFFFFFFu;
  static constexpr uint32_t kBoundaryFloor = 0xFFF00000u;
  static constexpr int kLevels = 6;
  static constexpr uint32_t kLen[kLevels] = {2, 4, 8, 16, 32, 64};

  struct Match {
    uint32_t end = kNone;
    uint32_t length = 0;
    uint32_t steps = 0;
    bool truncated = false;
  };

  explicit PromptLookup(uint32_t max_match = 64, uint32_t max_candidates = 64, uint32_t max_steps = 1024)
      : max_match_(max_match), max_cand_(max_candidates), max_steps_(max_steps) {
    if (max_match < 2 || max_match > 64) throw std::invalid_argument("max_match must be in [2, 64]");
    levels_ = 0;
    while (levels_ < kLevels && kLen[levels_] <= max_match) ++levels_;
    uint64_t p = 1;
    int lv = 0;
    for (uint32_t k = 1; k <= 64; ++k) {
      p *= kBase;
      if (lv < kLevels && k == kLen[lv]) pow_[lv++] = p;
    }
    clear();
  }

  void clear() {
    ids_.clear();
    prefix_.assign(1, 0);
    bits_ = 10;
    for (int l = 0; l < kLevels; ++l) {
      head_[l].assign(size_t(1) << bits_, kNone);
      prev_[l].clear();
    }
    next_boundary_ = 0xFFFFFFFFu;
  }

  size_t size() const { return ids_.size(); }
  const std::vector<uint32_t>& ids() const { return ids_; }

  void append(uint32_t id) {
    if (id >= kBoundaryFloor) throw std::invalid_argument("token id collides with the boundary range");
    push(id);
  }
  void append_many(const std::vector<uint32_t>& v) {
    for (uint32_t id : v) append(id);
  }
  void boundary() { push(next_boundary_--); }

  // keep the first n ids
  void truncate(size_t n) {
    while (ids_.size() > n) {
      const uint32_t end = (uint32_t)ids_.size() - 1;
      for (int l = 0; l < levels_; ++l) {
        if (end + 1 < kLen[l]) continue;
        const uint32_t b = bucket(hash(l, end));
        // the removed position is the most recent of its bucket
        if (head_[l][b] == end) head_[l][b] = prev_[l][end];
      }
      for (int l = 0; l < kLevels; ++l) prev_[l].pop_back();
      ids_.pop_back();
      prefix_.pop_back();
    }
  }

  Match match(uint32_t min_n, uint32_t source_before = kNone) const {
    if (min_n < 2 || min_n > max_match_) throw std::invalid_argument("min_n out of range");
    Match best;
    const uint32_t t = (uint32_t)ids_.size();
    if (t < 2) return best;
    const uint32_t last = t - 1;
    for (int l = levels_ - 1; l >= 0; --l) {
      const uint32_t k = kLen[l];
      if (k > t) continue;
      // a level below the largest key length <= min_n can only hold matches shorter than min_n
      if (k < min_n && l + 1 < levels_ && kLen[l + 1] <= min_n) break;
      const uint64_t h = hash(l, last);
      uint32_t e = head_[l][bucket(h)];
      uint32_t cands = 0, steps = 0;
      bool found = false;
      while (e != kNone) {
        if (e != last) {
          if (e + 1 >= source_before) {  // too recent for the caller: skip without spending the caps
            e = prev_[l][e];
            continue;
          }
          ++steps;
          ++best.steps;
          if (hash(l, e) == h && same(e, last, k)) {
            uint32_t m = k;
            while (m < max_match_ && m <= e && ids_[e - m] == ids_[last - m]) ++m;
            if (m >= min_n && (!found || m > best.length)) {
              best.end = e;
              best.length = m;
              found = true;
            } else if (!found && m > best.length) {
              best.length = m;
            }
            if (found && best.length >= max_match_) break;
            if (++cands >= max_cand_) {
              best.truncated = true;
              break;
            }
          }
          if (steps >= max_steps_) {
            best.truncated = true;
            break;
          }
        }
        e = prev_[l][e];
      }
      if (found) return best;
    }
    best.end = kNone;
    return best;
  }

  std::vector<uint32_t> propose(uint32_t max_k, uint32_t min_n, Match* info = nullptr,
                                uint32_t source_before = kNone) const {
    std::vector<uint32_t> out;
    Match m = match(min_n, source_before);
    if (info) *info = m;
    if (m.end == kNone || max_k == 0) return out;
    const uint32_t t = (uint32_t)ids_.size();
    for (uint32_t i = 0; i < max_k; ++i) {
      const uint32_t src = m.end + 1 + i;
      const uint32_t id = src < t ? ids_[src] : out[src - t];
      if (id >= kBoundaryFloor) break;
      out.push_back(id);
    }
    return out;
  }

 private:
  static constexpr uint64_t kBase = 0x9E3779B97F4A7C15ull | 1ull;

  uint64_t hash(int level, uint32_t end) const {  // window of kLen[level] ids ending at `end`
    const uint32_t k = kLen[level];
    return prefix_[end + 1] - prefix_[end + 1 - k] * pow_[level];
  }
  uint32_t bucket(uint64_t h) const { return (uint32_t)((h * 0xD6E8FEB86659FD93ull) >> (64 - bits_)); }
  bool same(uint32_t a, uint32_t b, uint32_t k) const {
    for (uint32_t i = 0; i < k; ++i)
      if (ids_[a - i] != ids_[b - i]) return false;
    return true;
  }
  void insert(int l, uint32_t end) {
    const uint32_t b = bucket(hash(l, end));
    prev_[l][end] = head_[l][b];
    head_[l][b] = end;
  }
  void push(uint32_t id) {
    ids_.push_back(id);
    prefix_.push_back(prefix_.back() * kBase + (uint64_t(id) + 0x1234567ull));
    const uint32_t end = (uint32_t)ids_.size() - 1;
    for (int l = 0; l < kLevels; ++l) prev_[l].push_back(kNone);
    if (ids_.size() * 2 > (size_t(1) << bits_)) {
      rebuild(bits_ + 1);
      return;
    }
    for (int l = 0; l < levels_; ++l)
      if (end + 1 >= kLen[l]) insert(l, end);
  }
  void rebuild(uint32_t bits) {
    bits_ = bits;
    for (int l = 0; l < levels_; ++l) {
      head_[l].assign(size_t(1) << bits_, kNone);
      for (uint32_t end = kLen[l] - 1; end < ids_.size(); ++end) insert(l, end);
    }
  }

  uint32_t max_match_, max_cand_, max_steps_;
  int levels_;
  std::vector<uint32_t> ids_;
  std::vector<uint64_t> prefix_;
  uint64_t pow_[kLevels];
  uint32_t bits_;
  std::vector<uint32_t> head_[kLevels], prev_[kLevels];
  uint32_t next_boundary_;
};

// Lookup inside a block drafter (reference: src/server/lookup_in_dflash.h:1-102): the copy proposer
// takes over from the learned drafter when the context has a long enough earlier occurrence, and
// widens the verify as the copy keeps being accepted.
//   enter: match length >= 8;  stay: >= 3;  verify width escalates 16 -> 32 -> 64 after each fully
//   accepted copy step and falls back to 16 on a rejection.
class LookupPolicy {
 public:
  static constexpr uint32_t kEnter = 8, kStay = 3;
  bool active() const { return active_; }
  uint32_t width() const { return width_; }
  // match length of the current context -> should this step be a copy step, and how wide?
  uint32_t decide(uint32_t match_len) {
    if (!active_) {
      if (match_len >= kEnter) {
        active_ = true;
        width_ = 16;
      }
    } else if (match_len < kStay) {
      active_ = false;
      width_ = 16;
    }
    return active_ ? width_ : 0;
  }
  void observe(uint32_t proposed, uint32_t accepted) {
    if (!active_) return;
    if (proposed > 0 && accepted == proposed) {
      if (width_ < 64) width_ *= 2;
    } else {
      width_ = 16;
      if (accepted == 0) active_ = false;
    }
  }

 private:
  bool active_ = false;
  uint32_t width_ = 16;
};

}  // namespace b2host
