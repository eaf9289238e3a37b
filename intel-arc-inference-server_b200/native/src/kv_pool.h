// Paged-KV page pool: host free list, reference counts, per-sequence page tables.
//
// Same contract as the reference's KvPool (src/runtime/kv_pool.h:24-85) with 16-token pages:
// pages come from a free list, a page shared by several sequences (a cached prefix) is
// reference counted and returns to the free list when its last holder lets go.  Page 0 is
// never handed out: unused block-table entries point at it, so a kernel that follows a stale
// entry reads the zero page and never another sequence's keys.
#pragma once
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

namespace b2host {

class KvPool {
 public:
  KvPool(int num_pages, int max_seqs, int max_blocks)
      : num_pages_(num_pages), max_seqs_(max_seqs), max_blocks_(max_blocks), ref_(num_pages, 0), tables_(max_seqs) {
    if (num_pages < 2) throw std::invalid_argument("KvPool needs at least 2 pages (page 0 is reserved)");
    free_.reserve(num_pages);
    for (int p = num_pages - 1; p >= 1; --p) free_.push_back(p);  // pop_back hands out 1, 2, 3, ...
  }

  int free_pages() const { return (int)free_.size(); }
  int num_pages() const { return num_pages_; }
  int max_blocks() const { return max_blocks_; }
  const std::vector<int>& table(int seq) const { return tables_.at(seq); }
  int refcount(int page) const { return ref_.at(page); }

  // Grow seq's table to n_blocks pages.  Returns true when the table changed.
  bool ensure(int seq, int n_blocks) {
    auto& t = tables_.at(seq);
    if (n_blocks > max_blocks_)
      throw std::length_error("sequence needs " + std::to_string(n_blocks) + " pages, table holds " +
                              std::to_string(max_blocks_));
    if ((int)t.size() >= n_blocks) return false;
    const int need = n_blocks - (int)t.size();
    if (need > (int)free_.size())
      throw std::runtime_error("KV pool exhausted: need " + std::to_string(need) + " pages, " +
                               std::to_string(free_.size()) + " free");
    for (int i = 0; i < need; ++i) {
      const int p = free_.back();
      free_.pop_back();
      ref_[p] = 1;
      t.push_back(p);
    }
    return true;
  }

  void truncate(int seq, int n_blocks) {
    auto& t = tables_.at(seq);
    while ((int)t.size() > n_blocks) {
      unref(t.back());
      t.pop_back();
    }
  }
  void release(int seq) { truncate(seq, 0); }

  // dst starts with the first n_blocks pages of src (prefix reuse between live sequences)
  void share(int src, int dst, int n_blocks) {
    release(dst);
    const auto& s = tables_.at(src);
    auto& d = tables_.at(dst);
    for (int i = 0; i < n_blocks && i < (int)s.size(); ++i) {
      ++ref_[s[i]];
      d.push_back(s[i]);
    }
  }
  // append pages that something else (the prefix cache) already holds
  void adopt(int seq, const std::vector<int>& pages) {
    auto& t = tables_.at(seq);
    if ((int)(t.size() + pages.size()) > max_blocks_) throw std::length_error("adopt: table overflow");
    for (int p : pages) {
      if (p <= 0 || p >= num_pages_ || ref_[p] == 0) throw std::invalid_argument("adopt: page is not live");
      ++ref_[p];
      t.push_back(p);
    }
  }
  void pin(int page) {
    if (page <= 0 || page >= num_pages_ || ref_[page] == 0) throw std::invalid_argument("pin: page is not live");
    ++ref_[page];
  }
  void unpin(int page) { unref(page); }

 private:
  void unref(int p) {
    if (p <= 0 || p >= num_pages_ || ref_[p] <= 0) throw std::logic_error("KvPool: unref of a free page");
    if (--ref_[p] == 0) free_.push_back(p);
  }
  int num_pages_, max_seqs_, max_blocks_;
  std::vector<int> free_, ref_;
  std::vector<std::vector<int>> tables_;
};

}  // namespace b2host
