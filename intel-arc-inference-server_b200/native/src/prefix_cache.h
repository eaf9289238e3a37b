// Prefix cache index: a tree of fixed-size token blocks whose KV lives in device pages and / or in
// pinned host slots.
//
// The reference keeps a tree of 2048-position KV blocks plus recurrent-state snapshots in pinned
// host RAM, keyed by a hash chain with an exact id compare, with LRU leaf eviction, pinning and
// Cold / Continue / Restore plans (src/server/prefix_cache.h:1-205, prefix_cache.cc:158-478).
// For the attention-only models served here the state part vanishes: a block is just the KV pages
// of `block_tokens` positions.  Two tiers: a block may hold references to device pages of the
// page pool (a hit costs nothing: the pages are adopted into the new sequence's table) and / or a
// slot of the pinned host store (a hit costs one H2D copy per block).  This class is the index
// and the policy only; the copies are done by the caller.
#pragma once
#include <cstdint>
#include <map>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

namespace b2host {

class PrefixCache {
 public:
  enum Kind { Cold = 0, Continue = 1, Restore = 2 };
  struct Plan {
    int kind = Cold;
    int matched_tokens = 0;      // positions whose KV need not be computed
    int resident_tokens = 0;     // of those, already in the slot (Continue)
    std::vector<int> path;       // nodes of the matched chain, root side first
  };
  struct Node {
    int parent = -1;
    std::vector<uint32_t> ids;
    std::vector<int> device_pages;
    int host_slot = -1;
    int pins = 0;
    int children = 0;
    int device_children = 0;
    uint64_t last_use = 0;
    bool live = false;
    uint64_t hash = 0;
  };

  explicit PrefixCache(int block_tokens) : block_(block_tokens) {
    if (block_tokens < 16 || block_tokens % 16) throw std::invalid_argument("block_tokens must be a multiple of 16");
  }
  int block_tokens() const { return block_; }
  int num_nodes() const { return live_; }
  const Node& node(int id) const { return nodes_.at(id); }

  // A root per cache form (KV dtype, drafter identity): blocks of different forms never mix.
  int root(const std::string& key) {
    auto it = roots_.find(key);
    if (it != roots_.end()) return it->second;
    const int id = alloc();
    nodes_[id].live = true;
    nodes_[id].pins = 1;  // roots are never evicted
    roots_[key] = id;
    return id;
  }

  // Longest chain of whole blocks under `root` that equals a prefix of ids[0 .. limit).
  std::vector<int> match(int root, const std::vector<uint32_t>& ids, int limit) {
    std::vector<int> path;
    int cur = root;
    const int nblk = std::min<int>(limit, (int)ids.size()) / block_;
    for (int b = 0; b < nblk; ++b) {
      const uint32_t* p = ids.data() + (size_t)b * block_;
      const int child = find_child(cur, p);
      if (child < 0) break;
      path.push_back(child);
      cur = child;
    }
    ++tick_;
    for (int n : path) nodes_[n].last_use = tick_;
    return path;
  }

  // The plan for a prompt arriving on a slot that already holds `resident` ids (its previous
  // request): Continue when the slot's own prefix is at least as long as the stored match.
  // `split_last` keeps one position out of the match so the prompt's last token is always run.
  Plan plan(int root, const std::vector<uint32_t>& prompt, const std::vector<uint32_t>& resident, bool split_last) {
    Plan pl;
    const int n = (int)prompt.size();
    // the last prompt token is always run (its logits are needed); split_last keeps one more position out
    const int limit = split_last ? n - 2 : n - 1;
    int common = 0;
    while (common < (int)resident.size() && common < limit && resident[common] == prompt[common]) ++common;
    pl.path = match(root, prompt, std::max(0, limit));
    const int stored = (int)pl.path.size() * block_;
    if (common >= stored && common > 0) {
      pl.kind = Continue;
      pl.matched_tokens = common;
      pl.resident_tokens = common;
      pl.path.clear();
    } else if (stored > 0) {
      pl.kind = Restore;
      pl.matched_tokens = stored;
    }
    return pl;
  }

  // Insert a block under `parent`.  Returns (node id, created).  An existing equal child is
  // returned untouched (created = false): the caller keeps ownership of its pages.
  std::pair<int, bool> insert(int parent, const std::vector<uint32_t>& block_ids, const std::vector<int>& device_pages) {
    if ((int)block_ids.size() != block_) throw std::invalid_argument("insert: block has the wrong length");
    if (!nodes_.at(parent).live) throw std::invalid_argument("insert: parent is not live");
    const int ex = find_child(parent, block_ids.data());
    if (ex >= 0) {
      nodes_[ex].last_use = ++tick_;
      return {ex, false};
    }
    const int id = alloc();
    Node& nd = nodes_[id];
    nd.parent = parent;
    nd.ids = block_ids;
    nd.device_pages = device_pages;
    nd.live = true;
    nd.last_use = ++tick_;
    nd.hash = hash_ids(block_ids.data());
    children_[key(parent, nd.hash)].push_back(id);
    nodes_[parent].children++;
    if (!device_pages.empty()) nodes_[parent].device_children++;
    ++live_;
    return {id, true};
  }

  void pin(int id) { nodes_.at(id).pins++; }
  void unpin(int id) {
    if (--nodes_.at(id).pins < 0) throw std::logic_error("unpin below zero");
  }
  void set_host_slot(int id, int slot) { nodes_.at(id).host_slot = slot; }
  void set_device_pages(int id, const std::vector<int>& pages) {
    Node& nd = nodes_.at(id);
    const bool had = !nd.device_pages.empty();
    nd.device_pages = pages;
    const bool has = !pages.empty();
    if (nd.parent >= 0 && had != has) nodes_[nd.parent].device_children += has ? 1 : -1;
  }

  // Least recently used unpinned block that holds device pages and whose children hold none
  // (so chains shrink from the leaf side); -1 when there is none.
  int device_victim() const {
    int best = -1;
    for (int i = 0; i < (int)nodes_.size(); ++i) {
      const Node& nd = nodes_[i];
      if (!nd.live || nd.pins || nd.device_pages.empty() || nd.device_children) continue;
      if (best < 0 || nd.last_use < nodes_[best].last_use) best = i;
    }
    return best;
  }
  // Least recently used unpinned leaf (no children at all): removing it frees its host slot.
  int leaf_victim() const {
    int best = -1;
    for (int i = 0; i < (int)nodes_.size(); ++i) {
      const Node& nd = nodes_[i];
      if (!nd.live || nd.pins || nd.children || nd.parent < 0) continue;
      if (best < 0 || nd.last_use < nodes_[best].last_use) best = i;
    }
    return best;
  }
  // Remove a leaf; returns (device pages, host slot) the caller must release.
  std::pair<std::vector<int>, int> remove(int id) {
    Node& nd = nodes_.at(id);
    if (!nd.live || nd.children || nd.pins || nd.parent < 0) throw std::logic_error("remove: not an unpinned leaf");
    auto& v = children_[key(nd.parent, nd.hash)];
    for (size_t i = 0; i < v.size(); ++i)
      if (v[i] == id) {
        v.erase(v.begin() + i);
        break;
      }
    if (v.empty()) children_.erase(key(nd.parent, nd.hash));
    nodes_[nd.parent].children--;
    if (!nd.device_pages.empty()) nodes_[nd.parent].device_children--;
    std::pair<std::vector<int>, int> out{nd.device_pages, nd.host_slot};
    nd = Node();
    free_ids_.push_back(id);
    --live_;
    return out;
  }

 private:
  int alloc() {
    if (!free_ids_.empty()) {
      const int id = free_ids_.back();
      free_ids_.pop_back();
      return id;
    }
    nodes_.emplace_back();
    return (int)nodes_.size() - 1;
  }
  uint64_t hash_ids(const uint32_t* p) const {
    uint64_t h = 0xcbf29ce484222325ull;
    for (int i = 0; i < block_; ++i) {
      h ^= p[i];
      h *= 0x100000001b3ull;
      h ^= h >> 29;
    }
    return h;
  }
  static uint64_t key(int parent, uint64_t h) { return h ^ (uint64_t(parent) * 0x9E3779B97F4A7C15ull); }
  int find_child(int parent, const uint32_t* p) const {
    const uint64_t h = hash_ids(p);
    auto it = children_.find(key(parent, h));
    if (it == children_.end()) return -1;
    for (int c : it->second) {
      const Node& nd = nodes_[c];
      if (nd.parent != parent || nd.hash != h) continue;
      bool eq = true;
      for (int i = 0; i < block_ && eq; ++i) eq = nd.ids[i] == p[i];  // the hash is a hint, the ids decide
      if (eq) return c;
    }
    return -1;
  }

  int block_;
  std::vector<Node> nodes_;
  std::vector<int> free_ids_;
  std::unordered_map<uint64_t, std::vector<int>> children_;
  std::map<std::string, int> roots_;
  uint64_t tick_ = 0;
  int live_ = 0;
};

}  // namespace b2host
