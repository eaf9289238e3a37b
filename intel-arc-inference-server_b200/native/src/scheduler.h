// Continuous-batching scheduler: the state machine of slots and waiting requests.
//
// One tick, as in the reference (src/server/scheduler.cc:988 `tick`; scheduler.h:1-311):
// cancellations first, then grants of free slots to waiting requests (a request goes to the
// slot that holds the longest prefix of its prompt when there is one), then at most one prefill
// chunk per engine, then one decode / speculative step over every row that is generating, within
// the row budget.  The scheduler decides; the caller runs the plan on its engine and reports
// what happened (prefill_done / tokens / fail).  A failure fails only the rows of that slot.
#pragma once
#include <algorithm>
#include <cstdint>
#include <deque>
#include <map>
#include <stdexcept>
#include <vector>

namespace b2host {

struct SchedOptions {
  int max_slots = 1;
  int max_queue = 4;          // waiting requests beyond this are refused (HTTP 503)
  int prefill_chunk = 4096;   // prompt positions ingested per tick
  int row_budget = 64;        // rows of one decode / verify step over all slots
  bool interleave = true;     // decode steps run between the prefill chunks of a long prompt
};

struct SchedAction {
  enum Kind { Release = 0, Grant = 1, Prefill = 2, Decode = 3, Reject = 4 };
  int kind = Decode;
  uint64_t req = 0;
  int slot = -1;
  int begin = 0, end = 0;        // Prefill: prompt positions [begin, end)
  bool last = false;             // Prefill: this chunk ends the prompt
  std::vector<int> slots;        // Decode: slots that take part
  std::vector<int> rows;         // Decode: rows granted to each of them (1 + drafts)
};

class Scheduler {
 public:
  explicit Scheduler(const SchedOptions& o) : o_(o), slots_(o.max_slots) {
    if (o.max_slots < 1) throw std::invalid_argument("max_slots must be at least 1");
  }

  // false: the queue is full, answer 503
  bool submit(uint64_t req, int prompt_len, int max_new, int preferred_slot = -1, int want_rows = 1) {
    if ((int)waiting_.size() >= o_.max_queue) return false;
    Waiting w;
    w.req = req; w.prompt_len = prompt_len; w.max_new = max_new; w.preferred = preferred_slot; w.seq = ++seq_;
    w.want_rows = std::max(1, want_rows);
    waiting_.push_back(w);
    return true;
  }
  void cancel(uint64_t req) {
    for (auto it = waiting_.begin(); it != waiting_.end(); ++it)
      if (it->req == req) {
        waiting_.erase(it);
        return;
      }
    for (auto& s : slots_)
      if (s.state != Free && s.req == req) s.cancelled = true;
  }
  int waiting() const { return (int)waiting_.size(); }
  int active() const {
    int n = 0;
    for (const auto& s : slots_) n += s.state != Free;
    return n;
  }
  bool idle() const { return waiting_.empty() && active() == 0; }
  int slot_of(uint64_t req) const {
    for (int i = 0; i < (int)slots_.size(); ++i)
      if (slots_[i].state != Free && slots_[i].req == req) return i;
    return -1;
  }
  // positions of the prompt that are already in the slot (prefix cache hit): prefill starts there
  void set_cached(int slot, int cached) { slots_.at(slot).prefilled = std::min(cached, slots_.at(slot).prompt_len - 1); }
  void set_rows(int slot, int rows) { slots_.at(slot).want_rows = std::max(1, rows); }

  std::vector<SchedAction> tick() {
    std::vector<SchedAction> plan;
    // 1. cancellations
    for (int i = 0; i < (int)slots_.size(); ++i) {
      Slot& s = slots_[i];
      if (s.state != Free && (s.cancelled || s.done)) {
        SchedAction a;
        a.kind = SchedAction::Release; a.slot = i; a.req = s.req;
        plan.push_back(a);
        s = Slot();
      }
    }
    // 2. grants (arrival order; a preferred slot is honoured when it is free)
    while (!waiting_.empty()) {
      const Waiting w = waiting_.front();
      int slot = -1;
      if (w.preferred >= 0 && w.preferred < (int)slots_.size() && slots_[w.preferred].state == Free) slot = w.preferred;
      for (int i = 0; slot < 0 && i < (int)slots_.size(); ++i)
        if (slots_[i].state == Free) slot = i;
      if (slot < 0) break;
      waiting_.pop_front();
      Slot& s = slots_[slot];
      s.state = Prefilling; s.req = w.req; s.prompt_len = w.prompt_len; s.max_new = w.max_new; s.seq = w.seq;
      s.want_rows = w.want_rows;
      SchedAction a;
      a.kind = SchedAction::Grant; a.slot = slot; a.req = w.req;
      plan.push_back(a);
    }
    // 3. at most one prefill chunk: the oldest prompt that is still being ingested
    int pf = -1;
    for (int i = 0; i < (int)slots_.size(); ++i)
      if (slots_[i].state == Prefilling && !slots_[i].busy && (pf < 0 || slots_[i].seq < slots_[pf].seq)) pf = i;
    bool any_decode = false;
    for (const auto& s : slots_) any_decode |= s.state == Decoding;
    if (pf >= 0) {
      Slot& s = slots_[pf];
      SchedAction a;
      a.kind = SchedAction::Prefill; a.slot = pf; a.req = s.req; a.begin = s.prefilled;
      a.end = std::min(s.prompt_len, s.prefilled + o_.prefill_chunk);
      a.last = a.end == s.prompt_len;
      s.busy = true;
      plan.push_back(a);
    }
    // 4. one decode step over the generating rows, within the row budget (oldest first)
    if (any_decode && (o_.interleave || pf < 0)) {
      std::vector<int> order;
      for (int i = 0; i < (int)slots_.size(); ++i)
        if (slots_[i].state == Decoding) order.push_back(i);
      std::sort(order.begin(), order.end(), [&](int a, int b) { return slots_[a].seq < slots_[b].seq; });
      SchedAction a;
      a.kind = SchedAction::Decode;
      int budget = o_.row_budget;
      // every slot gets its first row before anyone gets draft rows
      for (int i : order) {
        if (budget <= 0) break;
        a.slots.push_back(i);
        a.rows.push_back(1);
        --budget;
      }
      for (size_t k = 0; k < a.slots.size() && budget > 0; ++k) {
        const int extra = std::min(budget, slots_[a.slots[k]].want_rows - 1);
        a.rows[k] += extra;
        budget -= extra;
      }
      if (!a.slots.empty()) plan.push_back(a);
    }
    return plan;
  }

  // ---- reports from the caller
  void prefill_done(int slot, int end) {
    Slot& s = slots_.at(slot);
    s.busy = false;
    s.prefilled = end;
    if (end >= s.prompt_len) {
      s.state = Decoding;
      s.generated = 1;  // the prompt pass yields the first token
      if (s.generated >= s.max_new) s.done = true;
    }
  }
  // n new tokens were emitted for the slot; finished: EOS / stop / length reached
  void tokens(int slot, int n, bool finished) {
    Slot& s = slots_.at(slot);
    s.generated += n;
    if (finished || s.generated >= s.max_new) s.done = true;
  }
  void fail(int slot) { slots_.at(slot).done = true; }

 private:
  enum State { Free = 0, Prefilling = 1, Decoding = 2 };
  struct Slot {
    int state = Free;
    uint64_t req = 0;
    int prompt_len = 0, prefilled = 0, generated = 0, max_new = 0, want_rows = 1;
    uint64_t seq = 0;
    bool cancelled = false, done = false, busy = false;
  };
  struct Waiting {
    uint64_t req, seq;
    int prompt_len, max_new, preferred, want_rows;
  };
  SchedOptions o_;
  std::vector<Slot> slots_;
  std::deque<Waiting> waiting_;
  uint64_t seq_ = 0;
};

}  // namespace b2host
