// How many drafts to spend: per request (DraftLengthPolicy) and per step (ConfidenceStop).
//
// What these policies are for (the reference keeps an adaptive K per request and a per-step stop rule driven by the
// draft head's confidence: src/server/adaptive_k.h:100-134, src/server/step_k.h:54-85): a speculative iteration with
// k drafts costs draft(k) + verify(k + 1 rows) and yields 1 + (accepted drafts) tokens, so the best k depends on how
// often drafts are accepted; below some acceptance the plain step wins and speculation should pause, with an
// occasional probe to notice when the text becomes predictable again.
//
// Design here.  Costs are a table measured on the machine the server runs on (StepCosts; `bench.py --what spec`
// prints the B200 table that the defaults below were taken from, the CLI measures again at start-up).  The
// per-request policy keeps one acceptance estimate PER DRAFT POSITION (draft i is only tested when drafts 0..i-1 were
// accepted, and later positions of a head are less reliable than the first), as exponentially forgotten hit / trial
// counts started from a prior.  The expected yield of k drafts is 1 + a0 + a0 a1 + ... (k terms); the policy moves to
// the k with the best yield per cost when that beats the current k by a margin, and while it sits at k = 0 it probes
// with one draft after a waiting time that doubles while probes keep failing.  The per-step rule turns the head's
// stated probability into an acceptance probability with a small online logistic model per position (two weights,
// trained on every draft that was actually tested) and stops drafting when one more draft is not expected to pay.
#pragma once
#include <algorithm>
#include <array>
#include <cmath>
#include <cstdint>
#include <vector>

namespace b2host {

// Iteration costs in units of one plain decode step (one row, no drafts).
struct StepCosts {
  std::vector<double> verify_rows;   // [m - 1]: one trunk step over m rows; verify_rows[0] == 1 by definition
  std::vector<double> draft_depth;   // [k - 1]: producing k drafts with the draft head
  // 27B shape on one B200, depth 4096: multi-row steps stream the same weights as one row, a draft pass runs
  // one extra decoder layer and the head over a 32k-id draft vocabulary
  StepCosts() : verify_rows{1.00, 1.02, 1.04, 1.05, 1.07, 1.08, 1.10, 1.11}, draft_depth{0.11, 0.22, 0.33, 0.44, 0.55, 0.66, 0.77} {}
  StepCosts(std::vector<double> v, std::vector<double> d) : verify_rows(std::move(v)), draft_depth(std::move(d)) {}
  uint32_t deepest() const {   // most drafts both tables cover
    if (verify_rows.empty()) return 0;
    return (uint32_t)std::min(verify_rows.size() - 1, draft_depth.size());
  }
  double iteration(uint32_t k) const { return k == 0 ? 1.0 : verify_rows.at(k) + draft_depth.at(k - 1); }
  // drafts that cost nothing to produce (copied from the context): only the wider verify is paid
  StepCosts free_drafts() const {
    StepCosts c = *this;
    std::fill(c.draft_depth.begin(), c.draft_depth.end(), 0.0);
    c.draft_depth.resize(c.verify_rows.empty() ? 0 : c.verify_rows.size() - 1, 0.0);
    return c;
  }
};

struct DraftLengthOptions {
  uint32_t deepest = 3;          // never more drafts than this
  double prior_accept = 0.75;    // acceptance assumed before anything was seen ...
  double prior_trials = 3.0;     // ... with the weight of this many trials
  double forget = 0.92;          // weight of the past per observation of a position
  uint32_t settle = 2;           // first iterations always draft `deepest` (the estimates need data)
  double switch_margin = 0.04;   // move to another k only for this relative gain
  uint32_t probe_wait = 4;       // plain steps before the first probe; doubles after each failed probe ...
  uint32_t probe_wait_max = 48;  // ... up to this
  StepCosts costs;
};

class DraftLengthPolicy {
 public:
  explicit DraftLengthPolicy(const DraftLengthOptions& o = {})
      : opt_(o), deepest_(std::min(o.deepest, o.costs.deepest())), depth_(deepest_), wait_(o.probe_wait) {
    pos_.assign(std::max<uint32_t>(deepest_, 1), Estimate{o.prior_accept * o.prior_trials, o.prior_trials});
  }
  uint32_t deepest() const { return deepest_; }
  uint32_t current() const { return depth_; }
  // acceptance estimate of draft position i (0 = the first draft)
  double acceptance(uint32_t i) const {
    const Estimate& e = pos_[std::min<size_t>(i, pos_.size() - 1)];
    return e.trials > 0 ? e.hits / e.trials : 0.0;
  }
  // tokens an iteration with k drafts is expected to emit
  double expected_tokens(uint32_t k) const {
    double total = 1.0, chain = 1.0;
    for (uint32_t i = 0; i < k; ++i) {
      chain *= acceptance(i);
      total += chain;
    }
    return total;
  }
  double tokens_per_cost(uint32_t k) const { return expected_tokens(k) / opt_.costs.iteration(k); }
  uint32_t best_depth() const {
    uint32_t best = 0;
    for (uint32_t k = 1; k <= deepest_; ++k)
      if (tokens_per_cost(k) > tokens_per_cost(best)) best = k;
    return best;
  }
  // drafts to spend on the next iteration
  uint32_t next() const {
    if (deepest_ == 0) return 0;
    if (seen_ < opt_.settle) return deepest_;
    if (depth_ == 0 && idle_ >= wait_) return 1;
    return depth_;
  }
  // an iteration ran with k drafts of which `accepted` were kept
  void observe(uint32_t k, uint32_t accepted) {
    ++seen_;
    const bool probing = depth_ == 0 && k > 0;
    const uint32_t tested = std::min<uint32_t>(k, accepted + 1);   // the first rejected draft was tested, the rest not
    for (uint32_t i = 0; i < tested && i < pos_.size(); ++i) {
      pos_[i].hits = pos_[i].hits * opt_.forget + (i < accepted ? 1.0 : 0.0);
      pos_[i].trials = pos_[i].trials * opt_.forget + 1.0;
    }
    if (seen_ >= opt_.settle && deepest_ > 0) {
      const uint32_t want = best_depth();
      if (want != depth_ && tokens_per_cost(want) > tokens_per_cost(depth_) * (1.0 + opt_.switch_margin)) depth_ = want;
    }
    if (depth_ > 0) {
      idle_ = 0;
      wait_ = opt_.probe_wait;
    } else if (k == 0) {
      ++idle_;
    } else {
      idle_ = 0;
      if (probing) wait_ = std::min(wait_ * 2, opt_.probe_wait_max);   // the probe did not bring speculation back
    }
  }

 private:
  struct Estimate {
    double hits, trials;
  };
  DraftLengthOptions opt_;
  uint32_t deepest_;
  std::vector<Estimate> pos_;
  uint32_t depth_;
  uint32_t seen_ = 0, idle_ = 0, wait_;
};

// Head confidence -> acceptance probability.  One logistic model per draft position, q = sigmoid(b + w * logit(p)),
// started at the identity (b = 0, w = 1: believe the head) and trained online with one gradient step per tested
// draft.  A head that is over-confident at depth 2 ends with w < 1 or b < 0 there; nothing is binned.
class ConfidenceModel {
 public:
  static constexpr uint32_t kPositions = 8;
  explicit ConfidenceModel(double learning_rate = 0.05) : lr_(learning_rate) {
    for (auto& m : w_) m = {0.0, 1.0};
  }
  static double logit(double p) {
    p = std::min(std::max(p, 1e-4), 1.0 - 1e-4);
    return std::log(p / (1.0 - p));
  }
  double accept_prob(uint32_t i, double p) const {
    const Weights& m = w_[std::min(i, kPositions - 1)];
    return 1.0 / (1.0 + std::exp(-(m.bias + m.slope * logit(p))));
  }
  void learn(uint32_t i, double p, bool accepted) {
    Weights& m = w_[std::min(i, kPositions - 1)];
    const double z = logit(p), err = (accepted ? 1.0 : 0.0) - accept_prob(i, p);
    m.bias += lr_ * err;
    m.slope = std::max(0.0, m.slope + lr_ * err * z * 0.25);   // z spans about +-9: a smaller step keeps the slope calm
  }
  double bias(uint32_t i) const { return w_[std::min(i, kPositions - 1)].bias; }
  double slope(uint32_t i) const { return w_[std::min(i, kPositions - 1)].slope; }

 private:
  struct Weights {
    double bias, slope;
  };
  double lr_;
  std::array<Weights, kPositions> w_;
};

// Per-step rule: after each draft, with the head's probability of that draft in hand, either draft once more or verify now
// (possibly fewer drafts than were made: a weak last draft is cheaper to drop than to verify).
class ConfidenceStop {
 public:
  ConfidenceStop(const StepCosts& costs, uint32_t deepest, ConfidenceModel& model)
      : costs_(costs), model_(model), deepest_(std::min<uint32_t>({deepest, costs.deepest(), ConfidenceModel::kPositions})) {
    typical_.fill(0.75);
  }
  uint32_t deepest() const { return deepest_; }
  uint32_t verified() const { return verify_; }
  // before the first draft of a step: how many drafts may be made at most (0: take a plain step)
  uint32_t begin() {
    made_ = 0;
    verify_ = 0;
    decided_ = false;
    // with no confidence in hand yet, the positions' typical acceptance stands in
    double chain = 1.0, yield = 1.0, best = 1.0;
    uint32_t best_k = 0;
    for (uint32_t k = 1; k <= deepest_; ++k) {
      chain *= typical_[k - 1];
      yield += chain;
      const double r = yield / costs_.iteration(k);
      if (r > best) {
        best = r;
        best_k = k;
      }
    }
    if (best_k == 0 && ++plain_steps_ > 6) {   // look again now and then: one draft is cheap to test
      plain_steps_ = 0;
      best_k = 1;
    }
    limit_ = best_k == 0 ? 0 : deepest_;
    if (limit_ == 0) decided_ = true;
    return limit_;
  }
  // draft number j (1-based) came back with head probability p.  Returns -1: draft another; k >= 0: verify k drafts.
  int after_draft(uint32_t j, double p) {
    made_ = j;
    stated_[j - 1] = p;
    q_[j - 1] = model_.accept_prob(j - 1, p);
    // verify now: best prefix of what was made (all j drafts were paid for either way)
    double chain = 1.0, yield = 1.0, now_rate = 1.0 / (costs_.verify_rows.at(0) + costs_.draft_depth.at(j - 1));
    uint32_t now_k = 0;
    for (uint32_t k = 1; k <= j; ++k) {
      chain *= q_[k - 1];
      yield += chain;
      const double r = yield / (costs_.verify_rows.at(k) + costs_.draft_depth.at(j - 1));
      if (r > now_rate) {
        now_rate = r;
        now_k = k;
      }
    }
    if (j < limit_) {
      // one more draft: its acceptance is guessed from what position j usually reaches
      const double more = (yield + chain * typical_[j]) / (costs_.verify_rows.at(j + 1) + costs_.draft_depth.at(j));
      if (more > now_rate) return -1;
    }
    verify_ = now_k;
    decided_ = true;
    return (int)now_k;
  }
  // the verify kept `accepted` of the verified drafts
  void observe(uint32_t accepted) {
    if (!decided_) verify_ = made_;
    for (uint32_t i = 0; i < verify_; ++i) {
      const bool ok = i < accepted;
      model_.learn(i, stated_[i], ok);
      typical_[i] = 0.9 * typical_[i] + 0.1 * (ok ? 1.0 : 0.0);
      if (!ok) break;   // later drafts were not tested
    }
    if (made_ > 0) plain_steps_ = 0;
  }
  double typical(uint32_t i) const { return typical_[std::min(i, ConfidenceModel::kPositions - 1)]; }

 private:
  StepCosts costs_;
  ConfidenceModel& model_;
  uint32_t deepest_;
  std::array<double, ConfidenceModel::kPositions> typical_{}, stated_{}, q_{};
  uint32_t limit_ = 0, made_ = 0, verify_ = 0, plain_steps_ = 0;
  bool decided_ = false;
};

}  // namespace b2host
