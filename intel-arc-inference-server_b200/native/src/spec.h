// Speculative-decoding control on the host: the sampler's filter, acceptance rules, and the
// policies that choose how many drafts to make.
//
// Behaviour follows the reference's server/spec_accept.h:16-118 (filter_probs, repetition
// penalty, greedy / lossless sampled / point-mass / sparse-q acceptance with the same RNG
// order), server/adaptive_k.h:15-134 (per-request K from an acceptance EMA and a cost table)
// and server/step_k.h:25-85 (per-step K from the draft head's calibrated confidence).
#pragma once
#include <algorithm>
#include <array>
#include <cmath>
#include <cstdint>
#include <numeric>
#include <random>
#include <stdexcept>
#include <vector>

namespace b2host {

struct Sampling {
  float temperature = 0.f;  // <= 0: greedy at the call site; inside the filter treated as 1
  uint32_t top_k = 0;       // 0: no cap
  float top_p = 1.f;
  float repetition_penalty = 1.f;
};

// Filtered distribution: ids in descending logit order, probs = softmax over the top-k at the
// temperature, cut after the first prefix whose mass reaches top_p, NOT renormalised.
struct FilteredProbs {
  std::vector<uint32_t> ids;
  std::vector<double> probs;
  double mass = 0.0;
  double prob(uint32_t id) const {
    for (size_t i = 0; i < ids.size(); ++i)
      if (ids[i] == id) return mass > 0 ? probs[i] / mass : 0.0;
    return 0.0;
  }
};

inline FilteredProbs filter_probs(const float* logits, uint32_t vocab_used, const Sampling& s) {
  FilteredProbs f;
  const uint32_t k = s.top_k == 0 ? vocab_used : std::min(s.top_k, vocab_used);
  std::vector<uint32_t> idx(vocab_used);
  std::iota(idx.begin(), idx.end(), 0u);
  auto cmp = [&](uint32_t a, uint32_t b) { return logits[a] > logits[b] || (logits[a] == logits[b] && a < b); };
  if (k < vocab_used) std::partial_sort(idx.begin(), idx.begin() + k, idx.end(), cmp);
  else std::sort(idx.begin(), idx.end(), cmp);
  idx.resize(k);
  const double t = s.temperature > 0.f ? s.temperature : 1.0;
  const double mx = logits[idx[0]];
  std::vector<double> p(k);
  double z = 0;
  for (uint32_t i = 0; i < k; ++i) {
    p[i] = std::exp((double(logits[idx[i]]) - mx) / t);
    z += p[i];
  }
  double cum = 0;
  for (uint32_t i = 0; i < k; ++i) {
    const double pi = p[i] / z;
    f.ids.push_back(idx[i]);
    f.probs.push_back(pi);
    cum += pi;
    if (cum >= s.top_p) break;
  }
  f.mass = cum;
  return f;
}

// HF's repetition penalty: l < 0 ? l * penalty : l / penalty, each listed id once.
inline void apply_repetition_penalty(float* logits, uint32_t vocab_used, const std::vector<uint32_t>& ids,
                                     float penalty) {
  if (penalty == 1.0f) return;
  std::vector<uint32_t> u(ids);
  std::sort(u.begin(), u.end());
  u.erase(std::unique(u.begin(), u.end()), u.end());
  for (uint32_t id : u) {
    if (id >= vocab_used) continue;
    float& l = logits[id];
    l = l < 0 ? l * penalty : l / penalty;
  }
}

// 53 random bits as a double in [0, 1): spelled out so that the device sampler (ops/csrc/sampler.cu) draws the
// same number from the same seed whatever the standard library does in generate_canonical.
inline double uniform01(std::mt19937_64& rng) { return (double)(rng() >> 11) * (1.0 / 9007199254740992.0); }

inline uint32_t draw(const FilteredProbs& f, std::mt19937_64& rng) {
  const double u = uniform01(rng) * f.mass;
  double c = 0;
  for (size_t i = 0; i < f.ids.size(); ++i) {
    c += f.probs[i];
    if (u < c) return f.ids[i];
  }
  return f.ids.back();
}

inline uint32_t argmax_low_tie(const float* logits, uint32_t n) {
  uint32_t b = 0;
  for (uint32_t i = 1; i < n; ++i)
    if (logits[i] > logits[b]) b = i;
  return b;
}

struct AcceptResult {
  uint32_t accepted;
  uint32_t next_token;
};

// Greedy: keep d_i while d_i == argmax p_{i-1}; next = argmax p_j.
inline AcceptResult accept_greedy(const uint32_t* verify_argmax, const uint32_t* drafts, uint32_t k) {
  uint32_t j = 0;
  while (j < k && drafts[j] == verify_argmax[j]) ++j;
  return {j, verify_argmax[j]};
}

// residual draw from normalise(max(0, p - q)); falls back to p when the residual is empty
template <class QProb>
inline uint32_t draw_residual(const FilteredProbs& p, QProb qprob, std::mt19937_64& rng) {
  std::vector<double> r(p.ids.size());
  double z = 0;
  for (size_t i = 0; i < p.ids.size(); ++i) {
    r[i] = std::max(0.0, p.probs[i] / p.mass - qprob(p.ids[i]));
    z += r[i];
  }
  if (z <= 0) return draw(p, rng);
  const double u = uniform01(rng) * z;
  double c = 0;
  for (size_t i = 0; i < r.size(); ++i) {
    c += r[i];
    if (u < c) return p.ids[i];
  }
  return p.ids.back();
}

// Lossless sampled acceptance (Leviathan et al. 2023).  One uniform per draft considered, in
// order, then exactly one draw for the correction or the bonus.
inline AcceptResult accept_sampled(const float* p_rows, const float* q_rows, const uint32_t* drafts, uint32_t k,
                                   uint32_t vocab_used, size_t row_stride, const Sampling& s, std::mt19937_64& rng) {
  for (uint32_t i = 0; i < k; ++i) {
    const FilteredProbs p = filter_probs(p_rows + i * row_stride, vocab_used, s);
    const FilteredProbs q = filter_probs(q_rows + i * row_stride, vocab_used, s);
    const double qd = q.prob(drafts[i]);
    if (qd <= 0) throw std::logic_error("accept_sampled: draft has zero probability under q");
    const double u = uniform01(rng);
    if (u < std::min(1.0, p.prob(drafts[i]) / qd)) continue;
    return {i, draw_residual(p, [&](uint32_t id) { return q.prob(id); }, rng)};
  }
  return {k, draw(filter_probs(p_rows + k * row_stride, vocab_used, s), rng)};
}

// Deterministic drafts (prompt lookup): q is a point mass on d_i.
inline AcceptResult accept_point_mass(const float* p_rows, const uint32_t* drafts, uint32_t k, uint32_t vocab_used,
                                      size_t row_stride, const Sampling& s, std::mt19937_64& rng) {
  for (uint32_t i = 0; i < k; ++i) {
    const FilteredProbs p = filter_probs(p_rows + i * row_stride, vocab_used, s);
    const double u = uniform01(rng);
    if (u < p.prob(drafts[i])) continue;
    const uint32_t d = drafts[i];
    return {i, draw_residual(p, [&](uint32_t id) { return id == d ? 1.0 : 0.0; }, rng)};
  }
  return {k, draw(filter_probs(p_rows + k * row_stride, vocab_used, s), rng)};
}

// Sparse q of a block drafter's row: softmax(scores / T) over at most 16 candidates.
struct SparseQ {
  static constexpr uint32_t kMax = 16;
  uint32_t n = 0;
  uint32_t ids[kMax] = {};
  double probs[kMax] = {};
  double prob(uint32_t id) const {
    for (uint32_t i = 0; i < n; ++i)
      if (ids[i] == id) return probs[i];
    return 0.0;
  }
};
inline SparseQ sparse_q(const uint32_t* cand, const float* scores, uint32_t n, float temperature) {
  SparseQ q;
  q.n = std::min(n, SparseQ::kMax);
  const double t = temperature > 0 ? temperature : 1.0;
  double mx = -INFINITY;
  for (uint32_t i = 0; i < q.n; ++i)
    if (std::isfinite(scores[i])) mx = std::max(mx, double(scores[i]));
  double z = 0;
  for (uint32_t i = 0; i < q.n; ++i) {
    q.ids[i] = cand[i];
    q.probs[i] = std::isfinite(scores[i]) ? std::exp((scores[i] - mx) / t) : 0.0;
    z += q.probs[i];
  }
  for (uint32_t i = 0; i < q.n; ++i) q.probs[i] = z > 0 ? q.probs[i] / z : 0.0;
  return q;
}
inline AcceptResult accept_sparse(const float* p_rows, const SparseQ* q, const uint32_t* drafts, uint32_t k,
                                  uint32_t vocab_used, size_t row_stride, const Sampling& s, std::mt19937_64& rng) {
  for (uint32_t i = 0; i < k; ++i) {
    const FilteredProbs p = filter_probs(p_rows + i * row_stride, vocab_used, s);
    const double qd = q[i].prob(drafts[i]);
    if (qd <= 0) throw std::logic_error("accept_sparse: draft has zero probability under q");
    const double u = uniform01(rng);
    if (u < std::min(1.0, p.prob(drafts[i]) / qd)) continue;
    const SparseQ& qi = q[i];
    return {i, draw_residual(p, [&](uint32_t id) { return qi.prob(id); }, rng)};
  }
  return {k, draw(filter_probs(p_rows + k * row_stride, vocab_used, s), rng)};
}

}  // namespace b2host
