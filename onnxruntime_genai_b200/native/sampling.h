// Host-side logits processors and truncated categorical sampling.
//
// Semantics follow the reference's CPU path (src/sampling_distribution.h:26-79 for the penalties,
// :233-297 for the top-k -> temperature softmax -> top-p prefix -> renormalise pipeline, and
// src/speculative_sampling.h:39-177 for the speculative accept/correction math).  These routines
// are the oracle for the device sampler kernels and the production path for host-scored models.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <limits>
#include <numeric>
#include <random>
#include <stdexcept>
#include <vector>

namespace ogb {

constexpr float kLowestLogit = std::numeric_limits<float>::lowest();

// EOS cannot be produced while the sequence (length before this token) is shorter than min_length.
inline void ApplyMinLength(float* logits, int vocab, int current_length, int min_length,
                           const std::vector<int32_t>& eos_ids) {
  if (current_length >= min_length) return;
  for (int32_t e : eos_ids)
    if (e >= 0 && e < vocab) logits[e] = kLowestLogit;
}

// Each distinct token already in `prefix` is penalised once: negative scores are multiplied by
// the penalty, non-negative ones divided by it.
inline void ApplyRepetitionPenalty(float* logits, int vocab, const int32_t* prefix, size_t n, float penalty,
                                   std::vector<uint8_t>& seen) {
  if (penalty == 1.0f) return;
  if (seen.size() < size_t(vocab)) seen.assign(size_t(vocab), 0);
  for (size_t i = 0; i < n; ++i) {
    int32_t t = prefix[i];
    if (t < 0 || t >= vocab || seen[t]) continue;
    seen[t] = 1;
    float s = logits[t];
    logits[t] = s < 0 ? s * penalty : s / penalty;
  }
  for (size_t i = 0; i < n; ++i) {
    int32_t t = prefix[i];
    if (t >= 0 && t < vocab) seen[t] = 0;
  }
}

// Bans every token that would complete an n-gram that already occurs in `prefix`.
inline void ApplyNoRepeatNgram(float* logits, int vocab, const int32_t* prefix, size_t n, int ngram) {
  if (ngram <= 0 || n < size_t(ngram)) return;
  const size_t ctx = size_t(ngram - 1);
  const int32_t* tail = prefix + (n - ctx);
  for (size_t start = 0; start + size_t(ngram) <= n; ++start) {
    if (std::equal(tail, tail + ctx, prefix + start)) {
      int32_t banned = prefix[start + ctx];
      if (banned >= 0 && banned < vocab) logits[banned] = kLowestLogit;
    }
  }
}

inline void ApplyLogitsBitmask(float* logits, int vocab, const uint32_t* mask_words) {
  for (int v = 0; v < vocab; ++v)
    if (!((mask_words[v >> 5] >> (v & 31)) & 1u)) logits[v] = kLowestLogit;
}

inline int ArgMax(const float* logits, int vocab) {
  int best = 0;
  float bv = logits[0];
  for (int v = 1; v < vocab; ++v)
    if (logits[v] > bv) { bv = logits[v]; best = v; }
  return best;
}

// A sparse probability distribution: kept token ids (descending probability) and their
// renormalised probabilities (sum to one).
struct SparseDist {
  std::vector<int32_t> ids;
  std::vector<float> probs;
  float Prob(int32_t token) const {
    for (size_t i = 0; i < ids.size(); ++i)
      if (ids[i] == token) return probs[i];
    return 0.f;
  }
};

// top_k > 1 restricts to the k largest logits; 0 < top_p < 1 keeps the shortest prefix (by
// descending probability) whose cumulative probability reaches top_p; temperature divides logits.
// With neither filter active the full softmax is returned.
inline void BuildSampledDistribution(const float* logits, int vocab, int top_k, float top_p, float temperature,
                                     SparseDist& out, std::vector<int32_t>& scratch) {
  const float inv_t = 1.0f / temperature;
  const bool use_k = top_k > 1;
  const bool use_p = top_p > 0.f && top_p < 1.f;
  scratch.resize(size_t(vocab));
  std::iota(scratch.begin(), scratch.end(), 0);
  auto desc = [logits](int32_t a, int32_t b) { return logits[a] > logits[b]; };

  int m = use_k ? std::min(top_k, vocab) : vocab;
  if (use_k) {
    std::partial_sort(scratch.begin(), scratch.begin() + m, scratch.end(), desc);
  } else if (use_p) {
    // Exact nucleus over the whole vocabulary: grow a sorted prefix geometrically until its mass
    // (relative to the exact partition function) reaches top_p.
    float mx = *std::max_element(logits, logits + vocab);
    double z = 0;
    for (int v = 0; v < vocab; ++v) z += std::exp((logits[v] - mx) * inv_t);
    int sorted = 0, want = std::min(64, vocab);
    double cum = 0;
    int keep = vocab;
    while (true) {
      std::partial_sort(scratch.begin() + sorted, scratch.begin() + want, scratch.end(), desc);
      bool hit = false;
      for (int i = sorted; i < want; ++i) {
        cum += std::exp((logits[scratch[i]] - mx) * inv_t);
        if (cum >= double(top_p) * z) { keep = i + 1; hit = true; break; }
      }
      sorted = want;
      if (hit || want == vocab) break;
      want = std::min(want * 4, vocab);
    }
    m = keep;
  } else {
    std::sort(scratch.begin(), scratch.end(), desc);
  }

  const float mx = logits[scratch[0]];
  std::vector<float> p(static_cast<size_t>(m), 0.f);
  float sum = 0;
  for (int j = 0; j < m; ++j) { p[j] = std::exp((logits[scratch[j]] - mx) * inv_t); sum += p[j]; }
  if (sum > 0) for (auto& v : p) v /= sum;
  int keep = m;
  if (use_k && use_p) {
    float cum = 0;
    for (int j = 0; j < m; ++j) { cum += p[j]; if (cum >= top_p) { keep = j + 1; break; } }
  }
  float ks = 0;
  for (int j = 0; j < keep; ++j) ks += p[j];
  const float inv = ks > 0 ? 1.f / ks : 0.f;
  out.ids.assign(scratch.begin(), scratch.begin() + keep);
  out.probs.resize(size_t(keep));
  for (int j = 0; j < keep; ++j) out.probs[j] = p[j] * inv;
}

inline int32_t DrawFrom(const SparseDist& d, std::mt19937& rng) {
  if (d.ids.empty()) throw std::invalid_argument("cannot sample from an empty distribution");
  std::discrete_distribution<int> dist(d.probs.begin(), d.probs.end());
  return d.ids[size_t(dist(rng))];
}

inline void LogSoftmaxInPlace(float* x, int n) {
  float mx = *std::max_element(x, x + n);
  double s = 0;
  for (int i = 0; i < n; ++i) s += std::exp(double(x[i] - mx));
  float lse = mx + float(std::log(s));
  for (int i = 0; i < n; ++i) x[i] -= lse;
}

// ---------------------------------------------------------------------------- speculative math
// Probability of accepting a drafted token: min(1, p_target / p_draft); a token the draft could
// not have produced (p_draft == 0) is accepted only if the target gives it mass.
inline float AcceptProbability(float p_target, float p_draft) {
  if (p_draft <= 0.f) return p_target > 0.f ? 1.f : 0.f;
  return std::min(1.f, p_target / p_draft);
}

// Residual distribution max(0, p - q) renormalised; falls back to p when the residual is empty.
inline SparseDist CorrectionDistribution(const SparseDist& target, const SparseDist& draft) {
  SparseDist out;
  float sum = 0;
  for (size_t i = 0; i < target.ids.size(); ++i) {
    float r = target.probs[i] - draft.Prob(target.ids[i]);
    if (r > 0) { out.ids.push_back(target.ids[i]); out.probs.push_back(r); sum += r; }
  }
  if (sum <= 0) return target;
  for (auto& v : out.probs) v /= sum;
  return out;
}

}  // namespace ogb
