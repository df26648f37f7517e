// Speculative decoding building blocks that live on the host: the n-gram proposer index, the
// adaptive proposal-width controller, the zero-accept cooldown, round statistics and the
// accept / correct / bonus verification loop.
//
// Behavioural references: src/n_gram_lookup.h:23-108 (latest occurrence of the last N-1 tokens,
// optional chained lookup), src/speculative_decoding_strategy.h:31-197 (EWMA alpha 0.25,
// acceptance thresholds 0.75 / 0.50, K <= 16, adjacent-width probes), :199-245 (three
// zero-accept rounds -> one plain step), src/speculative_sampling.h:39-177 (accept with
// probability min(1, p_t/p_d); on the first rejection sample from max(0, p_t - p_d)
// renormalised; when everything is accepted take a bonus token from the last target row),
// src/speculative_stats.h:11-68.
#pragma once
#include <array>
#include <cmath>
#include <cstdint>
#include <random>
#include <unordered_map>
#include <vector>

#include "sampling.h"

namespace ogb {

// Index from (N-1)-token contexts to the most recent position where that context was followed
// by another token.  Keys are 64-bit FNV-1a hashes; a hit is verified against the history so a
// collision can only cause a miss, never a wrong proposal.
class NGramIndex {
 public:
  explicit NGramIndex(int ngram_size) : n_(ngram_size), ctx_(size_t(ngram_size - 1)) {
    if (ngram_size < 2) throw std::runtime_error("n-gram lookup requires ngram_size >= 2");
  }
  int NGramSize() const { return n_; }
  size_t HistorySize() const { return hist_.size(); }
  uint64_t Hits() const { return hits_; }
  uint64_t Misses() const { return misses_; }

  void Append(const int32_t* toks, size_t n) {
    for (size_t i = 0; i < n; ++i) {
      hist_.push_back(toks[i]);
      if (hist_.size() > ctx_) {
        size_t start = hist_.size() - ctx_ - 1;  // context [start, start+ctx) is followed by the new token
        latest_[HashAt(hist_.data() + start)] = start;
      }
    }
  }
  void Reset(const int32_t* toks = nullptr, size_t n = 0) {
    hist_.clear();
    latest_.clear();
    if (n) Append(toks, n);
  }

  std::vector<int32_t> Propose(size_t max_tokens, bool chained) {
    std::vector<int32_t> out;
    if (max_tokens == 0 || hist_.size() < ctx_) return out;
    std::vector<int32_t> ctx(hist_.end() - ptrdiff_t(ctx_), hist_.end());
    long pos = Find(ctx.data());
    if (pos < 0) { ++misses_; return out; }
    ++hits_;
    if (!chained) {
      size_t cont = size_t(pos) + ctx_;
      size_t cnt = std::min(max_tokens, hist_.size() - cont);
      out.assign(hist_.begin() + ptrdiff_t(cont), hist_.begin() + ptrdiff_t(cont + cnt));
      return out;
    }
    while (pos >= 0 && out.size() < max_tokens) {
      int32_t t = hist_[size_t(pos) + ctx_];
      out.push_back(t);
      ctx.erase(ctx.begin());
      ctx.push_back(t);
      pos = Find(ctx.data());
    }
    return out;
  }

 private:
  uint64_t HashAt(const int32_t* p) const {
    uint64_t h = 1469598103934665603ull;
    for (size_t i = 0; i < ctx_; ++i) { h ^= uint32_t(p[i]); h *= 1099511628211ull; }
    return h;
  }
  long Find(const int32_t* ctx) const {
    auto it = latest_.find(HashAt(ctx));
    if (it == latest_.end()) return -1;
    if (!std::equal(ctx, ctx + ctx_, hist_.begin() + ptrdiff_t(it->second))) return -1;
    return long(it->second);
  }
  int n_;
  size_t ctx_;
  std::vector<int32_t> hist_;
  std::unordered_map<uint64_t, size_t> latest_;
  uint64_t hits_{0}, misses_{0};
};

// Picks the number of drafted tokens per round.  Disabled (fixed K) unless min_adaptive_k > 0.
class AdaptiveK {
 public:
  static constexpr int kMaxK = 16;
  AdaptiveK(int fixed_k, int min_adaptive_k)
      : lo_(min_adaptive_k > 0 ? min_adaptive_k : fixed_k), hi_(min_adaptive_k > 0 ? kMaxK : fixed_k),
        on_(min_adaptive_k > 0), k_(lo_) {}
  int K() const { return k_; }
  int MinK() const { return lo_; }
  uint64_t Increases() const { return ups_; }
  uint64_t Decreases() const { return downs_; }
  uint64_t Probes() const { return probes_; }

  void Record(int k, int evaluated, int accepted, size_t committed, bool budget_filled, float ms) {
    if (!on_ || k != k_ || evaluated <= 0 || committed == 0 || !budget_filled || !(ms > 0) || !std::isfinite(ms)) return;
    Est& e = est_[size_t(k)];
    e.Add(float(committed), ms, float(accepted) / float(evaluated));
    if (origin_) {  // a probe is running
      ++probe_obs_;
      const Est& o = est_[size_t(origin_)];
      const bool up = k_ > origin_;
      if (o.Rate() > 0 && e.Rate() < o.Rate() * 0.80f) { EndProbe(false); return; }
      if (probe_obs_ >= 2) {
        bool rate_ok = o.Rate() <= 0 || e.Rate() >= o.Rate() * 0.97f;
        bool acc_ok = !up || e.acc >= 0.75f;
        EndProbe(rate_ok && acc_ok);
      }
      return;
    }
    ++stable_;
    if (wait_ > 0) { --wait_; return; }
    if (e.n < 2) return;
    if (e.acc < 0.50f && k_ > lo_) BeginProbe(k_ - 1);
    else if (e.acc >= 0.75f && k_ < hi_ && stable_ >= 2) BeginProbe(k_ + 1);
  }
  void Reset() { k_ = lo_; est_ = {}; origin_ = 0; probe_obs_ = stable_ = wait_ = 0; }

 private:
  struct Est {
    float tok{}, ms{}, acc{};
    size_t n{};
    void Add(float t, float m, float a) {
      if (n == 0) { tok = t; ms = m; acc = a; }
      else { tok += 0.25f * (t - tok); ms += 0.25f * (m - ms); acc += 0.25f * (a - acc); }
      ++n;
    }
    float Rate() const { return ms > 0 ? tok / ms : 0.f; }
  };
  void Move(int k) { if (k > k_) ++ups_; else if (k < k_) ++downs_; k_ = k; }
  void BeginProbe(int k) { origin_ = k_; probe_obs_ = 0; stable_ = 0; ++probes_; Move(k); }
  void EndProbe(bool keep) { if (!keep) Move(origin_); origin_ = 0; probe_obs_ = 0; stable_ = 0; wait_ = keep ? 1 : 6; }
  int lo_, hi_;
  bool on_;
  int k_;
  std::array<Est, kMaxK + 1> est_{};
  int origin_{0}, probe_obs_{0}, stable_{0}, wait_{0};
  uint64_t ups_{0}, downs_{0}, probes_{0};
};

// After three consecutive rounds that accepted nothing, one round is skipped (plain decoding).
class ZeroAcceptCooldown {
 public:
  explicit ZeroAcceptCooldown(bool enabled) : on_(enabled) {}
  bool ShouldSkipRound() {
    if (!on_ || streak_ < 3) return false;
    streak_ = 0;
    ++skips_;
    return true;
  }
  void Record(int evaluated, int accepted) {
    if (evaluated <= 0) return;
    streak_ = accepted == 0 ? streak_ + 1 : 0;
  }
  uint64_t Skips() const { return skips_; }

 private:
  bool on_;
  int streak_{0};
  uint64_t skips_{0};
};

struct SpeculativeStats {
  uint64_t rounds{}, proposed{}, evaluated{}, accepted{}, committed{}, bonus{}, corrections{}, standard_steps{},
      cooldown_skips{}, empty_proposals{};
  double propose_ms{}, verify_ms{};
  int effective_k{};
  double AcceptanceRate() const { return evaluated ? double(accepted) / double(evaluated) : 0.0; }
  double TokensPerRound() const { return rounds ? double(committed) / double(rounds) : 0.0; }
};

struct VerifyResult {
  int accepted{};                 // number of drafted tokens kept
  std::vector<int32_t> commit;    // accepted draft tokens followed by the correction or bonus token
  bool bonus{};
};

// Greedy verification: drafted token i is kept while it equals argmax of target row i; the first
// mismatch is replaced by the target's argmax; if all K match, row K supplies a bonus token.
// target_logits: [K+1, vocab].
inline VerifyResult VerifyGreedy(const int32_t* draft, int k, const float* target_logits, int vocab) {
  VerifyResult r;
  for (int i = 0; i < k; ++i) {
    int32_t t = ArgMax(target_logits + size_t(i) * vocab, vocab);
    if (t != draft[i]) { r.accepted = i; r.commit.push_back(t); return r; }
    r.commit.push_back(draft[i]);
  }
  r.accepted = k;
  r.bonus = true;
  r.commit.push_back(ArgMax(target_logits + size_t(k) * vocab, vocab));
  return r;
}

// Sampled verification. draft_dists[i] is the distribution drafted token i was drawn from (a
// one-hot distribution for deterministic proposers such as n-gram lookup); target_dists has K+1
// entries built with the same truncation parameters.
inline VerifyResult VerifySampled(const int32_t* draft, int k, const std::vector<SparseDist>& draft_dists,
                                  const std::vector<SparseDist>& target_dists, std::mt19937& rng) {
  VerifyResult r;
  std::uniform_real_distribution<float> uni(0.f, 1.f);
  for (int i = 0; i < k; ++i) {
    float pt = target_dists[size_t(i)].Prob(draft[i]);
    float pd = draft_dists[size_t(i)].Prob(draft[i]);
    if (uni(rng) < AcceptProbability(pt, pd)) { r.commit.push_back(draft[i]); continue; }
    r.accepted = i;
    r.commit.push_back(DrawFrom(CorrectionDistribution(target_dists[size_t(i)], draft_dists[size_t(i)]), rng));
    return r;
  }
  r.accepted = k;
  r.bonus = true;
  r.commit.push_back(DrawFrom(target_dists[size_t(k)], rng));
  return r;
}

}  // namespace ogb
