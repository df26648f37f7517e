#include "search.h"

#include <cstring>
#include <stdexcept>

namespace ogb {

static bool IsEos(const SearchParams& p, int32_t t) {
  return std::find(p.eos_token_ids.begin(), p.eos_token_ids.end(), t) != p.eos_token_ids.end();
}

// ------------------------------------------------------------------------------------ Sequences
Sequences::Sequences(int batch_beam, int max_length)
    : rows_(batch_beam), max_length_(max_length), cur_(size_t(batch_beam) * max_length, 0) {}

void Sequences::AppendPrompt(const int32_t* ids, int batch, int len, int num_beams) {
  if (batch * num_beams != rows_) throw std::runtime_error("append_tokens: batch size does not match search batch_size");
  if (length_ + len > max_length_)
    throw std::runtime_error("append_tokens: sequence length " + std::to_string(length_ + len) +
                             " exceeds max_length " + std::to_string(max_length_));
  for (int b = 0; b < batch; ++b)
    for (int k = 0; k < num_beams; ++k)
      std::memcpy(Row(b * num_beams + k) + length_, ids + size_t(b) * len, size_t(len) * sizeof(int32_t));
  length_ += len;
}

void Sequences::AppendColumn(const int32_t* tokens) {
  if (length_ >= max_length_) throw std::runtime_error("sequence buffer is full");
  for (int r = 0; r < rows_; ++r) Row(r)[length_] = tokens[r];
  ++length_;
}

void Sequences::AppendBeamColumn(const int32_t* src_rows, const int32_t* tokens) {
  if (length_ >= max_length_) throw std::runtime_error("sequence buffer is full");
  if (alt_.size() != cur_.size()) alt_.assign(cur_.size(), 0);
  for (int r = 0; r < rows_; ++r) {
    int32_t* dst = alt_.data() + size_t(r) * max_length_;
    std::memcpy(dst, Row(src_rows[r]), size_t(length_) * sizeof(int32_t));
    dst[length_] = tokens[r];
  }
  cur_.swap(alt_);
  ++length_;
}

void Sequences::DropLast(int new_length) {
  if (new_length < 0 || new_length > length_) throw std::runtime_error("rewind_to: length out of range");
  length_ = new_length;
}

// ------------------------------------------------------------------------------------ BeamScorer
BeamScorer::BeamScorer(const SearchParams& p)
    : p_(p), per_batch_(size_t(p.batch_size)), next_scores_(size_t(p.BatchBeam()), 0.f),
      next_tokens_(size_t(p.BatchBeam()), 0), next_rows_(size_t(p.BatchBeam()), 0), open_batches_(p.batch_size) {
  // Only the first beam of each entry starts live so that identical beams do not all pick the same token.
  for (int b = 0; b < p.batch_size; ++b) {
    for (int k = 1; k < p.num_beams; ++k) next_scores_[size_t(b * p.num_beams + k)] = -1e9f;
    for (int k = 0; k < p.num_beams; ++k) next_rows_[size_t(b * p.num_beams + k)] = b * p.num_beams + k;
  }
}

void BeamScorer::AddHypothesis(PerBatch& pb, const int32_t* toks, int len, float sum_logprobs) {
  float score = sum_logprobs / std::pow(float(len), p_.length_penalty);
  if (int(pb.best.size()) == p_.num_beams && score <= pb.best.back().score) return;
  BeamHypothesis h{std::vector<int32_t>(toks, toks + len), score};
  auto pos = std::find_if(pb.best.begin(), pb.best.end(), [&](const BeamHypothesis& x) { return score > x.score; });
  pb.best.insert(pos, std::move(h));
  if (int(pb.best.size()) > p_.num_beams) pb.best.pop_back();
}

void BeamScorer::Process(const Sequences& seq, const float* cs, const int32_t* ct, const int32_t* cb) {
  const int nb = p_.num_beams, cand = 2 * nb, len = seq.Length();
  for (int b = 0; b < p_.batch_size; ++b) {
    PerBatch& pb = per_batch_[size_t(b)];
    if (pb.done) {
      for (int k = 0; k < nb; ++k) {
        next_scores_[size_t(b * nb + k)] = 0.f;
        next_tokens_[size_t(b * nb + k)] = p_.pad_token_id;
        next_rows_[size_t(b * nb + k)] = b * nb;
      }
      continue;
    }
    int filled = 0;
    for (int j = 0; j < cand && filled < nb; ++j) {
      int32_t tok = ct[b * cand + j];
      float sc = cs[b * cand + j];
      int row = b * nb + cb[b * cand + j];
      if (IsEos(p_, tok)) {
        if (j >= nb) continue;  // an EOS candidate ranked below the beam width is dropped
        AddHypothesis(pb, seq.Row(row), len, sc);
      } else {
        next_scores_[size_t(b * nb + filled)] = sc;
        next_tokens_[size_t(b * nb + filled)] = tok;
        next_rows_[size_t(b * nb + filled)] = row;
        ++filled;
      }
    }
    if (filled != nb) throw std::runtime_error("beam search: fewer than num_beams live candidates");
    if (int(pb.best.size()) < nb) continue;
    if (!p_.early_stopping) {
      float best = *std::max_element(cs + b * cand, cs + b * cand + cand);
      float attainable = best / std::pow(float(len), p_.length_penalty);
      if (pb.best.back().score < attainable) continue;
    }
    pb.done = true;
    --open_batches_;
  }
}

void BeamScorer::Finalize(const Sequences& seq) {
  if (finalized_) return;
  finalized_ = true;
  for (int b = 0; b < p_.batch_size; ++b) {
    PerBatch& pb = per_batch_[size_t(b)];
    if (pb.done) continue;
    for (int k = 0; k < p_.num_beams; ++k) {
      int row = b * p_.num_beams + k;
      AddHypothesis(pb, seq.Row(row), seq.Length(), next_scores_[size_t(row)]);
    }
  }
}

const BeamHypothesis& BeamScorer::Hypothesis(int b, int rank) const {
  auto& best = per_batch_.at(size_t(b)).best;
  if (rank < 0 || rank >= int(best.size())) throw std::out_of_range("beam hypothesis rank out of range");
  return best[size_t(rank)];
}

// ------------------------------------------------------------------------------------ Search
Search::Search(const SearchParams& p)
    : p_(p), seq_(p.BatchBeam(), p.max_length), next_tokens_(size_t(p.BatchBeam()), 0),
      eos_seen_(size_t(p.BatchBeam()), 0), open_count_(p.BatchBeam()) {
  if (p.random_seed >= 0) rng_.seed(uint32_t(p.random_seed));
  else { std::random_device rd; rng_.seed(rd()); }
}

void Search::AppendTokens(const int32_t* ids, int batch, int len) {
  seq_.AppendPrompt(ids, batch, len, p_.num_beams);
  if (seq_.Length() >= p_.max_length) done_ = true;
}

void Search::RewindTo(int length) {
  seq_.DropLast(length);
  done_ = false;
  std::fill(eos_seen_.begin(), eos_seen_.end(), 0);
  open_count_ = p_.BatchBeam();
}

void Search::ApplyMinLength() {
  for (int r = 0; r < p_.BatchBeam(); ++r)
    ogb::ApplyMinLength(logits_ + size_t(r) * p_.vocab_size, p_.vocab_size, seq_.Length(), p_.min_length, p_.eos_token_ids);
}
void Search::ApplyRepetitionPenalty() {
  for (int r = 0; r < p_.BatchBeam(); ++r)
    ogb::ApplyRepetitionPenalty(logits_ + size_t(r) * p_.vocab_size, p_.vocab_size, seq_.Row(r), size_t(seq_.Length()),
                                p_.repetition_penalty, seen_scratch_);
}
void Search::ApplyNoRepeatNgram() {
  for (int r = 0; r < p_.BatchBeam(); ++r)
    ogb::ApplyNoRepeatNgram(logits_ + size_t(r) * p_.vocab_size, p_.vocab_size, seq_.Row(r), size_t(seq_.Length()),
                            p_.no_repeat_ngram_size);
}

void Search::FinishStep() {
  seq_.AppendColumn(next_tokens_.data());
  if (seq_.Length() >= p_.max_length) done_ = true;
}

void Search::CommitTokens(const int32_t* tokens) {
  for (int r = 0; r < p_.BatchBeam(); ++r) {
    if (eos_seen_[size_t(r)]) { next_tokens_[size_t(r)] = p_.pad_token_id; continue; }
    next_tokens_[size_t(r)] = tokens[r];
    if (IsEos(p_, tokens[r])) {
      eos_seen_[size_t(r)] = 1;
      if (--open_count_ == 0) done_ = true;
    }
  }
  FinishStep();
}

void Search::SelectTop() {
  if (!logits_) throw std::runtime_error("no logits set");
  std::vector<int32_t> picks(size_t(p_.BatchBeam()));
  for (int r = 0; r < p_.BatchBeam(); ++r)
    picks[size_t(r)] = eos_seen_[size_t(r)] ? p_.pad_token_id : ArgMax(logits_ + size_t(r) * p_.vocab_size, p_.vocab_size);
  CommitTokens(picks.data());
}

void Search::Sample(int k, float p, float t) {
  if (!logits_) throw std::runtime_error("no logits set");
  std::vector<int32_t> picks(size_t(p_.BatchBeam()));
  SparseDist d;
  for (int r = 0; r < p_.BatchBeam(); ++r) {
    if (eos_seen_[size_t(r)]) { picks[size_t(r)] = p_.pad_token_id; continue; }
    BuildSampledDistribution(logits_ + size_t(r) * p_.vocab_size, p_.vocab_size, k, p, t, d, idx_scratch_);
    picks[size_t(r)] = DrawFrom(d, rng_);
  }
  CommitTokens(picks.data());
}
void Search::SampleTopK(int k, float t) { Sample(k, 0.f, t); }
void Search::SampleTopP(float p, float t) { Sample(0, p, t); }
void Search::SampleTopKTopP(int k, float p, float t) { Sample(k, p, t); }

SearchCheckpoint Search::Save() const {
  return SearchCheckpoint{seq_.Length(), done_, open_count_, eos_seen_, next_tokens_, rng_};
}
void Search::Restore(const SearchCheckpoint& c) {
  seq_.DropLast(c.length);
  done_ = c.done;
  open_count_ = c.open_count;
  eos_seen_ = c.eos_seen;
  next_tokens_ = c.next_tokens;
  rng_ = c.rng;
}

// ------------------------------------------------------------------------------------ BeamSearch
BeamSearch::BeamSearch(const SearchParams& p) : Search(p), scorer_(p) {
  if (p.vocab_size < 2) throw std::runtime_error("beam search requires vocab_size >= 2");
}

void BeamSearch::CommitBeamStep(const float* cs, const int32_t* ct, const int32_t* cb) {
  scorer_.Process(seq_, cs, ct, cb);
  next_tokens_ = scorer_.NextTokens();
  seq_.AppendBeamColumn(scorer_.NextRows().data(), next_tokens_.data());
  if (scorer_.Done() || seq_.Length() >= p_.max_length) done_ = true;
}

void BeamSearch::SelectTop() {
  if (!logits_) throw std::runtime_error("no logits set");
  const int nb = p_.num_beams, V = p_.vocab_size, cand = 2 * nb;
  const auto& running = scorer_.NextScores();
  for (int r = 0; r < p_.BatchBeam(); ++r) {
    float* row = logits_ + size_t(r) * V;
    LogSoftmaxInPlace(row, V);
    float add = running[size_t(r)];
    for (int v = 0; v < V; ++v) row[v] += add;
  }
  std::vector<float> cs(size_t(p_.batch_size) * cand);
  std::vector<int32_t> ct(cs.size()), cb(cs.size());
  order_.resize(size_t(nb) * V);
  for (int b = 0; b < p_.batch_size; ++b) {
    const float* base = logits_ + size_t(b) * nb * V;
    std::iota(order_.begin(), order_.end(), 0);
    std::partial_sort(order_.begin(), order_.begin() + cand, order_.end(),
                      [base](int32_t x, int32_t y) { return base[x] > base[y]; });
    for (int j = 0; j < cand; ++j) {
      cs[size_t(b * cand + j)] = base[order_[size_t(j)]];
      cb[size_t(b * cand + j)] = order_[size_t(j)] / V;
      ct[size_t(b * cand + j)] = order_[size_t(j)] % V;
    }
  }
  CommitBeamStep(cs.data(), ct.data(), cb.data());
}

void BeamSearch::CommitBeamResult(const int32_t* tokens, const int32_t* rows, bool all_done) {
  device_scored_ = true;
  next_tokens_.assign(tokens, tokens + p_.BatchBeam());
  device_rows_.assign(rows, rows + p_.BatchBeam());
  for (int r = 0; r < p_.BatchBeam(); ++r)
    if (device_rows_[size_t(r)] < 0 || device_rows_[size_t(r)] >= p_.BatchBeam()) throw std::runtime_error("beam source row out of range");
  seq_.AppendBeamColumn(device_rows_.data(), next_tokens_.data());
  if (all_done || seq_.Length() >= p_.max_length) done_ = true;
}

void BeamSearch::SetHypothesis(int batch, int rank, const int32_t* tokens, int len, float score) {
  if (batch < 0 || batch >= p_.batch_size || rank < 0 || rank >= p_.num_beams || len < 0 || len > p_.max_length)
    throw std::out_of_range("beam hypothesis index out of range");
  device_scored_ = true;
  if (device_hyps_.empty()) device_hyps_.resize(size_t(p_.batch_size));
  auto& list = device_hyps_[size_t(batch)];
  if (int(list.size()) <= rank) list.resize(size_t(rank) + 1);
  list[size_t(rank)] = BeamHypothesis{std::vector<int32_t>(tokens, tokens + len), score};
}

const BeamHypothesis& BeamSearch::Hypothesis(int batch, int rank) const {
  if (!device_scored_) return scorer_.Hypothesis(batch, rank);
  if (batch < 0 || batch >= int(device_hyps_.size()) || rank < 0 || rank >= int(device_hyps_[size_t(batch)].size()))
    throw std::out_of_range("beam hypothesis rank out of range");
  return device_hyps_[size_t(batch)][size_t(rank)];
}

void BeamSearch::Finalize() {
  if (finalized_) return;
  finalized_ = true;
  if (!device_scored_) scorer_.Finalize(seq_);   // the device scorer ranks its own hypotheses (SetHypothesis)
}

std::unique_ptr<Search> MakeSearch(const SearchParams& p) {
  if (p.num_beams > 1) return std::make_unique<BeamSearch>(p);
  return std::make_unique<Search>(p);
}

}  // namespace ogb
